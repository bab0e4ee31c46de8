"""Causal GQA flash prefill with the sigmoid-gate epilogue, head_dim 256, on B200.

Mirrors the operator boundary of the reference's
``src/moespresso/runtime/qwen/full_attention.py``: the kernel call
``mlx_kquant.sdpa_fa_prefill_q8(queries, *past_k, *past_v, self_k, self_v, scale, ...)``
(:372-382) and the wrapper ``FlashPrefillD256Attention`` (:168-397) that routes an
eligible chunk to it and multiplies the result by ``sigmoid(gate)`` (:396-397).
Keys / values are dense 16-bit tensors here (past ++ self already concatenated).
"""
from __future__ import annotations

import ctypes as C

import torch

from .. import _abi
from .. import _torchabi as _t
from .._torchabi import dtype_code, last_dim_contiguous, ptr, require_cuda, status_word, stream_ptr, workspace

FLASH_HEAD_DIM = 256


def sdpa_fa_prefill(queries, keys, values, scale: float, *, gate=None, layout: str = "bhld", check: bool = False):
    """softmax(scale * Q K^T + causal) V [* sigmoid(gate)].

    layout "bhld": queries [1,Hq,L,D], keys / values [1,Hkv,P+L,D], gate [1,L,Hq*D] or
    [1,L,Hq,D]; returns [1,L,Hq*D] (the wrapper's ``out.transpose(0,2,1,3).reshape``).
    layout "lhd": queries [L,Hq,D], keys / values [P+L,Hkv,D], gate [L,Hq,D]; returns
    [L,Hq,D].  The first P = len(keys) - L keys are the past and are visible to every
    query; key P+j is visible to query i iff j <= i.
    """
    dev = require_cuda(queries, keys, values)
    lib = _abi.load()
    if layout == "bhld":
        if queries.ndim != 4 or int(queries.shape[0]) != 1:
            raise ValueError("flash prefill requires batch 1 [1, heads, tokens, head_dim] tensors")
        q = queries[0].permute(1, 0, 2)
        k = keys[0].permute(1, 0, 2)
        v = values[0].permute(1, 0, 2)
        g = None
        if gate is not None:
            g = gate.reshape(int(queries.shape[2]), int(queries.shape[1]), int(queries.shape[3]))
    elif layout == "lhd":
        q, k, v, g = queries, keys, values, gate
    else:
        raise ValueError("layout must be 'bhld' or 'lhd'")
    S, Hq, D = (int(x) for x in q.shape)
    Skv, Hkv = int(k.shape[0]), int(k.shape[1])
    if D != FLASH_HEAD_DIM:
        raise ValueError("flash prefill requires head_dim=256")
    if q.dtype not in (torch.bfloat16, torch.float16) or k.dtype != q.dtype or v.dtype != q.dtype:
        raise ValueError("flash prefill requires bfloat16 or float16 queries, keys and values of one dtype")
    if g is not None and g.dtype != q.dtype:
        g = g.to(q.dtype)
    q, k, v = last_dim_contiguous(q), last_dim_contiguous(k), last_dim_contiguous(v)
    if g is not None:
        g = last_dim_contiguous(g)
    out = torch.empty((S, Hq, D), dtype=q.dtype, device=dev)
    a = _abi.FlashPrefillArgs()
    a.q = ptr(q); a.q_stride_s, a.q_stride_h = q.stride(0), q.stride(1)
    a.k = ptr(k); a.k_stride_s, a.k_stride_h = k.stride(0), k.stride(1)
    a.v = ptr(v); a.v_stride_s, a.v_stride_h = v.stride(0), v.stride(1)
    a.gate = ptr(g)
    if g is not None:
        a.gate_stride_s, a.gate_stride_h = g.stride(0), g.stride(1)
    a.out = ptr(out); a.out_stride_s, a.out_stride_h = out.stride(0), out.stride(1)
    a.dtype = dtype_code(q)
    a.S, a.Skv, a.Hq, a.Hkv, a.D = S, Skv, Hq, Hkv, D
    a.scale = float(scale)
    ws = workspace(lib.mxb_flash_prefill_workspace_bytes(C.byref(a)), dev)
    a.workspace = ptr(ws); a.workspace_bytes = 0 if ws is None else ws.numel()
    status = status_word(dev) if check else None
    a.status = ptr(status)
    _abi.check(_t.launch("flash_prefill", lib.mxb_flash_prefill, a))
    if check and int(status.item()) != 0:
        raise _abi.MxbError("flash prefill: a device-side wait timed out")
    if layout == "bhld":
        return out.reshape(1, S, Hq * D)
    return out


class FlashPrefillD256Attention(torch.nn.Module):
    """Wrapper with the call shape of the reference's ``FlashPrefillD256Attention``
    (qwen/full_attention.py:168-397): ``inner`` owns ``q_proj`` (producing queries and
    gate interleaved per head), ``k_proj``, ``v_proj``, ``o_proj``, ``q_norm``, ``k_norm``
    and ``rope(x, offset)``; attributes ``num_attention_heads``, ``num_key_value_heads``,
    ``head_dim``, ``scale``.  A chunk is eligible when batch == 1, tokens > 1,
    mask == "causal" and head_dim == 256; anything else raises (this build keeps no
    fallback route), after counting the reason like the reference's fallback counters.
    ``cache`` is a dict holding dense 16-bit ``keys`` / ``values`` [1,Hkv,P,D] and
    ``offset``; it is updated in place (append)."""

    def __init__(self, inner):
        super().__init__()
        self.inner = inner
        self.flash_calls = 0
        self.rejected = {"batch": 0, "single_token": 0, "mask": 0, "head_dim": 0}

    def eligible(self, x, mask) -> bool:
        B, L, _ = x.shape
        if B != 1:
            self.rejected["batch"] += 1
            return False
        if L <= 1:
            self.rejected["single_token"] += 1
            return False
        if mask != "causal":
            self.rejected["mask"] += 1
            return False
        if int(self.inner.head_dim) != FLASH_HEAD_DIM:
            self.rejected["head_dim"] += 1
            return False
        return True

    def forward(self, x, mask=None, cache=None):
        if not self.eligible(x, mask):
            raise ValueError("flash prefill route is not eligible for this call (batch 1, tokens > 1, "
                             "mask='causal', head_dim=256 required)")
        inner = self.inner
        B, L, _ = x.shape
        Hq, Hkv, D = int(inner.num_attention_heads), int(inner.num_key_value_heads), int(inner.head_dim)
        qg = inner.q_proj(x).reshape(B, L, Hq, 2 * D)
        queries, gate = qg[..., :D], qg[..., D:]
        keys = inner.k_proj(x).reshape(B, L, Hkv, D)
        values = inner.v_proj(x).reshape(B, L, Hkv, D)
        queries = inner.q_norm(queries).transpose(1, 2)
        keys = inner.k_norm(keys).transpose(1, 2)
        values = values.transpose(1, 2)
        offset = 0 if cache is None else int(cache.get("offset", 0))
        queries = inner.rope(queries, offset)
        keys = inner.rope(keys, offset)
        if cache is not None:
            if cache.get("keys") is not None:
                keys = torch.cat([cache["keys"], keys], dim=2)
                values = torch.cat([cache["values"], values], dim=2)
            cache["keys"], cache["values"], cache["offset"] = keys, values, offset + L
        self.flash_calls += 1
        out = sdpa_fa_prefill(queries, keys, values, float(inner.scale), gate=gate.reshape(B, L, Hq * D))
        return inner.o_proj(out)


def install_flash_prefill_attention(model) -> int:
    """Wrap every layer's ``self_attn`` whose head_dim is 256
    (reference: qwen/full_attention.py:425-442).  Returns the number wrapped."""
    n = 0
    for layer in getattr(model, "layers", []):
        attn = getattr(layer, "self_attn", None)
        if attn is None or isinstance(attn, FlashPrefillD256Attention):
            continue
        if int(getattr(attn, "head_dim", 0)) == FLASH_HEAD_DIM:
            layer.self_attn = FlashPrefillD256Attention(attn)
            n += 1
    return n


def flash_prefill_attention_stats(model) -> dict:
    """Aggregated counters (reference: qwen/full_attention.py:445-470)."""
    stats = {"layers": 0, "flash_calls": 0, "rejected": {"batch": 0, "single_token": 0, "mask": 0, "head_dim": 0}}
    for layer in getattr(model, "layers", []):
        attn = getattr(layer, "self_attn", None)
        if isinstance(attn, FlashPrefillD256Attention):
            stats["layers"] += 1
            stats["flash_calls"] += attn.flash_calls
            for key, val in attn.rejected.items():
                stats["rejected"][key] += val
    return stats
