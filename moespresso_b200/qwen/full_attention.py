"""Causal GQA flash prefill with the sigmoid-gate epilogue, head_dim 256, on B200.

Mirrors the operator boundary of the reference's
``src/moespresso/runtime/qwen/full_attention.py``: the kernel call
``mlx_kquant.sdpa_fa_prefill_q8(queries, *past_k, *past_v, self_k, self_v, scale, ...)``
(:372-382) and the wrapper ``FlashPrefillD256Attention`` (:168-397) that routes an
eligible chunk to it and multiplies the result by ``sigmoid(gate)`` (:396-397).
``sdpa_fa_prefill`` takes dense 16-bit keys / values (past ++ self already concatenated: the form benchmark
configuration 2 runs); ``sdpa_fa_prefill_q8`` and ``sdpa_decode_q8`` take the served form, a past held in the
affine 8-bit format (group 64) of ``QuantizedKVCache``.
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


Q8_GROUP, Q8_BITS = 64, 8
DECODE_Q8_MIN_KEYS = 32768   # the reference routes decode to its q8 kernel from this context on (full_attention.py:76)


def quantize_affine_q8(x):
    """``mx.quantize(x, group_size=64, bits=8)``: x ``[..., D]`` (float32 / float16 / bfloat16, D a multiple of 64)
    -> (packed uint32 ``[..., D / 4]``, scales ``[..., D / 64]``, biases ``[..., D / 64]``)."""
    dev = require_cuda(x)
    D = int(x.shape[-1])
    if D % Q8_GROUP:
        raise ValueError("the last dimension must be a multiple of the group size 64")
    if x.dtype not in (torch.float32, torch.float16, torch.bfloat16):
        raise ValueError("rows must be float32, float16, or bfloat16")
    rows = x.reshape(-1, D).contiguous()
    n = int(rows.shape[0])
    packed = torch.empty((n, D // 4), dtype=torch.int32, device=dev)
    scales = torch.empty((n, D // Q8_GROUP), dtype=x.dtype, device=dev)
    biases = torch.empty_like(scales)
    if n:
        _q8_call("affine_q8_quantize", rows, D, packed, scales, biases, n, D)
    lead = tuple(x.shape[:-1])
    return packed.reshape(*lead, D // 4), scales.reshape(*lead, D // Q8_GROUP), biases.reshape(*lead, D // Q8_GROUP)


def dequantize_affine_q8(packed, scales, biases, *, dtype=None, out=None):
    """``mx.dequantize(packed, scales, biases, group_size=64, bits=8)`` -> ``[..., D]`` of ``dtype`` (default: the
    scales' type).  ``out``: a ``[n, D]`` view with unit feature stride to write into (its row stride is honoured)."""
    dev = require_cuda(packed, scales, biases)
    D = int(packed.shape[-1]) * 4
    n = int(packed.numel() // (D // 4))
    lead = tuple(packed.shape[:-1])
    if out is None:
        out = torch.empty((n, D), dtype=dtype or scales.dtype, device=dev)
        ret = out.reshape(*lead, D)
    else:
        if out.ndim != 2 or tuple(out.shape) != (n, D) or out.stride(1) != 1:
            raise ValueError("out must be [rows, D] with unit feature stride")
        ret = out
    if n:
        _q8_call("affine_q8_dequantize", out, int(out.stride(0)), packed.reshape(n, D // 4).contiguous(),
                 scales.reshape(n, -1).contiguous(), biases.reshape(n, -1).contiguous(), n, D)
    return ret


def _q8_call(name, rows, row_stride, packed, scales, biases, n, D):
    a = _abi.AffineQ8Args()
    a.x, a.x_dtype, a.x_row_stride = ptr(rows), dtype_code(rows), int(row_stride)
    a.packed, a.scales, a.biases, a.sb_dtype = ptr(packed), ptr(scales), ptr(biases), dtype_code(scales)
    a.n_rows, a.width = n, D
    _abi.check(_t.launch(name, getattr(_abi.load(), "mxb_" + name), a))


class QuantizedKVCache:
    """Pre-allocated affine-q8 KV cache with the surface of mlx-lm's ``QuantizedKVCache`` that the reference relies
    on (qwen/full_attention.py:200-236, 313-382): ``bits`` 8, ``group_size`` 64, ``offset``, ``keys`` / ``values``
    as (packed, scales, biases) of ``[1, Hkv, capacity, ...]``, ``state`` (views of the valid prefix) and
    ``update_and_fetch`` (quantise the new rows in place behind the prefix)."""

    bits, group_size = Q8_BITS, Q8_GROUP

    def __init__(self, n_kv_heads: int, head_dim: int, capacity: int, *, dtype=torch.bfloat16, device="cuda"):
        self.offset, self.capacity = 0, int(capacity)
        mk = lambda w, dt: torch.zeros((1, n_kv_heads, self.capacity, w), dtype=dt, device=device)
        self.keys = (mk(head_dim // 4, torch.int32), mk(head_dim // Q8_GROUP, dtype), mk(head_dim // Q8_GROUP, dtype))
        self.values = (mk(head_dim // 4, torch.int32), mk(head_dim // Q8_GROUP, dtype), mk(head_dim // Q8_GROUP, dtype))

    def _prefix(self, n):
        return tuple(t[:, :, :n] for t in self.keys), tuple(t[:, :, :n] for t in self.values)

    @property
    def state(self):
        return self._prefix(self.offset)

    def update_and_fetch(self, keys, values):
        """keys / values ``[1, Hkv, L, D]``: quantised into rows ``offset .. offset + L``; returns the quantised
        prefix including them."""
        L = int(keys.shape[2])
        if self.offset + L > self.capacity:
            raise ValueError("QuantizedKVCache capacity exceeded")
        for store, x in ((self.keys, keys), (self.values, values)):
            q = quantize_affine_q8(x.to(store[1].dtype))
            for dst, src in zip(store, q):
                dst[:, :, self.offset:self.offset + L].copy_(src)
        self.offset += L
        return self._prefix(self.offset)


class DenseKVCache:
    """Pre-allocated dense 16-bit KV cache for the dense flash route (appends in place, no re-copy of the past)."""

    def __init__(self, n_kv_heads: int, head_dim: int, capacity: int, *, dtype=torch.bfloat16, device="cuda"):
        self.offset, self.capacity = 0, int(capacity)
        self.keys = torch.zeros((1, n_kv_heads, self.capacity, head_dim), dtype=dtype, device=device)
        self.values = torch.zeros_like(self.keys)

    def update_and_fetch(self, keys, values):
        L = int(keys.shape[2])
        if self.offset + L > self.capacity:
            raise ValueError("DenseKVCache capacity exceeded")
        self.keys[:, :, self.offset:self.offset + L].copy_(keys)
        self.values[:, :, self.offset:self.offset + L].copy_(values)
        self.offset += L
        return self.keys[:, :, :self.offset], self.values[:, :, :self.offset]


def sdpa_fa_prefill_q8(queries, k_packed, k_scales, k_biases, v_packed, v_scales, v_biases, self_k, self_v, scale, *,
                       bq: int = 64, bk: int = 16, stage: int = 2, gate=None, check: bool = False):
    """Causal attention of a chunk over (affine-q8 past ++ self chunk) — the call the reference makes at
    qwen/full_attention.py:372-382.  queries ``[1, Hq, L, 256]``; past keys / values as (packed, scales, biases) of
    ``[1, Hkv, P, ...]``; self_k / self_v ``[1, Hkv, L, 256]`` (already through the q8 round trip, :364-369).
    Every past key is visible to every query; self key j to query i iff j <= i.  Returns ``[1, Hq, L, 256]`` in the
    queries' type (``[1, L, Hq * 256]`` in the operand type when ``gate`` ``[1, L, Hq * 256]`` is given: the
    wrapper's epilogue fused).  The past is expanded into the front of one [P + L] operand and the flash kernel runs
    on it; ``bq`` / ``bk`` / ``stage`` are the reference kernel's tile knobs and have no meaning here."""
    dev = require_cuda(queries, k_packed, self_k)
    B, Hq, L, D = (int(x) for x in queries.shape)
    Hkv, P = int(k_packed.shape[1]), int(k_packed.shape[2])
    if B != 1 or D != FLASH_HEAD_DIM:
        raise ValueError("flash prefill requires batch 1 and head_dim=256")
    op = self_k.dtype if self_k.dtype in (torch.bfloat16, torch.float16) else torch.bfloat16
    kfull = torch.empty((Hkv, P + L, D), dtype=op, device=dev)
    vfull = torch.empty_like(kfull)
    for h in range(Hkv):
        if P:
            dequantize_affine_q8(k_packed[0, h], k_scales[0, h], k_biases[0, h], out=kfull[h, :P])
            dequantize_affine_q8(v_packed[0, h], v_scales[0, h], v_biases[0, h], out=vfull[h, :P])
    kfull[:, P:].copy_(self_k[0])
    vfull[:, P:].copy_(self_v[0])
    q = queries[0].to(op).permute(1, 0, 2)                       # [L, Hq, D]
    g = None if gate is None else gate.reshape(L, Hq, D).to(op)
    out = sdpa_fa_prefill(q, kfull.permute(1, 0, 2), vfull.permute(1, 0, 2), scale, gate=g, layout="lhd", check=check)
    if gate is not None:
        return out.reshape(1, L, Hq * D)
    return out.permute(1, 0, 2)[None].to(queries.dtype)


def sdpa_decode_q8(queries, k_packed, k_scales, k_biases, v_packed, v_scales, v_biases, scale, *, group_size: int = 64,
                   bits: int = 8, splits: int = 128, stage: int = 2, compute: int = 1, tile_c: int = 16,
                   dimension_parallel_merge: bool = False):
    """One decode token over the affine-q8 cache — the call at qwen/full_attention.py:323-335.  queries
    ``[1, Hq, 1, 256]``; keys / values as (packed, scales, biases) of ``[1, Hkv, P, ...]`` (views of a larger
    buffer are fine).  ``splits`` CTAs per KV head scan disjoint key ranges and a log-sum-exp merge finishes;
    the remaining knobs belong to the reference kernel.  Returns ``[1, Hq, 1, 256]`` in the queries' type."""
    from ..deepseek_v4.indexed_attention_kernel import merge_partials
    if group_size != Q8_GROUP or bits != Q8_BITS:
        raise ValueError("q8 decode requires group_size=64 and bits=8")
    dev = require_cuda(queries, k_packed, v_packed)
    B, Hq, T, D = (int(x) for x in queries.shape)
    Hkv, P = int(k_packed.shape[1]), int(k_packed.shape[2])
    if B != 1 or T != 1 or D != FLASH_HEAD_DIM:
        raise ValueError("q8 decode requires one token of batch 1 and head_dim=256")
    tensors = (k_packed, k_scales, k_biases, v_packed, v_scales, v_biases)
    strides = {int(t.stride(1)) // int(t.shape[3]) for t in tensors}
    if len(strides) != 1 or any(t.stride(3) != 1 or t.stride(2) != t.shape[3] for t in tensors):
        raise ValueError("q8 decode: cache tensors must be row-contiguous views with one capacity")
    splits = max(1, min(int(splits), P))
    q = queries.reshape(Hq, D).contiguous()
    o_parts = torch.empty((splits, 1, 1, Hq, D), dtype=torch.float32, device=dev)
    ml_parts = torch.empty((splits, 1, 1, Hq, 2), dtype=torch.float32, device=dev)
    a = _abi.SdpaDecodeQ8Args()
    a.q, a.q_dtype = ptr(q), dtype_code(q)
    a.k_packed, a.k_scales, a.k_biases = ptr(k_packed), ptr(k_scales), ptr(k_biases)
    a.v_packed, a.v_scales, a.v_biases = ptr(v_packed), ptr(v_scales), ptr(v_biases)
    a.sb_dtype, a.head_stride_rows = dtype_code(k_scales), strides.pop()
    a.P, a.Hq, a.Hkv, a.D, a.scale, a.n_splits = P, Hq, Hkv, D, float(scale), splits
    a.o_parts, a.ml_parts = ptr(o_parts), ptr(ml_parts)
    _abi.check(_t.launch("sdpa_decode_q8", _abi.load().mxb_sdpa_decode_q8, a))
    out = merge_partials(o_parts, ml_parts, None)                # [1, 1, Hq, D]
    return out.reshape(1, Hq, 1, D).to(queries.dtype)


class FlashPrefillD256Attention(torch.nn.Module):
    """Wrapper with the call shape and routing of the reference's ``FlashPrefillD256Attention``
    (qwen/full_attention.py:168-397).  ``inner`` owns ``q_proj`` (producing queries and gate interleaved per head),
    ``k_proj``, ``v_proj``, ``o_proj``, ``q_norm``, ``k_norm`` and ``rope(x, offset)``; attributes
    ``num_attention_heads``, ``num_key_value_heads``, ``head_dim``, ``scale``.

    Routes, first match wins:
    * a chunk (tokens > 1) over a ``QuantizedKVCache`` (bits 8, group 64, offset >= 1), mask "causal", batch 1,
      head_dim 256 -> ``sdpa_fa_prefill_q8`` with the self chunk through the q8 round trip (:348-382);
    * one token over such a cache with at least ``DECODE_Q8_MIN_KEYS`` keys and no mask -> ``sdpa_decode_q8``
      (:313-335);
    * a chunk over a ``DenseKVCache`` / no past, mask "causal", batch 1, head_dim 256 -> the dense flash kernel
      (an extension: benchmark configuration 2);
    * anything else is delegated to ``inner(x, mask=mask, cache=cache)`` and counted, as the reference falls
      back to the stock path."""

    def __init__(self, inner):
        super().__init__()
        self.inner = inner
        self.flash_calls = 0
        self.decode_calls = 0
        self.dense_flash_calls = 0
        self.rejected = {"batch": 0, "single_token": 0, "mask": 0, "head_dim": 0, "cache": 0}

    def _geometry_ok(self, x) -> bool:
        if int(x.shape[0]) != 1:
            self.rejected["batch"] += 1
            return False
        if int(self.inner.head_dim) != FLASH_HEAD_DIM:
            self.rejected["head_dim"] += 1
            return False
        return True

    def _q8_cache(self, cache) -> bool:
        return (isinstance(cache, QuantizedKVCache) and cache.bits == Q8_BITS and cache.group_size == Q8_GROUP
                and cache.offset >= 1)

    def route(self, x, mask, cache) -> str:
        """"prefill_q8", "decode_q8", "dense" or "inner" (counting the first failing condition)."""
        L = int(x.shape[1])
        if L == 1:
            if (self._q8_cache(cache) and cache.offset + 1 >= DECODE_Q8_MIN_KEYS and mask is None
                    and self._geometry_ok(x)):
                return "decode_q8"
            self.rejected["single_token"] += 1
            return "inner"
        if mask != "causal":
            self.rejected["mask"] += 1
            return "inner"
        if not self._geometry_ok(x):
            return "inner"
        if self._q8_cache(cache):
            return "prefill_q8"
        if cache is None or isinstance(cache, DenseKVCache):
            return "dense"
        self.rejected["cache"] += 1
        return "inner"

    def forward(self, x, mask=None, cache=None):
        route = self.route(x, mask, cache)
        if route == "inner":
            return self.inner(x, mask=mask, cache=cache)
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
        offset = 0 if cache is None else int(cache.offset)
        queries = inner.rope(queries, offset)
        keys = inner.rope(keys, offset)
        gate = gate.reshape(B, L, Hq * D)
        if route == "decode_q8":
            qk, qv = cache.update_and_fetch(keys, values)
            self.decode_calls += 1
            out = sdpa_decode_q8(queries, *qk, *qv, float(inner.scale), group_size=Q8_GROUP, bits=Q8_BITS, splits=128,
                                 stage=2, compute=1, tile_c=16)
            out = out.transpose(1, 2).reshape(B, L, Hq * D)
            return inner.o_proj(out * torch.sigmoid(gate.to(out.dtype)))
        if route == "prefill_q8":
            past_k, past_v = cache.state                  # the prefix BEFORE the update appends the fresh chunk
            cache.update_and_fetch(keys, values)
            sb = cache.keys[1].dtype
            self_k = dequantize_affine_q8(*quantize_affine_q8(keys.to(sb)))      # the composed path's values (:364-369)
            self_v = dequantize_affine_q8(*quantize_affine_q8(values.to(sb)))
            self.flash_calls += 1
            out = sdpa_fa_prefill_q8(queries, *past_k, *past_v, self_k, self_v, float(inner.scale), bq=64, bk=16, stage=2,
                                     gate=gate)
            return inner.o_proj(out.to(x.dtype))
        if cache is not None:
            keys, values = cache.update_and_fetch(keys, values)
        self.dense_flash_calls += 1
        op = keys.dtype if keys.dtype in (torch.bfloat16, torch.float16) else torch.bfloat16
        out = sdpa_fa_prefill(queries.to(op), keys.to(op), values.to(op), float(inner.scale), gate=gate)
        return inner.o_proj(out.to(x.dtype))


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
    stats = {"layers": 0, "flash_calls": 0, "decode_calls": 0, "dense_flash_calls": 0,
             "rejected": {"batch": 0, "single_token": 0, "mask": 0, "head_dim": 0, "cache": 0}}
    for layer in getattr(model, "layers", []):
        attn = getattr(layer, "self_attn", None)
        if isinstance(attn, FlashPrefillD256Attention):
            stats["layers"] += 1
            stats["flash_calls"] += attn.flash_calls
            stats["decode_calls"] += attn.decode_calls
            stats["dense_flash_calls"] += attn.dense_flash_calls
            for key, val in attn.rejected.items():
                stats["rejected"][key] += val
    return stats
