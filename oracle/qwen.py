"""CPU oracle for the Qwen/Ornith causal GQA prefill attention (NumPy).

TEST INFRASTRUCTURE ONLY (same rule as ``oracle/ds4.py``).

PARITY UNPINNED: the reference computes this operator inside the third-party
package ``mlx-kquant`` 0.3.0 (git e165cafafa149493d298871c610e29e95ffa8f10,
``sdpa_fa_prefill_q8``), whose source is not part of the reference tree, and
its own tests for the call site (tests/test_qwen_flash_prefill_attention.py)
need MLX and are skipped on Linux.  This file restates the published
definition the reference's wrapper relies on
(src/moespresso/runtime/qwen/full_attention.py:279-397): softmax(Q K^T * scale
+ causal) V with each KV head shared by Hq/Hkv query heads (q head h uses kv
head h // (Hq/Hkv)), every past key visible, then ``out * sigmoid(gate)``
(:396-397).
"""
from __future__ import annotations

import numpy as np


def causal_gqa_prefill(q, k, v, gate=None, *, scale, past_len: int = 0, dtype=np.float64,
                       q_rows=None) -> np.ndarray:
    """q [S, Hq, D]; k, v [P+S, Hkv, D] (first ``past_len`` keys are the past,
    all visible); gate [S, Hq, D] or None.  Key j is visible to query row i iff
    j <= i + past_len.  Returns [S, Hq, D] (``q_rows``: only those query rows,
    used to bound the timed CPU baseline)."""
    f = dtype
    q = np.asarray(q, dtype=f)
    k = np.asarray(k, dtype=f)
    v = np.asarray(v, dtype=f)
    S, Hq, D = q.shape
    Hkv = k.shape[1]
    group = Hq // Hkv
    rows = np.arange(S) if q_rows is None else np.asarray(q_rows)
    out = np.zeros((rows.size, Hq, D), dtype=f)
    kpos = np.arange(k.shape[0])
    for h in range(Hq):
        kh = k[:, h // group, :]
        vh = v[:, h // group, :]
        s = (q[rows, h, :] @ kh.T) * f(scale)
        s = np.where(kpos[None, :] <= (rows[:, None] + past_len), s, -np.inf)
        m = s.max(axis=1, keepdims=True)
        p = np.exp(s - m)
        out[:, h, :] = (p @ vh) / p.sum(axis=1, keepdims=True)
    if gate is not None:
        g = np.asarray(gate, dtype=f)[rows]
        out = out * (1.0 / (1.0 + np.exp(-g)))
    return out


# --------------------------------------------------------------------------- #
# Affine 8-bit format (group 64) of the served Qwen KV cache.
#
# PARITY UNPINNED as well: mx.quantize / mx.dequantize belong to MLX, whose source is not part of the reference
# tree; the reference only calls them (src/moespresso/runtime/qwen/full_attention.py:364-369) and passes the
# cache's (packed, scales, biases) triples to mlx-kquant (:323-335, :372-382).  The functions below restate the
# definition MLX documents for mx.quantize: per group of 64, bias = min, scale = (max - min) / 255,
# element = round((w - bias) / scale), w ~= element * scale + bias, four elements per uint32 (lowest byte first).
# Scales and biases are rounded to the storage type first, then the elements are taken against the stored values.
# --------------------------------------------------------------------------- #

def _round_to(x, kind: str):
    x = np.asarray(x, dtype=np.float32)
    if kind == "f32":
        return x
    if kind == "f16":
        return x.astype(np.float16).astype(np.float32)
    u = x.view(np.uint32).astype(np.uint64)          # bf16, nearest even
    return ((u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFF0000).astype(np.uint32).view(np.float32)


def affine_q8_quantize(x, kind: str = "bf16"):
    """x [..., D] (values already representable in `kind`) -> (packed uint32 [..., D/4], scales, biases [..., D/64]
    as float32 holding values of type `kind`)."""
    x = np.asarray(x, dtype=np.float32)
    D = x.shape[-1]
    g = x.reshape(*x.shape[:-1], D // 64, 64)
    lo, hi = g.min(axis=-1), g.max(axis=-1)
    scale = _round_to((hi - lo) / np.float32(255.0), kind)
    bias = _round_to(lo, kind)
    inv = np.where(scale > 0, np.float32(1.0) / np.where(scale > 0, scale, 1), 0).astype(np.float32)
    q = np.clip(np.floor((g - bias[..., None]) * inv[..., None] + np.float32(0.5)), 0, 255).astype(np.uint32)
    q = q.reshape(*x.shape[:-1], D // 4, 4)
    packed = q[..., 0] | (q[..., 1] << 8) | (q[..., 2] << 16) | (q[..., 3] << 24)
    return packed.astype(np.uint32), scale, bias


def affine_q8_dequantize(packed, scales, biases):
    """-> float32 [..., D] (one fused multiply-add per element in float32, as the kernels evaluate it)."""
    packed = np.asarray(packed, dtype=np.uint32)
    q = np.stack([(packed >> (8 * i)) & 0xFF for i in range(4)], axis=-1).reshape(*packed.shape[:-1], -1)
    D = q.shape[-1]
    g = q.reshape(*q.shape[:-1], D // 64, 64).astype(np.float64)
    w = g * np.asarray(scales, np.float64)[..., None] + np.asarray(biases, np.float64)[..., None]
    return w.reshape(*q.shape[:-1], D).astype(np.float32)


def prefill_q8(q, past_k, past_v, self_k, self_v, gate=None, *, scale, kind: str = "bf16", q_rows=None):
    """The composed path the reference tests its kernel against (tests/test_qwen_flash_prefill_attention.py:114-141):
    dequantise the past, concatenate the self chunk, attend causally.  q [L, Hq, D]; past_k / past_v
    (packed, scales, biases) with leading shape [P, Hkv]; self_k / self_v [L, Hkv, D] float."""
    pk = affine_q8_dequantize(*past_k)
    pv = affine_q8_dequantize(*past_v)
    k = np.concatenate([pk, np.asarray(self_k, np.float32)], axis=0)
    v = np.concatenate([pv, np.asarray(self_v, np.float32)], axis=0)
    return causal_gqa_prefill(q, k, v, gate, scale=scale, past_len=pk.shape[0], q_rows=q_rows)
