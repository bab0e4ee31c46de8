"""DS4 decode indexer operators with the reference's names
(reference: src/moespresso/runtime/deepseek_v4/indexer_score_kernel.py).

``indexer_qat_rows``          Hadamard-128 + e2m1 round trip of 128-wide rows          (:284-317)
``fused_qat_indexer_scores``  QAT of the query heads, then the decode score row          (:354-409)
``fused_score_tail``          relu / scale / head weights / head sum / +inf tail / negate (:562-615)

Tensors are torch CUDA tensors; there is no CPU path.
"""
from __future__ import annotations

import torch

from .. import _abi
from .. import _torchabi as _t
from .._torchabi import dtype_code, ptr, require_cuda
from .indexed_attention_kernel import indexer_scores

_HEAD_DIM = 128
_MAX_HEADS = 64
_TAIL_MIN_HEADS = 32
_TAIL_MAX_HEADS = 64
_QUERY_DTYPES = (torch.float32, torch.float16, torch.bfloat16)


def indexer_qat_rows(x):
    """``x`` ``[..., 128]`` float32 / float16 / bfloat16 -> float32 of the same shape: the rows after the
    size-128 Walsh-Hadamard transform (scale 128^-0.5) and the e2m1 round trip over 32-element groups."""
    if x.ndim < 1 or int(x.shape[-1]) != _HEAD_DIM:
        raise ValueError("indexer QAT expects 128-wide rows")
    if x.dtype not in _QUERY_DTYPES:
        raise ValueError("indexer QAT rows must be float32, float16, or bfloat16")
    dev = require_cuda(x)
    rows2d = x.reshape(-1, _HEAD_DIM).contiguous()
    n_rows = int(rows2d.shape[0])
    if n_rows == 0:
        raise ValueError("indexer QAT expects at least one row")
    out = torch.empty((n_rows, _HEAD_DIM), dtype=torch.float32, device=dev)
    a = _abi.IndexerQatArgs()
    a.x, a.x_dtype, a.out, a.n_rows, a.width = ptr(rows2d), dtype_code(rows2d), ptr(out), n_rows, _HEAD_DIM
    _abi.check(_t.launch("indexer_qat", _abi.load().mxb_indexer_qat, a))
    return out.reshape(x.shape)


def fused_qat_indexer_scores(q, pooled_qat, weights, scale):
    """Decode indexer score row: ``scores[r] = sum_h max(qat(q_h) . pooled_r, 0) * scale * weights[h]``.

    q ``[1, n_heads, 1, 128]`` (float32 / float16 / bfloat16, post-rope, pre-QAT), pooled_qat float32
    ``[1, n_rows, 128]``, weights float32 ``[1, 1, n_heads]`` (already times ``n_heads ** -0.5``).
    Returns float32 ``[n_rows]``.  Two launches: the QAT of the query heads, then the exact fp32 score kernel."""
    if q.ndim != 4:
        raise ValueError("q must have shape [1, n_heads, 1, 128]")
    batch, n_heads, tokens, head_dim = (int(v) for v in q.shape)
    if batch != 1 or tokens != 1:
        raise ValueError("fused indexer scoring handles one decode token")
    if head_dim != _HEAD_DIM:
        raise ValueError("DS4 fused indexer scoring requires head_dim=128")
    if n_heads <= 0 or n_heads > _MAX_HEADS:
        raise ValueError("q must carry between 1 and 64 heads")
    if pooled_qat.ndim != 3 or int(pooled_qat.shape[0]) != 1 or int(pooled_qat.shape[2]) != head_dim:
        raise ValueError("pooled_qat must have shape [1, n_rows, 128]")
    n_rows = int(pooled_qat.shape[1])
    if n_rows <= 0:
        raise ValueError("pooled_qat must contain at least one row")
    if tuple(int(v) for v in weights.shape) != (1, 1, n_heads):
        raise ValueError("weights must have shape [1, 1, n_heads]")
    if q.dtype not in _QUERY_DTYPES:
        raise ValueError("q must be float32, float16, or bfloat16")
    if pooled_qat.dtype != torch.float32 or weights.dtype != torch.float32:
        raise ValueError("pooled_qat and weights must be float32")
    require_cuda(q, pooled_qat, weights)
    q_qat = indexer_qat_rows(q)                                            # [1, H, 1, 128] float32
    w = (weights.reshape(1, 1, n_heads) * float(scale)).contiguous()       # scale folded into the head weights
    out = indexer_scores(q_qat, w, pooled_qat.reshape(n_rows, head_dim).contiguous(), n_rows=n_rows,
                         exact_fp32=True)
    return out.reshape(n_rows)


def fused_score_tail(scores, weights_raw, params, *, scale):
    """Finish the fixed-state score chain: scores float32 ``[1, n_heads, 1, capacity]`` (per-head dot products),
    weights_raw ``[1, 1, n_heads]`` (raw projection, float32 / float16 / bfloat16), params int32 with the valid
    row count at index 1.  Returns float32 ``[1, 1, capacity]``: the negated scores on the valid prefix, ``+inf``
    behind it."""
    if scores.ndim != 4:
        raise ValueError("scores must have shape [1, n_heads, 1, capacity]")
    batch, n_heads, tokens, capacity = (int(v) for v in scores.shape)
    if batch != 1 or tokens != 1:
        raise ValueError("the fused score tail handles one decode token")
    if capacity <= 0:
        raise ValueError("scores must cover at least one capacity column")
    if not _TAIL_MIN_HEADS <= n_heads <= _TAIL_MAX_HEADS:
        raise ValueError("the score tail transcription covers 32 to 64 index heads")
    if scores.dtype != torch.float32:
        raise ValueError("scores must be float32")
    if tuple(int(v) for v in weights_raw.shape) != (1, 1, n_heads):
        raise ValueError("weights_raw must have shape [1, 1, n_heads]")
    if weights_raw.dtype not in _QUERY_DTYPES:
        raise ValueError("weights_raw must be float32, float16, or bfloat16")
    if params.dtype != torch.int32 or params.numel() < 2:
        raise ValueError("params must be int32 with the row count at index 1")
    dev = require_cuda(scores, weights_raw, params)
    s2 = scores.reshape(n_heads, capacity).contiguous()
    w1 = weights_raw.reshape(n_heads).contiguous()
    out = torch.empty((capacity,), dtype=torch.float32, device=dev)
    a = _abi.ScoreTailArgs()
    a.scores, a.weights_raw, a.w_dtype, a.params, a.out = ptr(s2), ptr(w1), dtype_code(w1), ptr(params), ptr(out)
    a.H, a.capacity, a.scale = n_heads, capacity, float(scale)
    _abi.check(_t.launch("score_tail", _abi.load().mxb_score_tail, a))
    return out.reshape(1, 1, capacity)
