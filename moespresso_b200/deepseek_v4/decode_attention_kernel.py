"""DS4 decode-side cache operators with the reference's names
(reference: src/moespresso/runtime/deepseek_v4/decode_attention_kernel.py).

``fp8_kv_prefix_rows``   E4M3FN round trip of the non-rotary prefix of 512-wide compressed-KV rows (:587-619)

``fused_decode_prep``    QAT of q, scores, exact top-k, and the prepared KV row (rope tail + FP8 round trip) (:669-730)
``fused_decode_sdpa``    rope on q, attention over the window (with the prepared row) and the selected rows, sink,
                         inverse rope (:733-786)

The two fused operators are compositions of this package's kernels (the reference runs each as one Metal launch);
``params`` is read on the device, so neither synchronises with the host and both can be captured in a CUDA graph.
"""
from __future__ import annotations

import torch

from .. import _abi
from .. import _torchabi as _t
from .._torchabi import ptr, require_cuda

_HEAD_DIM = 512


def fp8_kv_prefix_rows(x, *, replay: bool = False):
    """``x`` ``[..., 512]`` float32 -> float32 of the same shape: dims [0, 448) through DS4's E4M3FN round trip
    (power-of-two scale per 64-element block), dims [448, 512) unchanged.  ``replay=True`` evaluates the
    reference's NumPy replay form instead (compressor_diff.py:74-86: exact power-of-two scale, ties to even)."""
    if x.ndim < 1 or int(x.shape[-1]) != _HEAD_DIM:
        raise ValueError("fp8 rows expect 512-wide rows")
    if x.dtype != torch.float32:
        raise ValueError("fp8 rows must be float32")
    dev = require_cuda(x)
    rows2d = x.reshape(-1, _HEAD_DIM).contiguous()
    n_rows = int(rows2d.shape[0])
    if n_rows == 0:
        raise ValueError("fp8 rows expect at least one row")
    out = torch.empty((n_rows, _HEAD_DIM), dtype=torch.float32, device=dev)
    a = _abi.Fp8KvRowsArgs()
    a.x, a.out, a.n_rows, a.width, a.mode = ptr(rows2d), ptr(out), n_rows, _HEAD_DIM, 1 if replay else 0
    _abi.check(_t.launch("fp8_kv_rows", _abi.load().mxb_fp8_kv_rows, a))
    return out.reshape(x.shape)


_INDEX_HEAD_DIM = 128
_MAX_HEADS = 64
_ROPE_DIM = 64


def _position(params):
    """The token position as a one-element int64 device tensor (no host round trip)."""
    return params.reshape(-1)[0:1].to(torch.int64)


def fused_decode_prep(q_idx, pooled_qat, weights, kv_row, inv_freq, params, *, scale, topk):
    """Score, select, and prepare the KV row for one ratio-4 decode token (reference: :669-730).

    q_idx ``[n_heads, 128]`` (float32 / float16 / bfloat16, post-rope, pre-QAT), pooled_qat float32
    ``[n_rows, 128]``, weights float32 ``[n_heads]`` (already times ``n_heads ** -0.5``), kv_row float16 ``[512]``
    (post-norm, pre-rope), inv_freq float32 ``[32]``, params int32 with the token position first.
    Returns ``(sel int32 [topk], row float16 [512], scores float32 [n_rows])``: the selected pool rows (the exact
    top-k with ties to the lower row; ids ASCENDING here, where the reference emits the strictly-above rows first
    and the boundary ties after them — the same set), the roped and FP8-rounded KV row, and the scores.
    Composed of the QAT, score, top-k, FP8 round-trip and rope operators of this package (five launches)."""
    from .attention import apply_rope_tail, topk_select
    from .indexer_score_kernel import fused_qat_indexer_scores
    if q_idx.ndim != 2 or int(q_idx.shape[1]) != _INDEX_HEAD_DIM:
        raise ValueError("q_idx must have shape [n_heads, 128]")
    n_heads = int(q_idx.shape[0])
    if n_heads <= 0 or n_heads > _MAX_HEADS:
        raise ValueError("q_idx must carry between 1 and 64 heads")
    if q_idx.dtype not in (torch.float32, torch.float16, torch.bfloat16):
        raise ValueError("q_idx must be float32, float16, or bfloat16")
    if pooled_qat.ndim != 2 or int(pooled_qat.shape[1]) != _INDEX_HEAD_DIM or pooled_qat.dtype != torch.float32:
        raise ValueError("pooled_qat must be float32 [n_rows, 128]")
    n_rows = int(pooled_qat.shape[0])
    topk = int(topk)
    if not 0 < topk < n_rows:
        raise ValueError("topk must be positive and smaller than n_rows")
    if tuple(int(v) for v in weights.shape) != (n_heads,) or weights.dtype != torch.float32:
        raise ValueError("weights must be float32 [n_heads]")
    if tuple(int(v) for v in kv_row.shape) != (_HEAD_DIM,) or kv_row.dtype != torch.float16:
        raise ValueError("kv_row must be float16 [512]")
    if int(inv_freq.shape[-1]) != _ROPE_DIM // 2 or inv_freq.dtype != torch.float32:
        raise ValueError("inv_freq must be float32 [32]")
    require_cuda(q_idx, pooled_qat, weights, kv_row, inv_freq, params)
    scores = fused_qat_indexer_scores(q_idx.reshape(1, n_heads, 1, _INDEX_HEAD_DIM), pooled_qat[None],
                                      weights.reshape(1, 1, n_heads), scale)
    sel = topk_select(scores[None], topk)[0]
    # the round trip touches dims [0, 448), the rope dims [448, 512): they commute
    row = fp8_kv_prefix_rows(kv_row.float()[None])[0].to(torch.float16)
    roped = apply_rope_tail(kv_row.reshape(1, 1, _HEAD_DIM), _position(params), inv_freq=inv_freq, half_chain=True)
    row[_HEAD_DIM - _ROPE_DIM:] = roped.reshape(-1)[_HEAD_DIM - _ROPE_DIM:]
    return sel, row, scores


def fused_decode_sdpa(q, window, row, pooled, sel, sinks, inv_freq, params, *, scale):
    """Attend one decode token over the window and the selected pooled rows (reference: :733-786).

    q float16 ``[n_heads, 512]`` (post-norm, pre-rope), window float16 ``[window_rows, 512]`` (pre-update), row
    float16 ``[512]`` (from ``fused_decode_prep``; replaces ``window[write_idx]``), pooled float16 ``[n_rows, 512]``,
    sel int32 ``[topk]``, sinks float16 ``[n_heads]``, inv_freq float32 ``[32]``, params int32
    ``[position, write_idx]``.  Every window row and every selected row is a key and a value; the sink joins the
    maximum and the denominator once.  Returns float16 ``[n_heads, 512]`` after the inverse rope.
    Composed of the rope and sparse-attention operators of this package."""
    from .attention import apply_rope_tail
    from .indexed_attention_kernel import sparse_attention
    if q.ndim != 2 or int(q.shape[1]) != _HEAD_DIM or q.dtype != torch.float16:
        raise ValueError("q must be float16 [n_heads, 512]")
    n_heads = int(q.shape[0])
    if n_heads <= 0:
        raise ValueError("q must carry at least one head")
    if window.ndim != 2 or int(window.shape[1]) != _HEAD_DIM or window.dtype != torch.float16:
        raise ValueError("window must be float16 [window_rows, 512]")
    if tuple(int(v) for v in row.shape) != (_HEAD_DIM,) or row.dtype != torch.float16:
        raise ValueError("row must be float16 [512]")
    if pooled.ndim != 2 or int(pooled.shape[1]) != _HEAD_DIM or pooled.dtype != torch.float16:
        raise ValueError("pooled must be float16 [n_rows, 512]")
    if sel.ndim != 1 or sel.dtype != torch.int32:
        raise ValueError("sel must be int32 [topk]")
    if tuple(int(v) for v in sinks.shape) != (n_heads,) or sinks.dtype != torch.float16:
        raise ValueError("sinks must be float16 [n_heads]")
    if int(inv_freq.shape[-1]) != _ROPE_DIM // 2 or inv_freq.dtype != torch.float32:
        raise ValueError("inv_freq must be float32 [32]")
    require_cuda(q, window, row, pooled, sel, sinks, inv_freq, params)
    pos = _position(params)
    write_idx = params.reshape(-1)[1:2].to(torch.int64)
    window_rows = int(window.shape[0])
    qr = apply_rope_tail(q.reshape(1, n_heads, _HEAD_DIM).transpose(0, 1).contiguous(), pos, inv_freq=inv_freq,
                         half_chain=True)                                   # [H, 1, 512]
    # the prepared row replaces window[write_idx] (an index outside the window replaces nothing), on the device
    slot = torch.arange(window_rows, device=window.device, dtype=torch.int64)[:, None] == write_idx
    win = torch.where(slot, row[None], window)
    # all window rows are keys: place the window so that its last row is the newest position and nothing is clipped
    pos0 = torch.clamp(pos, min=window_rows - 1)
    out = sparse_attention(qr.reshape(1, n_heads, 1, _HEAD_DIM), pooled, sel.reshape(1, 1, -1), sinks.float(),
                           pos0=0, pos0_dev=pos0, window=0, ratio=0, raw_kv=win[None], raw_start=0,
                           scale=float(scale), d_v=_HEAD_DIM, out_dtype=torch.float16)
    out = out.reshape(n_heads, 1, _HEAD_DIM)
    return apply_rope_tail(out, pos, inv_freq=inv_freq, inverse=True, half_chain=True).reshape(n_heads, _HEAD_DIM)
