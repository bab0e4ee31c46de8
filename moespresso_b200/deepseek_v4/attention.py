"""Top-k selection and the indexer top-k contract on B200.

``causal_indexer_topk`` keeps the signature of the reference's NumPy contract
(``src/moespresso/runtime/deepseek_v4/attention.py:277-313``); ``topk_select`` is
the device operator behind it and behind the served ``argpartition`` + ``sort``
(``src/moespresso/runtime/deepseek_v4/model.py:1003-1005,1442-1451``).
"""
from __future__ import annotations

import ctypes as C

import torch

from .. import _abi
from .. import _torchabi as _t
from .._torchabi import ptr, require_cuda, stream_ptr, workspace


def topk_select(scores, k: int, *, valid=None, row_start=None, n=None, order: str = "index", digit_hist=None):
    """Ids of the k largest finite scores of every row; ties to the lower id;
    -inf / NaN never selected; -1 in unused slots.

    scores: float32 ``[..., n]`` (rows are the leading axes) or, with ``row_start``
    (int64 ``[rows]``) and ``valid`` (int32 ``[rows]``), one flat vector holding ragged
    rows, ``n`` = the longest row.  ``order="index"``: ids ascending (what the
    attention kernels walk); ``order="score"``: descending score, ties by ascending id
    (the order of the NumPy contract).  Returns int32 ``[..., k]``.  ``digit_hist``: int32 ``[rows, 2048]`` as
    ``indexer_scores(..., digit_hist=)`` left it for exactly these scores; the selection skips its first pass and
    leaves the counters at zero for the next step.
    """
    dev = require_cuda(scores)
    if scores.dtype != torch.float32:
        raise ValueError("scores must be float32")
    if int(k) <= 0:
        raise ValueError("topk must be positive")
    lib = _abi.load()
    scores = scores.contiguous()
    if row_start is None:
        lead = scores.shape[:-1]
        n_ = int(scores.shape[-1])
        rows = 1
        for s in lead:
            rows *= int(s)
        row_stride = n_
    else:
        lead = (int(row_start.numel()),)
        rows = lead[0]
        n_ = int(n)
        row_stride = 0
    out = torch.empty((rows, int(k)), dtype=torch.int32, device=dev)
    if rows == 0:
        return out.reshape(*lead, int(k))
    if valid is not None:
        valid = valid.to(torch.int32).contiguous()
    a = _abi.TopkArgs()
    a.scores = ptr(scores); a.row_stride = row_stride; a.row_start = ptr(row_start); a.row_count = ptr(valid)
    a.out_ids = ptr(out); a.rows = rows; a.n = n_; a.k = int(k)
    ws = workspace(lib.mxb_topk_workspace_bytes(rows, n_, int(k)), dev)
    a.workspace = ptr(ws); a.workspace_bytes = 0 if ws is None else ws.numel()
    if digit_hist is not None:
        if digit_hist.dtype != torch.int32 or tuple(digit_hist.shape) != (rows, 2048) or not digit_hist.is_contiguous():
            raise ValueError("digit_hist must be a contiguous int32 [rows, 2048] tensor")
        a.digit_hist = ptr(digit_hist)
    _abi.check(_t.launch("topk_select", lib.mxb_topk_select, a))
    out = out.reshape(*lead, int(k))
    if order == "score":
        if row_start is not None:
            raise ValueError("score order is available for rectangular score matrices only")
        flat = scores.reshape(rows, n_)
        ids = out.reshape(rows, int(k)).long()
        picked = torch.gather(flat, 1, ids.clamp(min=0))
        picked = torch.where(ids >= 0, picked, torch.full_like(picked, float("-inf")))
        perm = torch.sort(picked, dim=1, descending=True, stable=True).indices
        out = torch.gather(ids, 1, perm).to(torch.int32).reshape(*lead, int(k))
    elif order != "index":
        raise ValueError("order must be 'index' or 'score'")
    return out


def causal_indexer_topk(raw_scores, head_weights, query_positions, pool_indices, ratio: int, *, topk: int = 512,
                        index_head_dim: int = 128, n_heads: int = 64):
    """Device form of the reference's ``causal_indexer_topk``: raw per-head scores
    ``[queries, heads, pool_rows]`` and head weights ``[queries, heads]`` -> int64
    ``[queries, min(topk, pool_rows)]`` pool ids in descending-score order, ``-1`` padded."""
    if int(ratio) <= 0:
        raise ValueError("ratio must be positive")
    if int(topk) <= 0:
        raise ValueError("topk must be positive")
    require_cuda(raw_scores)
    raw = raw_scores.to(torch.float32)
    w = head_weights.to(torch.float32)
    if raw.ndim != 3:
        raise ValueError("raw_scores must have shape (queries, heads, pool_rows)")
    if tuple(w.shape) != tuple(raw.shape[:2]):
        raise ValueError("head_weights must have shape (queries, heads)")
    scale = (index_head_dim ** -0.5) * (n_heads ** -0.5)
    scores = (torch.clamp_min(raw, 0) * w[..., None]).sum(dim=1) * scale
    qpos = torch.as_tensor(query_positions, device=raw.device, dtype=torch.int64).reshape(-1)
    pool = torch.as_tensor(pool_indices, device=raw.device, dtype=torch.int64).reshape(-1)
    vis = ((pool[None, :] + 1) * int(ratio)) <= (qpos[:, None] + 1)
    scores = torch.where(vis, scores, torch.full_like(scores, float("-inf")))
    width = min(int(topk), int(pool.numel()))
    if width == 0:
        return torch.empty((raw.shape[0], 0), dtype=torch.int64, device=raw.device)
    ids = topk_select(scores, width, order="score").long()
    return torch.where(ids >= 0, pool[ids.clamp(min=0)], torch.full_like(ids, -1))


def topk_select_static(scores, k: int, out, *, valid=None, row_start=None, n=None):
    """``topk_select`` for callers that cannot allocate device memory at call time (a
    server with a frozen memory pool, code running inside an allocator callback): the
    caller passes the int32 output ``[rows, k]`` and the kernel's candidate scratch is the
    8 MiB array built into the library, so ``rows * n`` is limited to 2**20.  Ids come back
    ascending, ``-1`` padded, exactly as from ``topk_select``.  Calls share the scratch:
    keep them on one stream.  The first call on a device resolves the scratch address and
    should happen outside stream capture."""
    dev = require_cuda(scores, out)
    if scores.dtype != torch.float32 or not scores.is_contiguous():
        raise ValueError("scores must be contiguous float32")
    if out.dtype != torch.int32 or not out.is_contiguous():
        raise ValueError("out must be contiguous int32")
    lib = _abi.load()
    if row_start is None:
        n_ = int(scores.shape[-1])
        rows = scores.numel() // n_
        row_stride = n_
    else:
        rows, n_, row_stride = int(row_start.numel()), int(n), 0
    if out.numel() != rows * int(k):
        raise ValueError("out must have rows * k elements")
    a = _abi.TopkArgs()
    a.scores = ptr(scores); a.row_stride = row_stride; a.row_start = ptr(row_start); a.row_count = ptr(valid)
    a.out_ids = ptr(out); a.rows = rows; a.n = n_; a.k = int(k)
    _abi.check(_t.launch("topk_select_static", lib.mxb_topk_select_static, a))
    return out


# --------------------------------------------------------------------------- #
# partial rotary embedding (reference: src/moespresso/runtime/deepseek_v4/attention.py:20-31, 71-156)
# --------------------------------------------------------------------------- #
DS4_ROPE_DIM = 64
DS4_SWA_ROPE_BASE = 10000.0
DS4_COMPRESS_ROPE_BASE = 160000.0
DS4_YARN = {"factor": 16.0, "original_seq_len": 65536.0, "beta_fast": 32.0, "beta_slow": 1.0}


def rope_inverse_frequencies(dim: int, base: float, yarn=None):
    """RoPE inverse frequencies in float64 (host side), including DS4's pure-frequency YaRN variant
    (reference: attention.py:71-101).  Returns a NumPy array ``[dim / 2]``."""
    import math

    import numpy as np
    if dim <= 0 or dim % 2:
        raise ValueError("RoPE dim must be a positive even integer")
    freqs = 1.0 / (float(base) ** (np.arange(0, dim, 2, dtype=np.float64) / dim))
    if not yarn:
        return freqs
    factor, original = float(yarn["factor"]), float(yarn["original_seq_len"])
    beta_fast, beta_slow = float(yarn.get("beta_fast", 32.0)), float(yarn.get("beta_slow", 1.0))
    if factor <= 1.0 or original <= 0:
        return freqs

    def correction_dim(n: float) -> float:
        return dim * math.log(original / (n * 2.0 * math.pi)) / (2.0 * math.log(base))

    low = max(math.floor(correction_dim(beta_fast)), 0)
    high = min(math.ceil(correction_dim(beta_slow)), dim - 1)
    if low == high:
        high += 0.001
    smooth = 1.0 - np.clip((np.arange(dim // 2, dtype=np.float64) - low) / (high - low), 0.0, 1.0)
    return freqs / factor * (1.0 - smooth) + freqs * smooth


def apply_rope_tail(x, positions, *, base: float = None, yarn=None, rope_dim: int = DS4_ROPE_DIM,
                    inverse: bool = False, out=None, inv_freq=None, half_chain: bool = False):
    """DS4 partial RoPE on only the final ``rope_dim`` channels (interleaved pairs); the sequence axis is the
    second-to-last axis; leading channels are copied (reference: attention.py:114-156).

    x: CUDA tensor ``[..., seq, features]`` float32 / float16 / bfloat16; positions: ``seq`` integers (sequence,
    NumPy array or tensor).  Angles are formed in float64 and the result is rounded once to ``x.dtype``.
    ``out=x`` rotates in place.  ``inv_freq`` (``rope_dim / 2`` values) replaces ``base`` / ``yarn``;
    ``half_chain=True`` (float16 rows) rotates the way the fused decode kernels do: float32 angle, cos / sin and
    every product and sum rounded to float16."""
    import numpy as np
    if x.ndim < 2:
        raise ValueError("x must have at least sequence and feature dimensions")
    if rope_dim <= 0 or rope_dim % 2:
        raise ValueError("rope_dim must be a positive even integer")
    if int(x.shape[-1]) < rope_dim:
        raise ValueError("rope_dim cannot exceed the feature dimension")
    dev = require_cuda(x)
    if isinstance(positions, torch.Tensor):
        pos = positions.reshape(-1).to(device=dev, dtype=torch.int64)
    else:
        pos = torch.as_tensor(np.asarray(positions).reshape(-1).astype(np.int64), device=dev)
    if int(x.shape[-2]) != int(pos.numel()):
        raise ValueError("positions length must match x.shape[-2]")
    if x.dtype not in (torch.float32, torch.float16, torch.bfloat16):
        raise ValueError("x must be float32, float16, or bfloat16")
    x = x.contiguous()
    if out is None:
        out = torch.empty_like(x)
    elif out.shape != x.shape or out.dtype != x.dtype or not out.is_contiguous():
        raise ValueError("out must be a contiguous tensor with x's shape and dtype")
    if inv_freq is None:
        if base is None:
            raise ValueError("either base or inv_freq must be given")
        inv = torch.as_tensor(rope_inverse_frequencies(rope_dim, base, yarn), dtype=torch.float64, device=dev)
    else:
        inv = torch.as_tensor(inv_freq).reshape(-1).to(device=dev, dtype=torch.float64)
        if int(inv.numel()) != rope_dim // 2:
            raise ValueError("inv_freq must hold rope_dim / 2 values")
    if half_chain and x.dtype != torch.float16:
        raise ValueError("half_chain takes float16 rows")
    a = _abi.RopeTailArgs()
    a.x, a.out, a.x_dtype = ptr(x), ptr(out), _t.dtype_code(x)
    a.positions, a.inv_freq = ptr(pos), ptr(inv)
    a.n_rows = int(x.numel() // x.shape[-1])
    a.seq_len, a.width, a.rope_dim, a.inverse = int(x.shape[-2]), int(x.shape[-1]), int(rope_dim), 1 if inverse else 0
    a.half_chain = 1 if half_chain else 0
    if a.n_rows == 0:
        return out
    _abi.check(_t.launch("rope_tail", _abi.load().mxb_rope_tail, a))
    return out
