"""Indexed mixed attention and tiled indexer scores on B200.

Same function names, argument order and error behaviour as the reference module
``src/moespresso/runtime/deepseek_v4/indexed_attention_kernel.py`` (MLX/Metal);
tensors are ``torch`` CUDA tensors.  Keyword-only extensions that the reference
does not have (``scale``, ``d_v``, ``kv_scales``, ``out_dtype``) default to the
reference's behaviour: scale = head_dim**-0.5, V = the whole row, fp32 output.
"""
from __future__ import annotations

import ctypes as C

import torch

from .. import _abi
from .. import _torchabi as _t
from .._torchabi import dtype_code, last_dim_contiguous, ptr, require_cuda, status_word, stream_ptr, workspace

_CONSUMER_CALL_COUNTS = {"decode": 0, "prefill": 0, "banded": 0}
_SCORES_TILED_CALL_COUNTS = {"f16": 0, "bf16": 0, "f32": 0, "fp8": 0}


def prefill_consumer_call_counts() -> dict:
    """Per-route call counters (reference: indexed_attention_kernel.py:41-44)."""
    return dict(_CONSUMER_CALL_COUNTS)


def indexer_scores_call_counts() -> dict:
    """Per-operand-form call counters (reference: indexed_attention_kernel.py:45-48)."""
    return dict(_SCORES_TILED_CALL_COUNTS)


def check_status(status: torch.Tensor, what: str) -> None:
    """Raise if a kernel's bounded wait gave up (synchronises; call from tests / debug paths)."""
    if int(status.item()) != 0:
        raise _abi.MxbError(f"{what}: a device-side wait timed out (status {int(status.item())})")


# --------------------------------------------------------------------------- #
# shared launcher
# --------------------------------------------------------------------------- #

def sparse_attention(q4, comp_kv, topk3, sinks, *, pos0, window, ratio, raw_kv=None, raw_start=0,
                     scale=None, d_v=None, kv_scales=None, raw_scales=None, comp_row_start=None,
                     comp_row_count=None, n_comp=None, pos0_dev=None, out=None, out_dtype=torch.float32,
                     out_layout="bhtd", partial=False, n_splits=0, exact_fp32=False, check=False, status=None):
    """Launch the sparse attention kernel.

    q4 [B,H,T,Dqk] (any strides on the first three axes); comp_kv a flat
    [rows, Dqk] table (sequence b owns rows comp_row_start[b] .. +comp_row_count[b],
    default b*n_comp .. +n_comp); topk3 [B,T,k] int32; raw_kv [B,raw_cap,Dqk] or
    None.  Returns out [B,H,T,Dv] ("bhtd") or [B,T,H,Dv] ("bthd"); with
    ``partial=True`` returns (un-normalised fp32 out, ml [B,T,H,2]).  16-bit and int8
    tables with up to 64 heads run on the tensor-core kernel; ``exact_fp32=True`` forces
    the fp32 CUDA-core kernel (always used for float32 tables).  ``status``: a caller-owned int64 device
    buffer to use in place of the library's status word (``moespresso_b200.cycle_trace`` passes a larger one:
    an instrumented build writes its cycle stamps there).
    """
    dev = require_cuda(q4, comp_kv, topk3)
    lib = _abi.load()
    B, H, T, Dqk = (int(x) for x in q4.shape)
    q4 = last_dim_contiguous(q4)
    Dv = Dqk if d_v is None else int(d_v)
    k = int(topk3.shape[-1])
    if n_comp is None:
        n_comp = int(comp_kv.shape[0]) // B if comp_row_start is None else int(comp_kv.shape[0])
    raw_cap = 0 if raw_kv is None else int(raw_kv.shape[-2])
    if out_dtype not in (torch.float32, torch.bfloat16, torch.float16):
        raise ValueError("out_dtype must be float32, bfloat16 or float16")
    if partial:
        out_dtype = torch.float32
    if out is None:
        shape = (B, H, T, Dv) if out_layout == "bhtd" else (B, T, H, Dv)
        out = torch.empty(shape, dtype=out_dtype, device=dev)
    if out_layout == "bhtd":
        osb, osh, ost = out.stride(0), out.stride(1), out.stride(2)
    else:
        osb, ost, osh = out.stride(0), out.stride(1), out.stride(2)
    ml = torch.empty((B, T, H, 2), dtype=torch.float32, device=dev) if partial else None
    topk3 = topk3.to(torch.int32).contiguous()
    if sinks is not None:
        sinks = sinks.to(torch.float32).contiguous()
    comp_kv = comp_kv.contiguous()
    if raw_kv is not None:
        raw_kv = raw_kv.contiguous()

    a = _abi.SparseAttnArgs()
    a.q = ptr(q4); a.q_dtype = dtype_code(q4)
    a.q_stride_b, a.q_stride_h, a.q_stride_t = q4.stride(0), q4.stride(1), q4.stride(2)
    a.comp_kv = ptr(comp_kv); a.kv_dtype = dtype_code(comp_kv)
    a.comp_scales = ptr(kv_scales); a.comp_row_start = ptr(comp_row_start); a.comp_row_count = ptr(comp_row_count)
    a.n_comp = int(n_comp)
    a.raw_kv = ptr(raw_kv); a.raw_scales = ptr(raw_scales); a.raw_cap = raw_cap; a.raw_start = int(raw_start)
    a.topk = ptr(topk3); a.k = k; a.sinks = ptr(sinks)
    a.out = ptr(out); a.out_dtype = dtype_code(out)
    a.out_stride_b, a.out_stride_h, a.out_stride_t = osb, osh, ost
    a.partial_ml = ptr(ml)
    a.B, a.T, a.H, a.Dqk, a.Dv = B, T, H, Dqk, Dv
    a.scale = float(Dqk) ** -0.5 if scale is None else float(scale)
    a.pos0 = int(pos0); a.pos0_dev = ptr(pos0_dev); a.window = int(window); a.ratio = int(ratio)
    a.n_splits = int(n_splits)
    a.flags = _abi.SPARSE_EXACT_FP32 if exact_fp32 else 0
    ws = workspace(lib.mxb_sparse_attn_workspace_bytes(C.byref(a)), dev)
    a.workspace = ptr(ws); a.workspace_bytes = 0 if ws is None else ws.numel()
    own_status = status is None
    if own_status:
        status = status_word(dev) if check else None
    a.status = ptr(status)
    _abi.check(_t.launch("sparse_attn", lib.mxb_sparse_attn, a))
    if check and own_status:
        check_status(status, "sparse attention")
    return (out, ml) if partial else out


def merge_partials(o_parts, ml_parts, sinks=None, *, out_dtype=torch.float32):
    """o_parts [P,B,T,H,Dv] fp32, ml_parts [P,B,T,H,2] -> [B,T,H,Dv].  The sink joins here."""
    dev = require_cuda(o_parts, ml_parts)
    lib = _abi.load()
    P, B, T, H, Dv = (int(x) for x in o_parts.shape)
    o_parts = o_parts.contiguous(); ml_parts = ml_parts.contiguous()
    out = torch.empty((B, T, H, Dv), dtype=out_dtype, device=dev)
    if sinks is not None:
        sinks = sinks.to(torch.float32).contiguous()
    a = _abi.MergeArgs()
    a.o_parts = ptr(o_parts); a.ml_parts = ptr(ml_parts); a.sinks = ptr(sinks); a.out = ptr(out)
    a.out_dtype = dtype_code(out)
    a.out_stride_b, a.out_stride_t, a.out_stride_h = out.stride(0), out.stride(1), out.stride(2)
    a.P, a.B, a.T, a.H, a.Dv = P, B, T, H, Dv
    _abi.check(_t.launch("merge_partials", lib.mxb_merge_partials, a))
    return out


# --------------------------------------------------------------------------- #
# reference-named operators
# --------------------------------------------------------------------------- #

_KV_DTYPES = (torch.float32, torch.float16, torch.bfloat16, torch.int8)


def indexed_mixed_attention_decode(q, raw_kv, comp_kv, topk, sinks, *, pos0: int, window: int = 128,
                                   ratio: int = 4, raw_start: int = 0, scale=None, d_v=None,
                                   kv_scales=None, raw_scales=None, out_dtype=torch.float32):
    """One-token indexed mixed attention (reference: indexed_attention_kernel.py:1496-1568).

    q ``[n_heads, D]``; raw_kv ``[raw_cap, D]`` (or None: no raw window); comp_kv
    ``[n_comp, D]``; topk ``[top_k]``; sinks ``[n_heads]`` (or None).  Returns
    ``[n_heads, d_v]``.
    """
    if q.ndim != 2 or comp_kv.ndim != 2 or (raw_kv is not None and raw_kv.ndim != 2):
        raise ValueError("q, raw_kv, and comp_kv must be rank-2")
    n_heads, head_dim = int(q.shape[0]), int(q.shape[1])
    if int(comp_kv.shape[1]) != head_dim or (raw_kv is not None and int(raw_kv.shape[1]) != head_dim):
        raise ValueError("raw_kv and comp_kv width must match q")
    if topk.ndim != 1:
        raise ValueError("topk must be rank-1")
    if sinks is not None and tuple(sinks.shape) != (n_heads,):
        raise ValueError("sinks must have shape [n_heads]")
    if comp_kv.dtype not in _KV_DTYPES or (raw_kv is not None and raw_kv.dtype != comp_kv.dtype):
        raise ValueError("raw_kv and comp_kv must share one of float32, float16, bfloat16, int8")
    if raw_kv is not None:
        raw_cap = int(raw_kv.shape[0])
        if raw_cap <= 0:
            raise ValueError("raw_kv must contain at least one row")
        if not (0 <= int(raw_start) < raw_cap):
            raise ValueError("raw_start must be inside raw_kv")
    _CONSUMER_CALL_COUNTS["decode"] += 1
    out = sparse_attention(
        q[None, :, None, :], comp_kv, topk[None, None, :], sinks, pos0=pos0, window=window, ratio=ratio,
        raw_kv=None if raw_kv is None else raw_kv[None], raw_start=raw_start, scale=scale, d_v=d_v,
        kv_scales=kv_scales, raw_scales=raw_scales, out_dtype=out_dtype)
    return out[0, :, 0, :]


def _prefill_common(q, raw_kv, comp_kv, topk, sinks, *, pos0, window, ratio, raw_start, q_dtypes, what,
                    scale=None, d_v=None, route="prefill"):
    if q.ndim != 4 or comp_kv.ndim != 3 or (raw_kv is not None and raw_kv.ndim != 4):
        raise ValueError("q/raw_kv/comp_kv must have live BHLD/B1LD/BPD layouts")
    batch, n_heads, n_tokens, head_dim = (int(x) for x in q.shape)
    if batch <= 0 or n_tokens <= 0:
        raise ValueError("q must contain at least one batch and token")
    if n_heads % 8 != 0:
        raise ValueError("DS4 indexed prefill probe requires n_heads to be divisible by 8")
    if int(comp_kv.shape[0]) != batch or (raw_kv is not None and int(raw_kv.shape[0]) != batch):
        raise ValueError("raw_kv and comp_kv batch size must match q")
    if int(comp_kv.shape[-1]) != head_dim or (raw_kv is not None and int(raw_kv.shape[-1]) != head_dim):
        raise ValueError("raw_kv and comp_kv width must match q")
    if topk.ndim != 3 or int(topk.shape[0]) != batch or int(topk.shape[1]) != n_tokens:
        raise ValueError("topk must have shape [batch, tokens, top_k]")
    if sinks is not None and tuple(sinks.shape) != (n_heads,):
        raise ValueError("sinks must have shape [n_heads]")
    if q.dtype not in q_dtypes:
        raise ValueError(what)
    if int(window) < 0 or int(ratio) <= 0:
        raise ValueError("indexed prefill requires positive window and ratio")
    if raw_kv is not None:
        raw_cap = int(raw_kv.shape[2])
        if raw_cap <= 0:
            raise ValueError("raw_kv must contain at least one row")
        if not (0 <= int(raw_start) < raw_cap):
            raise ValueError("raw_start must be inside raw_kv")
        raw_kv = raw_kv[:, 0]
    _CONSUMER_CALL_COUNTS[route] += 1
    n_comp = int(comp_kv.shape[1])
    return sparse_attention(q, comp_kv.reshape(batch * n_comp, head_dim), topk, sinks, pos0=pos0,
                            window=window, ratio=ratio, raw_kv=raw_kv, raw_start=raw_start, scale=scale,
                            d_v=d_v, n_comp=n_comp)


def indexed_mixed_attention_prefill_live_f16(q, raw_kv, comp_kv, topk, sinks, *, pos0: int, window: int = 128,
                                             ratio: int = 4, raw_start: int = 0, scale=None, d_v=None):
    """Indexed prefill attention on the live ``[batch, heads, tokens, D]`` layout, 16-bit
    queries (reference: indexed_attention_kernel.py:1571-1676; bfloat16 is accepted as
    well as float16).  Returns float32 ``[batch, heads, tokens, d_v]``."""
    return _prefill_common(q, raw_kv, comp_kv, topk, sinks, pos0=pos0, window=window, ratio=ratio,
                           raw_start=raw_start, q_dtypes=(torch.float16, torch.bfloat16),
                           what="live prefill probe requires q to be float16", scale=scale, d_v=d_v)


def indexed_mixed_attention_prefill_live_f32(q, raw_kv, comp_kv, topk, sinks, *, pos0: int, window: int = 128,
                                             ratio: int = 4, raw_start: int = 0, scale=None, d_v=None):
    """float32-query form (reference: indexed_attention_kernel.py:1679-1779)."""
    return _prefill_common(q, raw_kv, comp_kv, topk, sinks, pos0=pos0, window=window, ratio=ratio,
                           raw_start=raw_start, q_dtypes=(torch.float32,),
                           what="live prefill probe requires q to be float32", scale=scale, d_v=d_v)


def indexed_mixed_attention_prefill(q, raw_kv, comp_kv, topk, sinks, *, pos0: int, window: int = 128,
                                    ratio: int = 4, raw_start: int = 0, scale=None, d_v=None):
    """Token-major probe form (reference: indexed_attention_kernel.py:2030-2108):
    q ``[tokens, heads, D]``, raw_kv ``[raw_cap, D]``, comp_kv ``[n_comp, D]``,
    topk ``[tokens, top_k]`` -> float32 ``[tokens, heads, d_v]``."""
    if q.ndim != 3 or comp_kv.ndim != 2 or (raw_kv is not None and raw_kv.ndim != 2):
        raise ValueError("q must be rank-3 and raw_kv/comp_kv rank-2")
    if topk.ndim != 2 or int(topk.shape[0]) != int(q.shape[0]):
        raise ValueError("topk must have shape [tokens, top_k]")
    out = _prefill_common(q.permute(1, 0, 2)[None], None if raw_kv is None else raw_kv[None, None],
                          comp_kv[None], topk[None], sinks, pos0=pos0, window=window, ratio=ratio,
                          raw_start=raw_start, q_dtypes=(torch.float32, torch.float16, torch.bfloat16),
                          what="q must be float32, float16 or bfloat16", scale=scale, d_v=d_v)
    return out[0].permute(1, 0, 2)


def banded_prefill_attention_live(q, raw_kv, comp_kv, topk, sinks, *, pos0: int, window: int, ratio: int,
                                  scale=None, d_v=None):
    """Banded (no indexer) prefill: ``topk`` is ``arange(pool)`` broadcast per token
    (reference: indexed_attention_kernel.py:1782-1885).  Fails closed like the reference:
    heads must be a multiple of 16 and window / ratio positive."""
    if q.ndim == 4 and int(q.shape[1]) % 16 != 0:
        raise ValueError("banded prefill requires the mma consumer: n_heads divisible by 16")
    if int(window) <= 0 or int(ratio) <= 0:
        raise ValueError("banded prefill requires positive window and ratio")
    return _prefill_common(q, raw_kv, comp_kv, topk, sinks, pos0=pos0, window=window, ratio=ratio,
                           raw_start=0, q_dtypes=(torch.float16, torch.bfloat16, torch.float32),
                           what="banded prefill requires float16 or float32 queries", scale=scale, d_v=d_v,
                           route="banded")


def indexer_q_qat_live(q):
    """Hadamard-128 + e2m1 round trip of live BHLD query rows (reference: indexed_attention_kernel.py:1989-2027).
    q float32 ``[batch, n_heads, tokens, 128]`` -> float32 of the same shape."""
    if q.ndim != 4:
        raise ValueError("q must have shape [batch, n_heads, tokens, 128]")
    if int(q.shape[0]) <= 0 or int(q.shape[2]) <= 0:
        raise ValueError("q must contain at least one batch and token")
    if int(q.shape[3]) != 128:
        raise ValueError("DS4 indexer QAT probe requires head_dim=128")
    if q.dtype != torch.float32:
        raise ValueError("q must be float32")
    from .indexer_score_kernel import indexer_qat_rows
    return indexer_qat_rows(q)


def indexer_score_operands(q, index_comp):
    """Operand form the score kernel wants (reference: indexed_attention_kernel.py:51-59):
    16-bit operands are used as they are, anything else is widened to float32."""
    if q.dtype in (torch.float16, torch.bfloat16) and index_comp.dtype == q.dtype:
        return q, index_comp
    return q.to(torch.float32), index_comp.to(torch.float32)


def indexer_scores_tiled_live(q, weights, index_comp, *, pos0: int, ratio: int = 4, exact_fp32: bool = False,
                              fp8_mma: bool = False, out=None, check: bool = False):
    """Indexer scores with the causal compressed-row mask
    (reference: indexed_attention_kernel.py:1888-1961).

    q ``[batch, heads, tokens, D]``, weights float32 ``[batch, tokens, heads]`` (all
    scale factors folded in), index_comp ``[batch, n_comp, D]``; D is 64 or 128.
    Operand pairs: both float32, both float16, both bfloat16, or 16-bit q with
    float8_e4m3fn rows.  Returns float32 ``[batch, tokens, n_comp]`` with ``-inf`` at rows
    ``>= min((pos0+t+1)//ratio, n_comp)``; ``ratio=0`` applies no mask.  ``fp8_mma=True``
    (float8 rows only) uses the FP8 tensor-core path directly: faster to feed, but its
    reduced-precision accumulation leaves ~1e-3 relative error in the scores.
    """
    if q.ndim != 4 or weights.ndim != 3 or index_comp.ndim != 3:
        raise ValueError("q, weights, and index_comp must be BHLD/BLH/BPD")
    batch, n_heads, n_tokens, head_dim = (int(x) for x in q.shape)
    n_comp = int(index_comp.shape[1])
    if batch <= 0 or n_tokens <= 0:
        raise ValueError("q must contain at least one batch and token")
    if head_dim not in (64, 128):
        raise ValueError("DS4 indexer score probe requires head_dim=128 (or 64)")
    if int(index_comp.shape[0]) != batch or int(index_comp.shape[2]) != head_dim:
        raise ValueError("index_comp must have shape [batch, n_comp, head_dim]")
    if tuple(weights.shape) != (batch, n_tokens, n_heads):
        raise ValueError("weights must have shape [batch, tokens, n_heads]")
    if weights.dtype != torch.float32:
        raise ValueError("weights must be float32")
    f8 = getattr(torch, "float8_e4m3fn", None)
    if index_comp.dtype == f8:
        if q.dtype not in (torch.float16, torch.bfloat16):
            raise ValueError("float8 index rows require float16 or bfloat16 q")
        form = "fp8"
    elif q.dtype in (torch.float16, torch.bfloat16) or index_comp.dtype in (torch.float16, torch.bfloat16):
        if q.dtype != index_comp.dtype:
            raise ValueError("half score operands require both q and index_comp as float16")
        form = "f16" if q.dtype == torch.float16 else "bf16"
    elif q.dtype == torch.float32 and index_comp.dtype == torch.float32:
        form = "f32"
    else:
        raise ValueError("q and index_comp must both be float32 or both be float16")
    if n_comp <= 0:
        raise ValueError("index_comp must contain at least one compressed row")
    _SCORES_TILED_CALL_COUNTS[form] += 1
    scores = indexer_scores(q, weights, index_comp.reshape(batch * n_comp, head_dim), n_rows=n_comp, pos0=pos0,
                            ratio=ratio, exact_fp32=exact_fp32, fp8_mma=fp8_mma, out=out, check=check)
    return scores


DIGIT_BINS = 2048   # first radix digit of the selection: the top 11 bits of the monotone score key


def scan_counts_digits(q, keys_flat, *, n_tokens: int, ratio: int, exact_fp32: bool = False, fp8_mma: bool = False) -> bool:
    """Does this call run on the decode scan, the kernel that can count the selection's first digit as it writes
    the scores (``digit_hist``)?  One token, no causal mask, FP8 keys, 16-bit q, 8 / 16 / 32 / 64 heads."""
    f8 = getattr(torch, "float8_e4m3fn", None)
    return (n_tokens == 1 and ratio == 0 and keys_flat.dtype == f8 and q.dtype in (torch.float16, torch.bfloat16)
            and int(q.shape[1]) in (8, 16, 32, 64) and int(q.shape[0]) <= 4096 and not exact_fp32 and not fp8_mma)


def indexer_scores(q, weights, keys_flat, *, n_rows, pos0=0, ratio=0, row_start=None, row_count=None,
                   exact_fp32=False, fp8_mma=False, out=None, check=False, digit_hist=None):
    """General launcher: q [B,H,T,D], weights [B,T,H] f32, keys_flat [rows_total, D].

    Uniform batches (row_start None): returns [B,T,n_rows].  Ragged batches (T == 1,
    row_start / row_count int64 / int32 device vectors): returns a flat [rows_total]
    score vector laid out like the key table.  ``digit_hist``: int32 ``[B, 2048]``, zero on entry — the decode
    scan (see ``scan_counts_digits``) adds every sequence's first-digit histogram of the scores it writes, for
    ``topk_select(..., digit_hist=)`` to start from."""
    dev = require_cuda(q, weights, keys_flat)
    lib = _abi.load()
    B, H, T, D = (int(x) for x in q.shape)
    q = last_dim_contiguous(q)
    weights = weights.contiguous()
    keys_flat = keys_flat.contiguous()
    rows_total = int(keys_flat.shape[0])
    a = _abi.IndexerScoresArgs()
    if row_start is None:
        if out is None:
            out = torch.empty((B, T, int(n_rows)), dtype=torch.float32, device=dev)
        a.score_stride_b, a.score_stride_t = out.stride(0), out.stride(1)
    else:
        if T != 1:
            raise ValueError("ragged indexer scores take one decode token per sequence")
        if out is None:
            out = torch.empty((rows_total,), dtype=torch.float32, device=dev)
        a.score_stride_b, a.score_stride_t = 0, 0
    status = status_word(dev) if check else None
    a.q = ptr(q); a.q_dtype = dtype_code(q)
    a.q_stride_b, a.q_stride_h, a.q_stride_t = q.stride(0), q.stride(1), q.stride(2)
    a.keys = ptr(keys_flat); a.key_dtype = dtype_code(keys_flat)
    a.weights = ptr(weights); a.scores = ptr(out)
    a.row_start = ptr(row_start); a.row_count = ptr(row_count)
    a.B, a.T, a.H, a.D = B, T, H, D
    a.n_rows = int(n_rows); a.rows_total = rows_total; a.pos0 = int(pos0); a.ratio = int(ratio)
    a.flags = (_abi.INDEXER_EXACT_FP32 if exact_fp32 else 0) | (_abi.INDEXER_FP8_MMA if fp8_mma else 0)
    a.status = ptr(status)
    if digit_hist is not None:
        if digit_hist.dtype != torch.int32 or tuple(digit_hist.shape) != (B, DIGIT_BINS) or not digit_hist.is_contiguous():
            raise ValueError("digit_hist must be a contiguous int32 [B, 2048] tensor")
        a.digit_hist = ptr(digit_hist)
    _abi.check(_t.launch("indexer_scores", lib.mxb_indexer_scores, a))
    if check:
        check_status(status, "indexer scores")
    return out
