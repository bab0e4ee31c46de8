"""ctypes binding of ``libmoespresso_b200.so`` (the C ABI of include/moespresso_b200.h).

The structures below mirror the header field for field.  There is no fallback:
if the shared library is missing and cannot be built, importing an operator
raises, and every operator raises when no CUDA device is present.
"""
from __future__ import annotations

import ctypes as C
import os

from . import _build

F32, F16, BF16, F8E4M3, I8 = 0, 1, 2, 3, 4
INDEXER_EXACT_FP32 = 1
INDEXER_FP8_MMA = 2
SPARSE_EXACT_FP32 = 1

_p = C.c_void_p
_i32 = C.c_int32
_i64 = C.c_int64
_f32 = C.c_float


class IndexerScoresArgs(C.Structure):
    _fields_ = [
        ("q", _p), ("q_dtype", _i32), ("q_stride_b", _i64), ("q_stride_h", _i64), ("q_stride_t", _i64),
        ("keys", _p), ("key_dtype", _i32), ("weights", _p), ("scores", _p),
        ("score_stride_b", _i64), ("score_stride_t", _i64),
        ("row_start", _p), ("row_count", _p),
        ("B", _i32), ("T", _i32), ("H", _i32), ("D", _i32),
        ("n_rows", _i64), ("rows_total", _i64), ("pos0", _i64),
        ("ratio", _i32), ("flags", _i32), ("status", _p), ("digit_hist", _p),
    ]


class TopkArgs(C.Structure):
    _fields_ = [
        ("scores", _p), ("row_stride", _i64), ("row_start", _p), ("row_count", _p), ("out_ids", _p),
        ("rows", _i32), ("n", _i64), ("k", _i32), ("workspace", _p), ("workspace_bytes", _i64), ("digit_hist", _p),
    ]


class IndexerQatArgs(C.Structure):
    _fields_ = [("x", _p), ("x_dtype", _i32), ("out", _p), ("n_rows", _i64), ("width", _i32)]


class ScoreTailArgs(C.Structure):
    _fields_ = [
        ("scores", _p), ("weights_raw", _p), ("w_dtype", _i32), ("params", _p), ("out", _p), ("H", _i32),
        ("capacity", _i64), ("scale", C.c_float),
    ]


class Fp8KvRowsArgs(C.Structure):
    _fields_ = [("x", _p), ("out", _p), ("n_rows", _i64), ("width", _i32), ("mode", _i32)]


class QuantizeKvInt8Args(C.Structure):
    _fields_ = [("x", _p), ("x_dtype", _i32), ("q", _p), ("scales", _p), ("n_rows", _i64), ("width", _i32)]


class AffineQ8Args(C.Structure):
    _fields_ = [("x", _p), ("x_dtype", _i32), ("x_row_stride", _i64), ("packed", _p), ("scales", _p), ("biases", _p),
                ("sb_dtype", _i32), ("n_rows", _i64), ("width", _i32)]


class SdpaDecodeQ8Args(C.Structure):
    _fields_ = [("q", _p), ("q_dtype", _i32), ("k_packed", _p), ("k_scales", _p), ("k_biases", _p),
                ("v_packed", _p), ("v_scales", _p), ("v_biases", _p), ("sb_dtype", _i32), ("head_stride_rows", _i64),
                ("P", _i32), ("Hq", _i32), ("Hkv", _i32), ("D", _i32), ("scale", C.c_float), ("n_splits", _i32),
                ("o_parts", _p), ("ml_parts", _p)]


class RopeTailArgs(C.Structure):
    _fields_ = [
        ("x", _p), ("out", _p), ("x_dtype", _i32), ("positions", _p), ("inv_freq", _p), ("n_rows", _i64),
        ("seq_len", _i32), ("width", _i32), ("rope_dim", _i32), ("inverse", _i32), ("half_chain", _i32),
    ]


class SparseAttnArgs(C.Structure):
    _fields_ = [
        ("q", _p), ("q_dtype", _i32), ("q_stride_b", _i64), ("q_stride_h", _i64), ("q_stride_t", _i64),
        ("comp_kv", _p), ("kv_dtype", _i32), ("comp_scales", _p), ("comp_row_start", _p),
        ("comp_row_count", _p), ("n_comp", _i64),
        ("raw_kv", _p), ("raw_scales", _p), ("raw_cap", _i32), ("raw_start", _i32),
        ("topk", _p), ("k", _i32), ("sinks", _p),
        ("out", _p), ("out_dtype", _i32), ("out_stride_b", _i64), ("out_stride_h", _i64), ("out_stride_t", _i64),
        ("partial_ml", _p),
        ("B", _i32), ("T", _i32), ("H", _i32), ("Dqk", _i32), ("Dv", _i32), ("scale", _f32),
        ("pos0", _i64), ("pos0_dev", _p), ("window", _i32), ("ratio", _i32), ("n_splits", _i32), ("flags", _i32),
        ("workspace", _p), ("workspace_bytes", _i64), ("status", _p),
    ]


class MergeArgs(C.Structure):
    _fields_ = [
        ("o_parts", _p), ("ml_parts", _p), ("sinks", _p), ("out", _p), ("out_dtype", _i32),
        ("out_stride_b", _i64), ("out_stride_h", _i64), ("out_stride_t", _i64),
        ("P", _i32), ("B", _i32), ("T", _i32), ("H", _i32), ("Dv", _i32),
    ]


class FlashPrefillArgs(C.Structure):
    _fields_ = [
        ("q", _p), ("q_stride_s", _i64), ("q_stride_h", _i64),
        ("k", _p), ("k_stride_s", _i64), ("k_stride_h", _i64),
        ("v", _p), ("v_stride_s", _i64), ("v_stride_h", _i64),
        ("gate", _p), ("gate_stride_s", _i64), ("gate_stride_h", _i64),
        ("out", _p), ("out_stride_s", _i64), ("out_stride_h", _i64),
        ("dtype", _i32), ("S", _i32), ("Skv", _i32), ("Hq", _i32), ("Hkv", _i32), ("D", _i32),
        ("scale", _f32), ("workspace", _p), ("workspace_bytes", _i64), ("status", _p),
    ]


class RangeCandidatesArgs(C.Structure):
    _fields_ = [("scores", _p), ("ids", _p), ("out_scores", _p), ("out_ids", _p), ("k", _i32), ("row_lo", _i64)]


class RangeLocalIdsArgs(C.Structure):
    _fields_ = [("pos", _p), ("cand_ids", _p), ("cand_rank_stride", _i64), ("out", _p), ("k", _i32),
                ("row_lo", _i64), ("rows_local", _i64)]


EXPORTS = {
    "mxb_abi_version": (C.c_int, []),
    "mxb_last_error": (C.c_char_p, []),
    "mxb_kernel_launches": (C.c_int64, []),
    "mxb_copy_h2d_async": (C.c_int, [_p, _p, _i64, _p]),
    "mxb_indexer_scores": (C.c_int, [C.POINTER(IndexerScoresArgs), _p]),
    "mxb_indexer_qat": (C.c_int, [C.POINTER(IndexerQatArgs), _p]),
    "mxb_score_tail": (C.c_int, [C.POINTER(ScoreTailArgs), _p]),
    "mxb_fp8_kv_rows": (C.c_int, [C.POINTER(Fp8KvRowsArgs), _p]),
    "mxb_quantize_kv_int8": (C.c_int, [C.POINTER(QuantizeKvInt8Args), _p]),
    "mxb_rope_tail": (C.c_int, [C.POINTER(RopeTailArgs), _p]),
    "mxb_affine_q8_quantize": (C.c_int, [C.POINTER(AffineQ8Args), _p]),
    "mxb_affine_q8_dequantize": (C.c_int, [C.POINTER(AffineQ8Args), _p]),
    "mxb_sdpa_decode_q8": (C.c_int, [C.POINTER(SdpaDecodeQ8Args), _p]),
    "mxb_range_candidates": (C.c_int, [C.POINTER(RangeCandidatesArgs), _p]),
    "mxb_range_local_ids": (C.c_int, [C.POINTER(RangeLocalIdsArgs), _p]),
    "mxb_topk_workspace_bytes": (_i64, [_i32, _i64, _i32]),
    "mxb_topk_select": (C.c_int, [C.POINTER(TopkArgs), _p]),
    "mxb_topk_select_static": (C.c_int, [C.POINTER(TopkArgs), _p]),
    "mxb_sparse_attn_workspace_bytes": (_i64, [C.POINTER(SparseAttnArgs)]),
    "mxb_sparse_attn": (C.c_int, [C.POINTER(SparseAttnArgs), _p]),
    "mxb_merge_partials": (C.c_int, [C.POINTER(MergeArgs), _p]),
    "mxb_flash_prefill_workspace_bytes": (_i64, [C.POINTER(FlashPrefillArgs)]),
    "mxb_flash_prefill": (C.c_int, [C.POINTER(FlashPrefillArgs), _p]),
}

_lib = None


def lib_path() -> str:
    return _build.LIB


def load():
    """Load (building first when a compiler is at hand and the sources changed)."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(_build.LIB) or (not _build.is_current() and _can_build()):
        _build.build()
    lib = C.CDLL(_build.LIB)
    for name, (res, args) in EXPORTS.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    if lib.mxb_abi_version() != 1:
        raise RuntimeError("libmoespresso_b200.so has an unexpected ABI version")
    _lib = lib
    return lib


def _can_build() -> bool:
    import shutil
    return bool(shutil.which("nvcc") or os.path.exists("/usr/local/cuda/bin/nvcc"))


class MxbError(RuntimeError):
    pass


def check(rc: int) -> None:
    """0 passes; contract violations raise ValueError with the library's message
    (the reference raises ValueError from its Python wrappers); anything else
    raises MxbError."""
    if rc == 0:
        return
    msg = load().mxb_last_error().decode("utf-8", "replace")
    if rc == -1:
        raise ValueError(msg)
    raise MxbError(f"moespresso_b200 error {rc}: {msg}")
