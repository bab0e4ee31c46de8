"""DS4 decode-side cache operators with the reference's names
(reference: src/moespresso/runtime/deepseek_v4/decode_attention_kernel.py).

``fp8_kv_prefix_rows``   E4M3FN round trip of the non-rotary prefix of 512-wide compressed-KV rows (:587-619)

The attention part of ``fused_decode_sdpa`` (:733) and the score + select part of ``fused_decode_prep`` (:669) are
``indexed_attention_kernel.indexed_mixed_attention_decode`` and ``decode_step.sparse_decode_step``; their rotary
prologue / epilogue is not part of this package.
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
