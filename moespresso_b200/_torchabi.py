"""Glue between torch CUDA tensors and the C ABI: dtype codes, pointers, streams,
argument structures.  Torch is used for device memory and streams only."""
from __future__ import annotations

import ctypes as C

import torch

from . import _abi

_DTYPES = {
    torch.float32: _abi.F32,
    torch.float16: _abi.F16,
    torch.bfloat16: _abi.BF16,
    torch.int8: _abi.I8,
}
if hasattr(torch, "float8_e4m3fn"):
    _DTYPES[torch.float8_e4m3fn] = _abi.F8E4M3


def dtype_code(t: torch.Tensor) -> int:
    try:
        return _DTYPES[t.dtype]
    except KeyError:
        raise ValueError(f"unsupported dtype {t.dtype}") from None


def require_cuda(*tensors) -> torch.device:
    dev = None
    for t in tensors:
        if t is None:
            continue
        if not isinstance(t, torch.Tensor) or not t.is_cuda:
            raise RuntimeError(
                "moespresso_b200 operators run on CUDA tensors only; there is no CPU path")
        if dev is None:
            dev = t.device
        elif t.device != dev:
            raise ValueError("all tensors must live on the same CUDA device")
    if dev is None:
        raise RuntimeError("moespresso_b200 operators need at least one CUDA tensor")
    return dev


def ptr(t) -> int | None:
    return None if t is None else t.data_ptr()


def stream_ptr() -> C.c_void_p:
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def workspace(nbytes: int, device) -> torch.Tensor | None:
    if nbytes <= 0:
        return None
    return torch.empty(int(nbytes), dtype=torch.uint8, device=device)


def status_word(device) -> torch.Tensor:
    return torch.zeros(1, dtype=torch.int32, device=device)


def last_dim_contiguous(t: torch.Tensor) -> torch.Tensor:
    return t if t.stride(-1) == 1 else t.contiguous()


# Optional per-entry-point device timing: set TIMER to a dict and every launch records a
# pair of CUDA events on the current stream around the C call (name -> [(start, end), ...]).
TIMER = None


def launch(name: str, fn, args) -> int:
    if TIMER is None:
        return fn(C.byref(args), stream_ptr())
    e0 = torch.cuda.Event(enable_timing=True)
    e1 = torch.cuda.Event(enable_timing=True)
    e0.record()
    rc = fn(C.byref(args), stream_ptr())
    e1.record()
    TIMER.setdefault(name, []).append((e0, e1))
    return rc
