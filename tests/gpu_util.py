"""Helpers shared by the GPU parity tests."""
import numpy as np
import pytest
import torch

from moespresso_b200 import synth


def need_gpu():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    return torch.device("cuda:0")


def dev(x, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(x)).cuda()
    return t if dtype is None else t.to(dtype)


def fp8_from_bits(bits):
    return torch.from_numpy(np.ascontiguousarray(bits)).cuda().view(torch.float8_e4m3fn)


def max_abs(a, b):
    a = a.detach().float().cpu().numpy().astype(np.float64) if isinstance(a, torch.Tensor) else np.asarray(a, np.float64)
    b = b.detach().float().cpu().numpy().astype(np.float64) if isinstance(b, torch.Tensor) else np.asarray(b, np.float64)
    return float(np.max(np.abs(a - b))) if a.size else 0.0


def bf16_round(x):
    return synth.to_bf16_f32(np.asarray(x, np.float32))


def f16_round(x):
    return np.asarray(x, np.float32).astype(np.float16).astype(np.float32)


def first_digit_hist(scores):
    """2048-bin histogram of the top 11 bits of the selection keys of finite scores (NumPy): the key of x is its
    bit pattern with the sign bit set for x >= 0 (-0 counts as +0) and all bits flipped for x < 0."""
    x = np.asarray(scores, dtype=np.float32)
    x = x[np.isfinite(x)] + np.float32(0.0)
    b = x.view(np.uint32)
    key = np.where(b & np.uint32(0x80000000), ~b, b | np.uint32(0x80000000))
    return np.bincount((key >> np.uint32(21)).astype(np.int64), minlength=2048).astype(np.int32)
