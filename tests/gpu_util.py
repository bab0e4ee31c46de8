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
