"""Seeded synthetic inputs with the shapes, sizes and value distributions of the five
benchmark configurations (host NumPy arrays; callers move them to the device).

No activations of a real model are available, so every configuration is synthetic:
``numpy.random.default_rng(seed)`` draws in the order written below.
"""
from __future__ import annotations

import numpy as np

E4M3_MAX = 448.0


def _e4m3_table() -> np.ndarray:
    t = np.zeros(256, dtype=np.float32)
    for b in range(256):
        sign = -1.0 if b & 0x80 else 1.0
        e, m = (b >> 3) & 0xF, b & 0x7
        if e == 0xF and m == 0x7:
            t[b] = np.nan
        elif e == 0:
            t[b] = sign * (m / 8.0) * 2.0 ** -6
        else:
            t[b] = sign * (1.0 + m / 8.0) * 2.0 ** (e - 7)
    return t


_E4M3 = _e4m3_table()


def to_e4m3_bits(x: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even FP8 E4M3FN encoding (saturating at +-448), as uint8."""
    import torch
    t = torch.from_numpy(np.ascontiguousarray(np.asarray(x, dtype=np.float32)))
    return t.clamp(-E4M3_MAX, E4M3_MAX).to(torch.float8_e4m3fn).view(torch.uint8).numpy()


def to_bf16_f32(x: np.ndarray) -> np.ndarray:
    """Round float32 to bfloat16 (nearest even) and return it widened back to float32."""
    u = np.asarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    r = ((u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFF0000).astype(np.uint32)
    return r.view(np.float32)


def config1(seed: int = 0, *, ctx: int = 4096, k: int = 512, H: int = 64, Dqk: int = 576, Dv: int = 512,
            Hi: int = 16, Di: int = 64) -> dict:
    """fp32 single-sequence sparse decode (the CPU-runnable case)."""
    rng = np.random.default_rng(seed)
    return dict(
        q=rng.standard_normal((H, Dqk), dtype=np.float32),
        kv=rng.standard_normal((ctx, Dqk), dtype=np.float32),
        idx_q=rng.standard_normal((Hi, Di), dtype=np.float32),
        idx_keys=rng.standard_normal((ctx, Di), dtype=np.float32),
        idx_w=(rng.standard_normal((Hi,), dtype=np.float32) / 4).astype(np.float32),
        k=k, scale=Dqk ** -0.5, d_v=Dv,
    )


def config3(seed: int = 1, *, B: int = 32, lo: int = 32768, hi: int = 131072, k: int = 2048, H: int = 64,
            Dqk: int = 576, Dv: int = 512, Hi: int = 16, Di: int = 64, lens=None) -> dict:
    """Batched sparse decode: bf16 queries, int8 latent KV with per-token fp16 scales,
    FP8-E4M3 index keys.  Float fields hold values already rounded to their storage type."""
    rng = np.random.default_rng(seed)
    lens = rng.integers(lo, hi + 1, size=B).astype(np.int64) if lens is None else np.asarray(lens, np.int64)
    B = int(lens.size)
    total = int(lens.sum())
    row_start = np.concatenate([[0], np.cumsum(lens)[:-1]]).astype(np.int64)
    q = to_bf16_f32(rng.standard_normal((B, H, Dqk), dtype=np.float32))
    kv = rng.integers(-127, 128, size=(total, Dqk), dtype=np.int8)
    scales = np.exp(rng.uniform(np.log(1e-3), np.log(1e-1), size=total)).astype(np.float16)
    idx_q = to_bf16_f32(rng.standard_normal((B, Hi, Di), dtype=np.float32))
    idx_key_bits = to_e4m3_bits(rng.standard_normal((total, Di), dtype=np.float32))
    idx_w = (rng.standard_normal((B, Hi), dtype=np.float32) / 4).astype(np.float32)
    return dict(lens=lens, row_start=row_start, q=q, kv=kv, kv_scales=scales, idx_q=idx_q,
                idx_key_bits=idx_key_bits, idx_w=idx_w, k=k, scale=Dqk ** -0.5, d_v=Dv)


def e4m3_bits_to_f32(bits: np.ndarray) -> np.ndarray:
    return _E4M3[np.asarray(bits, dtype=np.uint8)]


def config2(seed: int = 0, *, S: int = 8192, Hq: int = 16, Hkv: int = 2, D: int = 256) -> dict:
    """Qwen-style causal GQA prefill, bf16 (values already rounded to bf16)."""
    rng = np.random.default_rng(seed)
    mk = lambda *shape: to_bf16_f32(0.5 * rng.standard_normal(shape, dtype=np.float32))
    q, k, v = mk(S, Hq, D), mk(S, Hkv, D), mk(S, Hkv, D)
    gate = to_bf16_f32(rng.standard_normal((S, Hq, D), dtype=np.float32))
    return dict(q=q, k=k, v=v, gate=gate, scale=1.0 / 16.0)


def config4(seed: int = 2, *, T: int = 4096, history: int = 131072, ratio: int = 4, k: int = 2048, H: int = 64,
            Dqk: int = 576, Dv: int = 512, Hi: int = 16, Di: int = 64) -> dict:
    """Chunked sparse prefill over ratio-4 compressed KV, bf16."""
    rng = np.random.default_rng(seed)
    R = history // ratio
    return dict(
        pos0=history - T, ratio=ratio, k=k, scale=Dqk ** -0.5, d_v=Dv,
        kv=to_bf16_f32(rng.standard_normal((R, Dqk), dtype=np.float32)),
        q=to_bf16_f32(rng.standard_normal((T, H, Dqk), dtype=np.float32)),
        idx_q=to_bf16_f32(rng.standard_normal((T, Hi, Di), dtype=np.float32)),
        idx_keys=to_bf16_f32(rng.standard_normal((R, Di), dtype=np.float32)),
        idx_w=(rng.standard_normal((T, Hi), dtype=np.float32) / 4).astype(np.float32),
    )
