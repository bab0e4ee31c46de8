"""Times (or just runs) the q8 decode attention over a synthetic affine-q8 cache.

    python -m moespresso_b200.qwen.q8_decode_probe [keys=131072] [splits=128] [repeats=50]

Builds a cache of ``keys`` rows (2 KV heads, 16 query heads, head_dim 256, bf16 scales and biases) with
``QuantizedKVCache.update_and_fetch`` and calls ``sdpa_decode_q8`` on it: three eager calls, then, when
``repeats`` > 0, a CUDA graph of one call (decode kernel + merge) replayed ``repeats`` times between two events.
With ``repeats`` = 0 it is a short program to put under a profiler.  Needs a GPU.
"""
from __future__ import annotations

import sys

import torch

from .full_attention import QuantizedKVCache, sdpa_decode_q8


def main(argv) -> int:
    keys = int(argv[1]) if len(argv) > 1 else 131072
    splits = int(argv[2]) if len(argv) > 2 else 128
    repeats = int(argv[3]) if len(argv) > 3 else 50
    dev = torch.device("cuda")
    gen = torch.Generator(device=dev).manual_seed(5)
    hq, hkv, d = 16, 2, 256
    rows = lambda n: (0.5 * torch.randn(1, hkv, n, d, generator=gen, device=dev, dtype=torch.float32)).to(torch.bfloat16)
    cache = QuantizedKVCache(hkv, d, keys)
    for lo in range(0, keys, 16384):
        n = min(16384, keys - lo)
        cache.update_and_fetch(rows(n), rows(n))
    q = torch.randn((1, hq, 1, d), generator=gen, device=dev, dtype=torch.float32)
    call = lambda: sdpa_decode_q8(q, *cache.keys, *cache.values, d ** -0.5, splits=splits)
    for _ in range(3):
        out = call()
    torch.cuda.synchronize()
    if repeats <= 0:
        print(f"{keys} keys, {splits} splits: ran; sum |out| = {float(out.float().abs().sum()):.4f}")
        return 0
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        call()
    for _ in range(3):
        graph.replay()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(repeats):
        graph.replay()
    b.record()
    torch.cuda.synchronize()
    us = a.elapsed_time(b) / repeats * 1e3
    nbytes = 2 * hkv * keys * (d + 2 * (d // 64) * 2)
    print(f"{keys} keys, {splits} splits: {us:.1f} us per call (decode kernel + merge), {nbytes / us / 1e3:.0f} GB/s of cache bytes")
    return 0


if __name__ == "__main__":
    sys.exit(main(sys.argv))
