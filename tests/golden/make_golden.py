"""Generate ``ds4_golden.npz`` by RUNNING the reference's own pure-NumPy code.

Run once in a container that has the reference checkout:

    python tests/golden/make_golden.py <path to the reference checkout>

It imports ``moespresso.runtime.deepseek_v4.attention`` and
``moespresso.correctness.deepseek_v4.attention_diff`` from the reference tree
(both import without MLX), feeds them seeded inputs and stores inputs and
outputs.  The resulting file travels with the repository; the reference does
not.  ``tests/test_oracle_golden.py`` replays the vectors against ``oracle/``.
"""
from __future__ import annotations

import os
import sys

import numpy as np


def main(ref_root: str) -> None:
    sys.path.insert(0, os.path.join(ref_root, "src"))
    from moespresso.runtime.deepseek_v4 import attention as ref
    from moespresso.correctness.deepseek_v4 import attention_diff as refdiff

    rng = np.random.default_rng(20261125)
    g: dict[str, np.ndarray] = {}

    # visibility tables
    qpos = np.array([0, 2, 3, 4, 7, 127, 128, 511, 4095, 65535, 65536, 1048575], dtype=np.int64)
    pool = np.arange(40, dtype=np.int64)
    for ratio in (4, 128):
        g[f"vis_r{ratio}"] = ref.compressed_visibility(qpos, pool, ratio)
        g[f"viscount_r{ratio}"] = ref.visible_compressed_count(qpos, ratio)
    g["vis_qpos"] = qpos
    g["vis_pool"] = pool

    # sink softmax
    for i, (n, dv) in enumerate([(1, 2), (7, 5), (33, 16)]):
        s = rng.normal(size=(3, n)) * 3
        v = rng.normal(size=(n, dv))
        sk = rng.normal(size=(3,))
        if i == 1:
            sk[0] = -np.inf
        g[f"sink{i}_scores"], g[f"sink{i}_values"], g[f"sink{i}_sinks"] = s, v, sk
        g[f"sink{i}_out"] = ref.sink_softmax_attention(s, v, sk)

    # indexer scores + causal top-k, with exact ties and masked rows
    for i, (T, H, R, D, k, ratio, q0) in enumerate(
        [(5, 4, 24, 8, 6, 4, 40), (3, 16, 64, 64, 16, 4, 250), (4, 2, 12, 4, 12, 4, 5)]
    ):
        raw = rng.normal(size=(T, H, R))
        if i == 2:
            raw = np.round(raw)          # many ties
        w = rng.normal(size=(T, H)) / 4
        if i == 2:
            w = np.ones((T, H))
        qp = q0 + np.arange(T, dtype=np.int64)
        pool_i = np.arange(R, dtype=np.int64)
        g[f"idx{i}_raw"], g[f"idx{i}_w"], g[f"idx{i}_qpos"] = raw, w, qp
        g[f"idx{i}_meta"] = np.array([D, H, k, ratio], dtype=np.int64)
        g[f"idx{i}_weighted"] = ref.indexer_weighted_scores(raw, w, index_head_dim=D, n_heads=H)
        g[f"idx{i}_causal"] = ref.causal_indexer_scores(raw, w, qp, pool_i, ratio,
                                                        index_head_dim=D, n_heads=H)
        g[f"idx{i}_topk"] = ref.causal_indexer_topk(raw, w, qp, pool_i, ratio, topk=k,
                                                    index_head_dim=D, n_heads=H)

    # windowed raw attention with sinks (fp32 NumPy reference of the raw-window part)
    for i, (T, H, D, window) in enumerate([(9, 4, 32, 4), (12, 8, 64, 0), (6, 2, 16, 128)]):
        qc = rng.normal(size=(T, H, D)).astype(np.float32)
        kv = rng.normal(size=(T, D)).astype(np.float32)
        sk = rng.normal(size=(H,)).astype(np.float32)
        g[f"raw{i}_q"], g[f"raw{i}_kv"], g[f"raw{i}_sinks"] = qc, kv, sk
        g[f"raw{i}_meta"] = np.array([window], dtype=np.int64)
        g[f"raw{i}_out"] = refdiff.raw_prefill_attention(
            qc, kv, sk, scale=float(D) ** -0.5, window=window, qk_half=False, value_half=False)

    out = os.path.join(os.path.dirname(os.path.abspath(__file__)), "ds4_golden.npz")
    np.savez_compressed(out, **g)
    print("wrote", out, len(g), "arrays")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: python " + sys.argv[0] + " <path to the reference checkout>")
    main(sys.argv[1])
