"""Generate ``fp8kv_golden.npz`` by RUNNING the reference's own pure-NumPy FP8 KV round trip.

Run once in a container that has the reference checkout:

    python tests/golden/make_golden_fp8kv.py <path to the reference checkout>

It imports ``moespresso.correctness.deepseek_v4.compressor_diff`` from the reference tree (imports without
MLX) and stores seeded 512-wide rows with the output of its ``_fp8_kv_round`` and, for the value table,
``_e4m3fn_dequant``.  ``tests/test_oracle_golden.py`` replays the vectors against ``oracle/``.
"""
from __future__ import annotations

import os
import sys

import numpy as np


def main(ref_root: str) -> None:
    sys.path.insert(0, os.path.join(ref_root, "src"))
    from moespresso.correctness.deepseek_v4 import compressor_diff as ref

    rng = np.random.default_rng(20261126)
    rows = np.concatenate([
        rng.standard_normal((24, 512)),                                  # plain activations
        rng.standard_normal((8, 512)) * 300.0,                           # large: scales above 1
        rng.standard_normal((8, 512)) * 1e-3,                            # small: near the 1e-4 floor
        rng.standard_normal((4, 512)) * 1e-6,                            # below the floor
        np.zeros((1, 512)),
    ]).astype(np.float32)
    rows[5, 64:128] = 0.0                                                # one all-zero block
    rows[6, :64] = np.linspace(-448.0, 448.0, 64)                        # a block whose scale is exactly 1
    g = {
        "rows": rows,
        "rounded": ref._fp8_kv_round(rows),
        "table": ref.E4M3FN_VALUES.astype(np.float32),
    }
    probe = np.concatenate([rng.uniform(-500, 500, 4096), rng.uniform(-1, 1, 4096) * 0.02]).astype(np.float32)
    g["dequant_in"] = probe
    g["dequant_out"] = ref._e4m3fn_dequant(probe)
    out = os.path.join(os.path.dirname(os.path.abspath(__file__)), "fp8kv_golden.npz")
    np.savez_compressed(out, **g)
    print("wrote", out, {k: v.shape for k, v in g.items()})


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: python " + sys.argv[0] + " <path to the reference checkout>")
    main(sys.argv[1])
