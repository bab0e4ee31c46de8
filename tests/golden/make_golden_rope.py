"""Generate ``rope_golden.npz`` by RUNNING the reference's own pure-NumPy RoPE functions.

    python tests/golden/make_golden_rope.py <path to the reference checkout>

Imports ``moespresso.runtime.deepseek_v4.attention`` from the reference tree (no MLX needed) and stores the
inverse frequencies (plain and YaRN), and seeded rows before and after ``apply_rope_tail`` (forward and inverse).
"""
from __future__ import annotations

import os
import sys

import numpy as np


def main(ref_root: str) -> None:
    sys.path.insert(0, os.path.join(ref_root, "src"))
    from moespresso.runtime.deepseek_v4 import attention as ref

    rng = np.random.default_rng(20261127)
    g = {
        "inv_freq_swa": ref.rope_inverse_frequencies(ref.DS4_ROPE_DIM, ref.DS4_SWA_ROPE_BASE, None),
        "inv_freq_yarn": ref.rope_inverse_frequencies(ref.DS4_ROPE_DIM, ref.DS4_COMPRESS_ROPE_BASE, ref.DS4_YARN),
        "yarn_factor": np.float64(ref.DS4_YARN["factor"]),
        "yarn_original_seq_len": np.float64(ref.DS4_YARN["original_seq_len"]),
        "yarn_beta_fast": np.float64(ref.DS4_YARN.get("beta_fast", 32.0)),
        "yarn_beta_slow": np.float64(ref.DS4_YARN.get("beta_slow", 1.0)),
        "swa_base": np.float64(ref.DS4_SWA_ROPE_BASE),
        "compress_base": np.float64(ref.DS4_COMPRESS_ROPE_BASE),
    }
    pos = np.array([0, 1, 2, 17, 4095, 65536, 1048575], dtype=np.int64)
    x = rng.standard_normal((3, len(pos), 512)).astype(np.float32)
    g["pos"] = pos
    g["x"] = x
    g["fwd_yarn"] = ref.apply_rope_tail(x, pos, base=ref.DS4_COMPRESS_ROPE_BASE, yarn=ref.DS4_YARN)
    g["inv_yarn"] = ref.apply_rope_tail(g["fwd_yarn"], pos, base=ref.DS4_COMPRESS_ROPE_BASE, yarn=ref.DS4_YARN,
                                        inverse=True)
    g["fwd_swa"] = ref.apply_rope_tail(x, pos, base=ref.DS4_SWA_ROPE_BASE, yarn=None)
    g["angles_yarn"] = ref.rope_angles(pos, base=ref.DS4_COMPRESS_ROPE_BASE, yarn=ref.DS4_YARN)
    out = os.path.join(os.path.dirname(os.path.abspath(__file__)), "rope_golden.npz")
    np.savez_compressed(out, **g)
    print("wrote", out, {k: np.shape(v) for k, v in g.items()})


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: python " + sys.argv[0] + " <path to the reference checkout>")
    main(sys.argv[1])
