"""Cycle trace of one CTA of the tensor-core sparse attention kernel (a development aid).

``csrc/sparse_attn_tc.cu`` carries ``TRS(row, unit)`` stamps that compile to nothing in the regular library.
Built with ``-DMXB_TRACE_SP`` they store ``clock64()`` of CTA 0 into a 32 x 16 table of int64 behind the caller's
``status`` pointer: row = which event, column = unit (the first 16 units of the CTA).  This module builds that
variant next to the regular library (``moespresso_b200/build/trace/``, same flags plus the macro), runs one of the
two benchmark shapes through it and prints the table relative to the CTA's start:

    python -m moespresso_b200.cycle_trace c3     # batch 32 decode, int8 tables, top-k 2048, 4 splits per sequence
    python -m moespresso_b200.cycle_trace c4     # 592 tokens of a prefill chunk, bf16 table of 32768 rows

Rows (per unit unless noted): 0 gather warps reach the unit, 1 its row buffer is free, 2 all its gathers are
issued, 3 logit issuer sees the first slab, 4 logit MMAs committed, 5 softmax sees S^T, 6 before / 7 after the
CTA-wide vote on the reference maxima, 12 P^T stored, 8 P^T handed over, 9 value issuer sees P^T, 10 value MMAs
committed, 13 / 15 widening warps start / finish the unit, 16-27 the widening warps' halves and blocks,
11 (columns 0-4): CTA start, prologue done, softmax loop done, last P V done, CTA end.

The numbers come from one CTA of one launch and include the cost of the stamps themselves (a store per event):
use them to see which role waits for which, not as a timing of the kernel (``bench.py`` times that).
Needs a GPU; the traced library is never used by the package itself.
"""
from __future__ import annotations

import os
import subprocess
import sys

from . import _build

TRACE_DIR = os.path.join(_build.HERE, "build", "trace")
TRACE_LIB = os.path.join(TRACE_DIR, "libmoespresso_b200_trace_sp.so")
EVENTS = {0: "gather_top", 1: "rowbuf_free", 2: "gathers_issued", 3: "qk_first_slab", 4: "qk_commit", 5: "softmax_s_ready",
          6: "vote_in", 7: "vote_out", 12: "p_stored", 8: "p_ready", 9: "pv_sees_p", 10: "pv_commit", 13: "widen_start",
          15: "widen_end"}


def build_trace_library() -> str:
    """Regular objects + ``sparse_attn_tc.cu`` recompiled with ``-DMXB_TRACE_SP``; returns the library's path."""
    _build.build()
    os.makedirs(TRACE_DIR, exist_ok=True)
    nvcc = _build._nvcc()
    flags = [f for f in _build.NVCC_FLAGS if f not in ("-Xptxas", "-v")]
    obj = os.path.join(TRACE_DIR, "sparse_attn_tc.o")
    subprocess.run([nvcc, *flags, "-DMXB_TRACE_SP", "-c", os.path.join(_build.CSRC, "sparse_attn_tc.cu"), "-o", obj],
                   check=True)
    objs = [os.path.join(_build.HERE, "build", s.replace(".cu", ".o")) for s in _build.SOURCES if s != "sparse_attn_tc.cu"]
    subprocess.run([nvcc, "-shared", "-o", TRACE_LIB, *objs, obj, "-gencode", "arch=compute_100a,code=sm_100a",
                    "-lcudart_static", "-Xcompiler", "-fPIC"], check=True)
    return TRACE_LIB


def trace(case: str):
    """Runs ``case`` ("c3" or "c4") through the traced library; returns (table [32,16] of cycles relative to the CTA's
    start as a NumPy array, number of units to show, kernel + merge time in ms)."""
    import numpy as np
    import torch
    lib = TRACE_LIB if os.path.exists(TRACE_LIB) else build_trace_library()
    _build.LIB = lib                       # this process talks to the traced library only
    _build.is_current = lambda: True
    from . import synth
    from .deepseek_v4 import indexed_attention_kernel as iak
    dev = torch.device("cuda")
    table = torch.zeros(32 * 16, dtype=torch.int64, device=dev)
    if case == "c3":
        c = synth.config3(seed=1)
        kv, sc = torch.from_numpy(c["kv"]).to(dev), torch.from_numpy(c["kv_scales"]).to(dev)
        rs, rc = torch.from_numpy(c["row_start"]).to(dev), torch.from_numpy(c["lens"].astype(np.int32)).to(dev)
        q = torch.from_numpy(c["q"]).to(dev).to(torch.bfloat16)
        rng = np.random.default_rng(0)
        ids = torch.from_numpy(np.stack([np.sort(rng.choice(int(n), 2048, replace=False)) for n in c["lens"]])
                               .astype(np.int32)).to(dev)

        def run(status):
            return iak.sparse_attention(q[:, :, None, :], kv, ids[:, None, :], None, pos0=0, window=0, ratio=0,
                                        scale=c["scale"], d_v=512, kv_scales=sc, comp_row_start=rs, comp_row_count=rc,
                                        n_comp=int(c["lens"].max()), n_splits=4, status=status)
        units = 8
    elif case == "c4":
        T, R, k = 592, 32768, 2048
        g = torch.Generator(device=dev)
        g.manual_seed(2)
        q = torch.randn((T, 64, 576), device=dev, generator=g).to(torch.bfloat16)
        kv = torch.randn((R, 576), device=dev, generator=g).to(torch.bfloat16)
        ids = torch.stack([torch.sort(torch.randperm(R - 4096, device=dev, generator=g)[:k])[0] for _ in range(T)]).to(torch.int32)

        def run(status):
            return iak.sparse_attention(q.permute(1, 0, 2)[None], kv, ids[None], None, pos0=131072 - T, window=0, ratio=4,
                                        scale=576 ** -0.5, d_v=512, n_comp=R, out_layout="bthd", status=status)
        units = 16
    else:
        raise ValueError("case must be 'c3' or 'c4'")
    for _ in range(3):
        run(table)
    torch.cuda.synchronize()
    table.zero_()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)   # the traced run finds none of its rows in L2,
    flush.zero_()                                                    # as inside a step that has just scanned the keys
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    run(table)
    e1.record()
    torch.cuda.synchronize()
    t = table.cpu().numpy().reshape(32, 16)
    return np.where(t != 0, t - t[11, 0], 0), units, e0.elapsed_time(e1)


def main(argv) -> int:
    if len(argv) != 2 or argv[1] not in ("c3", "c4", "build"):
        print(__doc__)
        return 2
    if argv[1] == "build":
        print(build_trace_library())
        return 0
    t, units, ms = trace(argv[1])
    print(f"{argv[1]}: kernel (+ merge) {ms * 1e3:.1f} us with the stamps; cycles of CTA 0 relative to its start")
    print("prologue done %d | softmax loop done %d | last P V done %d | CTA end %d" % tuple(int(t[11, i]) for i in (1, 2, 3, 4)))
    if t[11, 5:8].any():
        print("cluster merge: (m, l) exchanged %d | blocks pushed %d | blocks arrived %d" % tuple(int(t[11, i]) for i in (5, 6, 7)))
    order = [0, 1, 2, 3, 4, 5, 6, 7, 12, 8, 9, 10, 13, 15]
    print("unit " + " ".join(f"{EVENTS[r]:>15s}" for r in order))
    for u in range(units):
        print(f"{u:4d} " + " ".join(f"{int(t[r, u]):15d}" for r in order))
    if t[28:31].any():
        print("units whose reference maxima moved: column maxima done, previous P V and sums done, O^T rescaled")
        for u in range(units):
            if t[28, u]:
                print(f"{u:4d} {int(t[29, u]):10d} {int(t[30, u]):10d} {int(t[28, u]):10d}")
    if t[16:28].any():
        print("widening warp 0, per unit: rows 16-27 (half starts, preloads done, block stores done)")
        for u in range(min(units, 8)):
            print(f"{u:4d} " + " ".join(f"{int(t[r, u]):8d}" for r in range(16, 28)))
    return 0


if __name__ == "__main__":
    sys.exit(main(sys.argv))
