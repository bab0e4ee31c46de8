#!/usr/bin/env python
"""Benchmark of the sparse-decode attention hot path (and, as extras, the other configurations).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Headline workload: the batched DS-V4-shaped sparse decode step — batch 32, context ~ U[32K, 128K] per
sequence, top-k 2048, bf16 queries over an int8 latent KV cache with per-token fp16 scales, FP8-E4M3 index
keys, 64 heads x 576 (V = first 512), indexer 16 heads x 64, seed 1.  One "step" = indexer score -> top-k ->
indexed sparse attention for the whole batch (one decoded token per sequence), so tokens/s = batch / step
time.  With N > 1 every rank holds its own batch of 32 sequences (sequence sharding, no collective on the
data path): weak scaling.

Prints ONE JSON line on rank 0.
* `value` is timed with the inputs resident in HBM: windows of K steps (one CUDA graph per step) between two
  CUDA events, repeated until the timed region is at least 250 ms; the median window is reported (the minimum
  beside it), the maximum over ranks of every window.
* `e2e` goes through the public Python operator with the step's inputs in pinned host memory and the result
  read back to the host inside the timed region.  The latent KV and index-key tables are the decode cache
  (state that lives on the device between steps, like weights); the per-step inputs are the queries, indexer
  queries and head weights.
* `roofline` describes the whole step: the bytes the step has to move (index keys once, the selected rows,
  queries in, outputs out; scores are not counted because a fused selection need not materialise them) over
  the step time, against the measured and the nominal HBM bandwidth; `extras.kernels` breaks it down.
* `extras.c5a` / `extras.c5b` are the multi-GPU configurations: 256 sequences of 131072 rows dealt to the
  ranks (strong scaling of one fixed batch, no collective), and one sequence of 1,048,576 rows range-sharded
  over the ranks (two NCCL all-gathers and a log-sum-exp merge per step), checked bit for bit against the
  single-GPU selection on rank 0.
"""
from __future__ import annotations

import argparse
import datetime
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "sparse_decode_attn_tokens_per_s"
UNIT = "tokens/s"
WORKLOAD = "c3_batched_sparse_decode_b32_ctx32k-128k_topk2048_int8kv_fp8idx"
H, DQK, DV, HI, DI = 64, 576, 512, 16, 64
MIN_TIMED_MS = 250.0
QUERY_SETS = 4   # batches of queries taken in rotation by consecutive steps (4 x 38 MB of selected rows > L2)


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return float(d["hbm_gbs"]), float(d["bf16_tflops"]), "measured"
    return 6650.0, 1590.0, "fallback"


def workload_config(batch: int, rows_total: int, topk: int, world: int) -> dict:
    """The `config` object; both arms print the same keys."""
    return {"workload": WORKLOAD, "batch_per_gpu": batch, "rows_total_per_gpu": rows_total, "topk": topk,
            "heads": H, "d_qk": DQK, "d_v": DV, "indexer": "16x64 fp8-e4m3 keys", "kv": "int8 + fp16 per-token scale",
            "parallelism": f"sequence-sharded x{world}, no collective",
            "l2": ("inputs (1.7 GB per GPU) exceed L2, no flush needed; consecutive steps take 4 query sets in rotation, so "
                   "the rows a step gathers are not the ones the last steps left in L2")}


def step_bytes(lens, k: int) -> int:
    """Bytes one decode step has to move: every index key once, the selected int8 rows with their scales,
    q and the indexer q in, the bf16 output out.  Scores are not counted (a fused selection keeps them on chip)."""
    lens = np.asarray(lens, dtype=np.int64)
    per_seq = lens * DI + min(k, int(lens.max())) * (DQK + 2) + H * DQK * 2 + H * DV * 2 + HI * DI * 2
    return int(per_seq.sum())


class ClockSampler:
    """nvidia-smi samples during the timed region (read-only query)."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.rows = []
        self.proc = None
        self.gpu = gpu_index

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "50",
                 "-i", str(self.gpu)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.time(), [x.strip() for x in line.split(",")]))

    def stop(self, t_lo: float | None = None, t_hi: float | None = None) -> dict:
        """Summary of the samples taken in [t_lo, t_hi] (all samples if the window holds none)."""
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        inside = [r for ts, r in self.rows if t_lo is not None and t_lo <= ts <= t_hi]
        rows = inside or [r for _, r in self.rows]
        sm, smax, reasons = [], [], set()
        for r in rows:
            try:
                sm.append(float(r[1])); smax.append(float(r[2]))
            except Exception:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(smax) if smax else None,
                "reasons": sorted(reasons), "samples": len(sm), "samples_inside_timed_region": len(inside)}


# --------------------------------------------------------------------------- #
# CPU arm (the oracle's float32 NumPy formulation, timed)
# --------------------------------------------------------------------------- #

def cpu_decode_batch(c, seqs) -> float:
    """Seconds the NumPy formulation needs for the given sequences of workload `c`."""
    from moespresso_b200 import synth
    from oracle import ds4
    t0 = time.perf_counter()
    for b in seqs:
        s, n = int(c["row_start"][b]), int(c["lens"][b])
        keys = synth.e4m3_bits_to_f32(c["idx_key_bits"][s:s + n])
        ds4.sparse_decode_step(c["q"][b], c["kv"][s:s + n], c["idx_q"][b], keys, c["idx_w"][b], k=c["k"],
                               scale=c["scale"], d_v=c["d_v"], kv_scales=c["kv_scales"][s:s + n], dtype=np.float32)
    return time.perf_counter() - t0


def run_reference(args):
    """The reference formulation of the path on the host cores (NumPy; MLX, which the
    reference uses, has no Linux build here).  Rank 0 only."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    from moespresso_b200 import synth
    cores = len(os.sched_getaffinity(0))
    c = synth.config3(seed=1)
    B = int(c["lens"].size)
    sample = list(range(B))
    for _ in range(args.warmup):
        cpu_decode_batch(c, sample[:4])
    t = 0.0
    for _ in range(args.steps):
        t += cpu_decode_batch(c, sample)
    ms = t / args.steps * 1e3
    val = B / (ms / 1e3)
    line = {
        "impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(B, int(c["lens"].sum()), int(c["k"]), max(1, args.gpus)),
        "cpu_baseline": {"value": val, "unit": UNIT, "cores": cores, "kind": "port",
                         "sample": f"all {B} sequences of one rank's batch per step, NumPy float32 (BLAS threads = {cores})"},
        "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


# --------------------------------------------------------------------------- #
# GPU arm
# --------------------------------------------------------------------------- #

def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-extras", action="store_true", help="skip the secondary workloads (c1, c2, c4, c5)")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-graph", action="store_true", help="launch the step eagerly instead of as a CUDA graph")
    ap.add_argument("--small", action="store_true", help="reduced sizes (for profiling captures only)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
        return

    import torch
    import torch.distributed as dist

    from moespresso_b200 import _abi, synth
    from moespresso_b200.deepseek_v4.attention import topk_select
    from moespresso_b200.deepseek_v4.decode_step import LatentCache, SparseDecodePlan, sparse_decode_step
    from moespresso_b200.deepseek_v4.indexed_attention_kernel import indexer_scores, sparse_attention

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: there is no CPU path for the product kernels")
    lib = _abi.load()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=60))
    W = max(args.warmup, 3)
    K = max(args.steps, 1)

    if args.small:
        # 8 long sequences: index keys (~133 MB) still exceed L2, everything on the device stays under 2 GB
        c = synth.config3(seed=1 + rank, B=8, lo=240000, hi=280000)
    else:
        c = synth.config3(seed=1 + rank)
    B = int(c["lens"].size)
    total = int(c["lens"].sum())
    kk, scale, d_v = int(c["k"]), float(c["scale"]), int(c["d_v"])
    cache = LatentCache(
        kv=torch.from_numpy(c["kv"]).to(dev), kv_scales=torch.from_numpy(c["kv_scales"]).to(dev),
        idx_keys=torch.from_numpy(c["idx_key_bits"]).to(dev).view(torch.float8_e4m3fn),
        row_start=torch.from_numpy(c["row_start"]).to(dev),
        row_count=torch.from_numpy(c["lens"].astype(np.int32)).to(dev), max_rows=int(c["lens"].max()))
    q_h = torch.from_numpy(c["q"]).to(torch.bfloat16).pin_memory()
    iq_h = torch.from_numpy(c["idx_q"]).to(torch.bfloat16).pin_memory()
    iw_h = torch.from_numpy(c["idx_w"]).pin_memory()
    q_d, iq_d, iw_d = q_h.to(dev), iq_h.to(dev), iw_h.to(dev)
    out_h = torch.empty((B, H, d_v), dtype=torch.bfloat16).pin_memory()   # the step's result in the activation type

    plan = SparseDecodePlan(cache, heads=H, d_qk=DQK, idx_heads=HI, idx_dim=DI, k=kk, scale=scale, d_v=d_v,
                            q_dtype=torch.bfloat16, out_dtype=torch.bfloat16, graph=not args.no_graph)
    plan.load_inputs(q_d, iq_d, iw_d)
    # Consecutive timed steps take different query sets, in rotation: the rows a step selects (38 MB) and gathers are
    # then not the ones the previous steps left in L2 (the key scan marks its reads evict-first, so what the other
    # kernels touched would otherwise still be there when the same inputs came round again).
    rng_q = np.random.default_rng(1000 + rank)
    host_sets = [(q_h, iq_h, iw_h)]
    plans = [plan]
    for _ in range(QUERY_SETS - 1):
        qj = torch.from_numpy(rng_q.standard_normal((B, H, DQK), dtype=np.float32)).to(torch.bfloat16).pin_memory()
        iqj = torch.from_numpy(rng_q.standard_normal((B, HI, DI), dtype=np.float32)).to(torch.bfloat16).pin_memory()
        iwj = torch.from_numpy((rng_q.standard_normal((B, HI), dtype=np.float32) / 4).astype(np.float32)).pin_memory()
        pj = SparseDecodePlan(cache, heads=H, d_qk=DQK, idx_heads=HI, idx_dim=DI, k=kk, scale=scale, d_v=d_v,
                              q_dtype=torch.bfloat16, out_dtype=torch.bfloat16, graph=not args.no_graph)
        pj.load_inputs(qj.to(dev), iqj.to(dev), iwj.to(dev))
        host_sets.append((qj, iqj, iwj))
        plans.append(pj)
    turn = [0]

    def rotating_step():
        plans[turn[0] % QUERY_SETS].launch()
        turn[0] += 1

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(xs):
        t = torch.tensor(list(xs), dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return [float(x) for x in t.tolist()]

    def timed_windows(step, k_steps: int, min_ms: float, max_windows: int = 400):
        """Windows of `k_steps` calls of `step` between two events, repeated until `min_ms` of timed region;
        every rank runs the same number of windows.  Returns ms per step of every window (max over ranks)."""
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
        ev[0].record()
        for _ in range(k_steps):
            step()
        ev[1].record()
        torch.cuda.synchronize()
        first = max_over_ranks([ev[0].elapsed_time(ev[1])])[0]
        n = int(min(max_windows, max(1, np.ceil(min_ms / max(first, 1e-3)))))
        events = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(n)]
        barrier()
        for a, b in events:
            a.record()
            for _ in range(k_steps):
                step()
            b.record()
        barrier()
        return [x / k_steps for x in max_over_ranks([a.elapsed_time(b) for a, b in events])]

    sampler = ClockSampler(local)
    sampler.start()
    for _ in range(max(W, QUERY_SETS)):
        rotating_step()
    barrier()
    # ---- timed region: windows of K steps, inputs resident in HBM
    t_lo = time.time()
    windows = timed_windows(rotating_step, K, MIN_TIMED_MS)
    t_hi = time.time()
    ms_step = float(np.median(windows))
    ms_min = float(np.min(windows))

    # ---- per-stage device time: each entry point captured as its own CUDA graph and replayed between two events
    # (no host gaps inside the timed region).  The index keys (167 MB) exceed L2 between replays; the attention
    # stage replays the same ids, so its 38 MB of gathered rows stay L2-resident across replays, whereas the timed
    # steps above rotate their query sets and gather rows that L2 does not hold: the stage times add up to a few
    # microseconds less than the step.
    launches0 = int(lib.mxb_kernel_launches())
    out_e, ids_e, sc_e = sparse_decode_step(q_d, iq_d, iw_d, cache, k=kk, scale=scale, d_v=d_v, return_ids=True,
                                            return_scores=True, out_dtype=torch.bfloat16)
    torch.cuda.synchronize()
    kernels_per_step = int(lib.mxb_kernel_launches()) - launches0   # counted by the library itself

    def stage_us(fn) -> float:
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(3):
                fn()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            fn()
        for _ in range(3):
            g.replay()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(5 * K):
            g.replay()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / (5 * K) * 1e3

    # The scan counts the selection's first radix digit (plan.digit_hist), so the selection cannot be replayed on
    # its own (it clears the counters it starts from): it is timed as (scan + selection) - scan.
    fused = plan.digit_hist is not None
    hist_a = torch.zeros_like(plan.digit_hist) if fused else None   # only ever added to: the scan's work is the same
    hist_b = torch.zeros_like(plan.digit_hist) if fused else None   # counted and cleared once per replay

    def scan(hist):
        return indexer_scores(iq_d[:, :, None, :], iw_d[:, None, :].contiguous(), cache.idx_keys, n_rows=cache.max_rows,
                              row_start=cache.row_start, row_count=cache.row_count, digit_hist=hist)

    stage = {"indexer_scores": stage_us(lambda: scan(hist_a))}
    if fused:
        both = stage_us(lambda: topk_select(scan(hist_b), kk, valid=cache.row_count, row_start=cache.row_start,
                                            n=cache.max_rows, digit_hist=hist_b))
        stage["topk_select"] = both - stage["indexer_scores"]
    else:
        stage["topk_select"] = stage_us(lambda: topk_select(sc_e, kk, valid=cache.row_count, row_start=cache.row_start,
                                                            n=cache.max_rows))
    stage["sparse_attn"] = stage_us(lambda: sparse_attention(
        q_d[:, :, None, :], cache.kv, ids_e[:, None, :], None, pos0=0, window=0, ratio=0, scale=scale, d_v=d_v,
        kv_scales=cache.kv_scales, comp_row_start=cache.row_start, comp_row_count=cache.row_count,
        n_comp=cache.max_rows, out_dtype=torch.bfloat16))
    # The same stage with its rows coming from HBM, as inside the timed steps: one graph per query set (each with the
    # ids its own step selected), replayed in rotation.
    attn_graphs = []
    for pj in plans:
        if pj.ids is None:
            break
        gj = torch.cuda.CUDAGraph()
        fnj = lambda pj=pj: sparse_attention(
            pj.q[:, :, None, :], cache.kv, pj.ids[:, None, :], None, pos0=0, window=0, ratio=0, scale=scale, d_v=d_v,
            kv_scales=cache.kv_scales, comp_row_start=cache.row_start, comp_row_count=cache.row_count,
            n_comp=cache.max_rows, out_dtype=torch.bfloat16)
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            fnj()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        with torch.cuda.graph(gj):
            fnj()
        attn_graphs.append(gj)
    stage_rotating = None
    if len(attn_graphs) == QUERY_SETS:
        for gj in attn_graphs:
            gj.replay()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        reps = 5 * K
        a.record()
        for i in range(reps):
            attn_graphs[i % QUERY_SETS].replay()
        b.record()
        torch.cuda.synchronize()
        stage_rotating = a.elapsed_time(b) / reps * 1e3

    # ---- end to end: pinned host inputs -> device -> step -> result back on the host, every step
    in_hs = []
    for pj, (qj, iqj, iwj) in zip(plans, host_sets):
        in_h, (qv, iqv, iwv) = pj.host_buffer()   # the step's inputs live in one pinned buffer: one H2D copy
        qv.copy_(qj)
        iqv.copy_(iqj)
        iwv.copy_(iwj)
        in_hs.append(in_h)

    def e2e_step():
        j = turn[0] % QUERY_SETS
        turn[0] += 1
        out_h.copy_(plans[j].run_packed(in_hs[j]), non_blocking=True)
        torch.cuda.current_stream().synchronize()   # the caller consumes the result of every step

    for _ in range(2):
        e2e_step()
    e2e_windows = timed_windows(e2e_step, K, MIN_TIMED_MS)
    ms_e2e = float(np.median(e2e_windows))
    clocks = sampler.stop(t_lo, t_hi)

    hbm, tf, which = measured_peaks()
    # ---- roofline of the whole step (HBM-bound: key scan + row gather); per-kernel figures beside it
    alg_bytes = step_bytes(c["lens"], kk)
    achieved = alg_bytes / (ms_step * 1e-3) / 1e9
    kbytes = {
        # FP8 keys read once, fp32 scores written once
        "indexer_scores": total * DI + total * 4 + B * (HI * DI * 2 + HI * 4),
        # scores read once, ids written
        "topk_select": total * 4 + B * kk * 4,
        # selected int8 rows + scales, ids, q in, bf16 output out
        "sparse_attn": B * (kk * (DQK + 2) + kk * 4 + H * DQK * 2 + H * d_v * 2),
    }
    kernels = {name: {"us": stage[name], "algorithmic_bytes": kbytes[name],
                      "GBs": kbytes[name] / (stage[name] * 1e-6) / 1e9,
                      "frac_of_measured_hbm": kbytes[name] / (stage[name] * 1e-6) / 1e9 / hbm}
               for name in stage}
    dominant = max(stage, key=stage.get)
    kernel_names = {"indexer_scores": "indexer_decode_kernel<64, 16 heads>", "topk_select": "topk_cluster_kernel",
                    "sparse_attn": "sparse_attn_tc_kernel<int8 kv, bf16 q> (splits merged inside a cluster)"}
    # DRAM traffic from ncu captures on the --small case (profiles/), scaled by the units each launch processes:
    # the key scan reads 65.0 B and writes 4.8 B per key row; the attention kernel reads 787 B per gathered row
    # (576-byte rows start at any 64-byte offset: sector rounding) plus q; the selection re-reads the scores
    traffic = total * (65.0 + 4.8) + total * 4.0 + B * (kk * 787.0 + H * DQK * 2 + H * d_v * 2)

    line = {
        "metric": METRIC, "value": world * B / (ms_step * 1e-3), "unit": UNIT, "n_gpus": world, "steps": K,
        "warmup": W, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic",
        "config": workload_config(B, total, kk, world),
        "timing": {"windows": len(windows), "steps_per_window": K, "timed_region_ms": float(np.sum(windows)) * K,
                   "ms_per_step_median": ms_step, "ms_per_step_min": ms_min},
        "e2e": {"value": world * B / (ms_e2e * 1e-3), "unit": UNIT,
                "h2d_bytes_per_step": int(in_h.numel()),
                "d2h_bytes_per_step": int(out_h.numel() * out_h.element_size()), "ms_per_step": ms_e2e,
                "windows": len(e2e_windows)},
        "gpu_launches": kernels_per_step * K * len(windows),
        "launch": (f"one CUDA graph per step ({kernels_per_step} kernels of this library)" if not args.no_graph
                   else f"eager ({kernels_per_step} kernels of this library per step)"),
        "stage_us": stage,
        "sparse_attn_us_rows_from_hbm": stage_rotating,   # the attention stage replayed over the four query sets in turn
        "stage_note": ("each entry point replayed as its own CUDA graph; topk_select = (scan + selection) - scan, because the "
                       "scan counts the selection's first radix digit; sparse_attn replays the same ids (L2-warm rows); "
                       "sparse_attn_us_rows_from_hbm replays it over the four query sets in turn"
                       if fused else "each entry point replayed as its own CUDA graph; sparse_attn replays the same ids (L2-warm rows; "
                               "inside the timed steps, which rotate query sets, the rows come from HBM: sparse_attn_us_rows_from_hbm "
                               "is the same stage replayed over the four query sets in turn)"),
        "roofline": {"bound": "hbm", "kernel": kernel_names[dominant], "scope": "whole decode step",
                     "achieved": achieved, "peak": hbm, "unit": "GB/s", "frac": achieved / hbm, "peak_source": which,
                     "traffic": traffic, "algorithmic_bytes": alg_bytes, "launch_us": ms_step * 1e3,
                     "frac_of_nominal_8TBs": achieved / 8000.0},
        "clocks": clocks,
    }
    if args.small:
        line["config"]["workload"] = WORKLOAD + "_SMALL"

    extras = {"kernels": kernels}
    failed = False
    if not args.no_extras and not args.small:
        del plan, plans, pj, cache
        torch.cuda.empty_cache()
        if rank == 0:
            extras.update(run_extras(torch, dev, tf))
        # The secondary multi-GPU workloads synchronise the ranks through the rendezvous store (host side), not
        # through NCCL: a rank that fails says so there, the others stop waiting at once and skip what is left,
        # and the headline line is still printed (a CUDA error is sticky: nothing on the device can follow it).
        store = dist.distributed_c10d._get_default_store() if world > 1 else None
        tags = iter(range(1 << 20))

        def soft_barrier():
            torch.cuda.synchronize()
            if store is None:
                return
            key = f"mxb/bar/{next(tags)}"
            store.add(key, 1)
            t0 = time.time()
            while int(store.add(key, 0)) < world:
                if store.check(["mxb/failed"]):
                    raise RuntimeError("another rank failed in a secondary workload")
                if time.time() - t0 > 300:
                    raise RuntimeError("a rank did not reach the barrier within 300 s")
                time.sleep(0.0005)

        def soft_max(xs):
            if store is None:
                return [float(x) for x in xs]
            key = f"mxb/max/{next(tags)}"
            store.set(f"{key}/{rank}", json.dumps([float(x) for x in xs]))
            soft_barrier()
            cols = [json.loads(store.get(f"{key}/{r}")) for r in range(world)]
            return [max(c[i] for c in cols) for i in range(len(cols[0]))]

        for name, fn in (("c5a", lambda: run_c5a(torch, dist, dev, rank, world, hbm, soft_barrier, soft_max)),
                         ("c5b", lambda: run_c5b(torch, dist, dev, rank, world, soft_barrier, soft_max))):
            if failed:
                extras[name + "_error"] = "skipped: an earlier secondary workload failed"
                continue
            try:
                soft_barrier()                     # nobody starts a workload that a failed rank will never join
                extras[name] = fn()
            except Exception as e:   # report, do not hide
                extras[name + "_error"] = repr(e)
                failed = True
                if store is not None:
                    store.set("mxb/failed", str(rank))
    line["extras"] = extras
    if rank == 0 and not args.no_cpu:
        cores = len(os.sched_getaffinity(0))
        seqs = list(range(B))
        t = cpu_decode_batch(c, seqs)
        line["cpu_baseline"] = {"value": len(seqs) / t, "unit": UNIT, "cores": cores, "kind": "port",
                                "sample": f"one pass over all {len(seqs)} sequences of the batch, NumPy float32"}
    if rank == 0:
        print(json.dumps(line), flush=True)
    if failed:
        os._exit(0)   # the device (or a peer) is in an error state: no orderly teardown of CUDA / NCCL is possible
    if world > 1:
        dist.destroy_process_group()


# --------------------------------------------------------------------------- #
# multi-GPU configurations (also run at N = 1)
# --------------------------------------------------------------------------- #

def _device_tables(torch, dev, n_rows: int, seed: int):
    """int8 latent rows, fp16 scales (log-uniform in [1e-3, 1e-1]) and FP8 index keys, generated on the device."""
    g = torch.Generator(device=dev).manual_seed(seed)
    kv = torch.randint(-127, 128, (n_rows, DQK), generator=g, device=dev, dtype=torch.int8)
    u = torch.rand(n_rows, generator=g, device=dev)
    scales = torch.exp(u * (np.log(1e-1) - np.log(1e-3)) + np.log(1e-3)).to(torch.float16)
    keys = torch.empty((n_rows, DI), dtype=torch.float8_e4m3fn, device=dev)
    step = 1 << 22
    for lo in range(0, n_rows, step):   # in pieces: the fp32 normal draw of all keys at once would take 8.6 GB
        hi = min(lo + step, n_rows)
        keys[lo:hi] = torch.randn((hi - lo, DI), generator=g, device=dev).to(torch.float8_e4m3fn)
    return kv, scales, keys


def run_c5a(torch, dist, dev, rank, world, hbm, barrier, max_over_ranks) -> dict:
    """256 sequences x 131072 rows, seed 3, dealt to the ranks by context length: one fixed batch, no collective
    (strong scaling).  Every rank generates and holds only its own sequences."""
    from moespresso_b200 import dist as mdist
    from moespresso_b200.deepseek_v4.decode_step import LatentCache, SparseDecodePlan
    Bt, L, kk = 256, 131072, 2048
    mine = mdist.assign_sequences([L] * Bt, world)[rank]
    nb = len(mine)
    kv, scales, keys = _device_tables(torch, dev, nb * L, 3000 + rank)
    cache = LatentCache(kv=kv, kv_scales=scales, idx_keys=keys,
                        row_start=torch.arange(nb, device=dev, dtype=torch.int64) * L,
                        row_count=torch.full((nb,), L, dtype=torch.int32, device=dev), max_rows=L)
    g = torch.Generator(device=dev).manual_seed(3)
    q = torch.randn((Bt, H, DQK), generator=g, device=dev).to(torch.bfloat16)[mine]
    iq = torch.randn((Bt, HI, DI), generator=g, device=dev).to(torch.bfloat16)[mine]
    iw = (torch.randn((Bt, HI), generator=g, device=dev) / 4)[mine]
    plan = SparseDecodePlan(cache, heads=H, d_qk=DQK, idx_heads=HI, idx_dim=DI, k=kk, scale=DQK ** -0.5, d_v=DV,
                            q_dtype=torch.bfloat16, out_dtype=torch.bfloat16)
    plan.load_inputs(q, iq, iw)
    for _ in range(3):
        plan.launch()
    barrier()
    reps = 10
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(reps):
        plan.launch()
    b.record()
    barrier()
    ms = max_over_ranks([a.elapsed_time(b) / reps])[0]
    per_gpu_bytes = step_bytes([L] * nb, kk)
    out = {"batch": Bt, "rows_per_sequence": L, "sequences_on_this_rank": nb, "topk": kk, "scaling": "strong",
           "collective": "none", "us_per_step": ms * 1e3, "tokens_per_s": Bt / (ms * 1e-3),
           "per_gpu_GBs": per_gpu_bytes / (ms * 1e-3) / 1e9,
           "per_gpu_frac_of_measured_hbm": per_gpu_bytes / (ms * 1e-3) / 1e9 / hbm}
    del plan, cache, kv, scales, keys
    torch.cuda.empty_cache()
    return out


def run_c5b(torch, dist, dev, rank, world, barrier, max_over_ranks) -> dict:
    """One sequence of 1,048,576 rows, seed 3, range-sharded over the ranks: local scores and top-k, all-gather of
    the candidates, identical global selection, local partial attention, all-gather of the partials, merge.
    Every rank draws the same table and keeps its own range; rank 0 also runs the single-GPU step on the whole
    table and the results are compared (selection bit for bit)."""
    from moespresso_b200 import dist as mdist
    from moespresso_b200.deepseek_v4.decode_step import LatentCache, sparse_decode_step
    R, kk = 1 << 20, 2048
    kv, scales, keys = _device_tables(torch, dev, R, 3)          # the same draw on every rank
    g = torch.Generator(device=dev).manual_seed(33)
    q = torch.randn((H, DQK), generator=g, device=dev).to(torch.bfloat16)
    iq = torch.randn((HI, DI), generator=g, device=dev).to(torch.bfloat16)
    iw = torch.randn((HI,), generator=g, device=dev) / 4
    lo, hi = mdist.row_range(R, world, rank, align=128)
    shard = mdist.RangeShard(kv=kv[lo:hi], kv_scales=scales[lo:hi], idx_keys=keys[lo:hi], row_lo=lo)
    out = {"rows": R, "topk": kk, "rows_on_this_rank": hi - lo, "collective": "2 x all_gather (NCCL) per step"
           if world > 1 else "none (one rank)"}
    if world == 1 and not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29541")
        dist.init_process_group("nccl", rank=0, world_size=1, device_id=dev,
                                timeout=datetime.timedelta(seconds=60))
        own_group = True
    else:
        own_group = False
    # correctness against the single-GPU step (eager driver, which can report the attended ids)
    res, attended = mdist.range_sharded_decode_step(q, iq, iw, shard, k=kk, scale=DQK ** -0.5, d_v=DV, return_ids=True)
    counts = [torch.zeros(1, dtype=torch.int64, device=dev) for _ in range(world)]
    dist.all_gather(counts, torch.tensor([attended.numel()], dtype=torch.int64, device=dev))
    padded = torch.full((kk,), -1, dtype=torch.int64, device=dev)
    padded[:attended.numel()] = attended
    gathered = [torch.empty_like(padded) for _ in range(world)]
    dist.all_gather(gathered, padded)
    if rank == 0:
        cache = LatentCache(kv=kv, kv_scales=scales, idx_keys=keys, row_start=torch.zeros(1, dtype=torch.int64, device=dev),
                            row_count=torch.tensor([R], dtype=torch.int32, device=dev), max_rows=R)
        ref, ref_ids = sparse_decode_step(q[None], iq[None], iw[None], cache, k=kk, scale=DQK ** -0.5, d_v=DV,
                                          return_ids=True)
        got = torch.cat([t[:int(n.item())] for t, n in zip(gathered, counts)])
        out["ids_equal_single_gpu"] = bool(got.numel() == kk and
                                           torch.equal(torch.sort(got)[0].to(torch.int32), ref_ids[0]))
        out["max_abs_vs_single_gpu"] = float((res.float() - ref[0].float()).abs().max().item())
    plan = mdist.RangeDecodePlan(shard, heads=H, d_qk=DQK, idx_heads=HI, idx_dim=DI, k=kk, scale=DQK ** -0.5, d_v=DV)
    for _ in range(5):
        plan.step(q, iq, iw)
    barrier()
    reps = 20
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(reps):
        plan.step(q, iq, iw)
    b.record()
    barrier()
    out["us_per_step"] = max_over_ranks([a.elapsed_time(b) / reps])[0] * 1e3
    phases = plan.timed_step(q, iq, iw, reps=reps)   # device time of the three local phases and the two collectives
    for name, us in zip(("candidates_us", "allgather_candidates_us", "partial_attention_us", "allgather_partials_us",
                         "merge_us"), max_over_ranks(phases)):
        out[name] = us
    if rank == 0:
        out["plan_max_abs_vs_eager"] = float((plan.out.float() - res.float()).abs().max().item())
    if own_group:
        dist.destroy_process_group()
    del plan, shard, kv, scales, keys
    torch.cuda.empty_cache()
    return out


def run_extras(torch, dev, tf_peak) -> dict:
    """Secondary workloads, single GPU: config 1 (fp32 decode, latency), config 2 (Qwen prefill), config 4 (chunk of
    sparse prefill)."""
    from moespresso_b200 import synth
    from moespresso_b200.deepseek_v4.decode_step import LatentCache, sparse_decode_step
    from moespresso_b200.qwen.full_attention import sdpa_fa_prefill
    ex = {}

    def timeit(fn, iters=20, warm=3):
        for _ in range(warm):
            fn()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(iters):
            fn()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / iters

    try:
        c = synth.config1()
        t = lambda x: torch.from_numpy(x).to(dev)
        cache = LatentCache(kv=t(c["kv"]), kv_scales=None, idx_keys=t(c["idx_keys"]),
                            row_start=torch.zeros(1, dtype=torch.int64, device=dev),
                            row_count=torch.tensor([4096], dtype=torch.int32, device=dev), max_rows=4096)
        q, iq, iw = t(c["q"])[None], t(c["idx_q"])[None], t(c["idx_w"])[None]
        ms = timeit(lambda: sparse_decode_step(q, iq, iw, cache, k=c["k"], scale=c["scale"], d_v=c["d_v"]))
        ex["c1_fp32_decode_step_eager_us"] = ms * 1e3          # one Python call per operator: host-bound
        from moespresso_b200.deepseek_v4.decode_step import SparseDecodePlan
        plan = SparseDecodePlan(cache, heads=int(q.shape[1]), d_qk=int(q.shape[2]), idx_heads=int(iq.shape[1]),
                                idx_dim=int(iq.shape[2]), k=int(c["k"]), scale=c["scale"], d_v=c["d_v"],
                                q_dtype=torch.float32)
        plan.load_inputs(q, iq, iw)
        ms = timeit(plan.launch, iters=200)
        ex["c1_fp32_decode_step_us"] = ms * 1e3                # the same step as one CUDA graph launch
    except Exception as e:  # report, do not hide
        ex["c1_error"] = repr(e)
    try:
        c = synth.config2()
        t = lambda x: torch.from_numpy(x).to(dev).to(torch.bfloat16)
        q, k, v, g = t(c["q"]), t(c["k"]), t(c["v"]), t(c["gate"])
        ms = timeit(lambda: sdpa_fa_prefill(q, k, v, c["scale"], gate=g, layout="lhd"), iters=10)
        S, Hq, D = q.shape
        flops = 4.0 * Hq * D * S * (S + 1) / 2
        ex["c2_qwen_prefill_ms"] = ms
        ex["c2_qwen_prefill_tflops_causal"] = flops / (ms * 1e-3) / 1e12
        ex["c2_frac_of_bf16_peak"] = ex["c2_qwen_prefill_tflops_causal"] / tf_peak
    except Exception as e:
        ex["c2_error"] = repr(e)
    try:
        # Qwen q8 KV cache (the served form of configuration 2): one 4096-token chunk over a 28672-token affine-q8
        # past (context 32768 after the chunk), and one decode token over 131072 cached keys.
        from moespresso_b200.qwen.full_attention import (QuantizedKVCache, dequantize_affine_q8, quantize_affine_q8,
                                                         sdpa_decode_q8, sdpa_fa_prefill_q8)
        g8 = torch.Generator(device=dev).manual_seed(5)
        rn8 = lambda *sh: (0.5 * torch.randn(*sh, generator=g8, device=dev, dtype=torch.float32)).to(torch.bfloat16)
        Hq8, Hkv8, D8, L8, P8, PD8 = 16, 2, 256, 4096, 28672, 131072
        cache8 = QuantizedKVCache(Hkv8, D8, PD8)
        for lo in range(0, PD8, 16384):
            cache8.update_and_fetch(rn8(1, Hkv8, 16384, D8), rn8(1, Hkv8, 16384, D8))
        past_k = tuple(x[:, :, :P8] for x in cache8.keys)
        past_v = tuple(x[:, :, :P8] for x in cache8.values)
        q8, gate8 = rn8(1, Hq8, L8, D8), rn8(1, L8, Hq8 * D8)
        sk = dequantize_affine_q8(*quantize_affine_q8(rn8(1, Hkv8, L8, D8)))
        sv = dequantize_affine_q8(*quantize_affine_q8(rn8(1, Hkv8, L8, D8)))
        ms = timeit(lambda: sdpa_fa_prefill_q8(q8, *past_k, *past_v, sk, sv, D8 ** -0.5, gate=gate8), iters=5)
        flops = 4.0 * Hq8 * D8 * (L8 * P8 + L8 * (L8 + 1) / 2)
        ex["qwen_q8_prefill_chunk_ms"] = ms
        ex["qwen_q8_prefill_chunk_tflops"] = flops / (ms * 1e-3) / 1e12
        ex["qwen_q8_prefill_chunk_frac_of_bf16_peak"] = ex["qwen_q8_prefill_chunk_tflops"] / tf_peak
        qd = torch.randn((1, Hq8, 1, D8), generator=g8, device=dev, dtype=torch.float32)
        dec = lambda: sdpa_decode_q8(qd, *cache8.keys, *cache8.values, D8 ** -0.5, splits=128)
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(3):
                dec()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        g_dec = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g_dec):          # decode kernel + merge as one graph launch: device time, no host gaps
            dec()
        ms = timeit(g_dec.replay, iters=50)
        q8_bytes = 2 * Hkv8 * PD8 * (D8 + 2 * (D8 // 64) * 2)     # packed words + bf16 scales and biases, keys and values
        ex["qwen_q8_decode_us"] = ms * 1e3
        ex["qwen_q8_decode_GBs"] = q8_bytes / (ms * 1e-3) / 1e9
        ex["qwen_q8_decode_frac_of_measured_hbm"] = ex["qwen_q8_decode_GBs"] / measured_peaks()[0]
        del cache8, past_k, past_v
    except Exception as e:
        ex["qwen_q8_error"] = repr(e)
    try:
        # config 4: 4096-token chunk over 32768 ratio-4 compressed rows, top-k 2048 per token, bf16.
        # Inputs are generated on the device (same shapes and N(0,1) distributions as synth.config4).
        from moespresso_b200 import _torchabi
        from moespresso_b200.deepseek_v4.prefill_step import sparse_prefill_step
        T, R, kk = 4096, 32768, 2048
        g = torch.Generator(device=dev).manual_seed(2)
        rn = lambda *sh: torch.randn(*sh, generator=g, device=dev, dtype=torch.float32)
        kv, q = rn(R, DQK).to(torch.bfloat16), rn(T, H, DQK).to(torch.bfloat16)
        iq, ik, iw = rn(T, HI, DI).to(torch.bfloat16), rn(R, DI).to(torch.bfloat16), rn(T, HI) / 4
        run = lambda: sparse_prefill_step(q, kv, iq, ik, iw, pos0=131072 - T, ratio=4, k=kk, scale=DQK ** -0.5,
                                          d_v=DV, window=0)
        run(); torch.cuda.synchronize()
        _torchabi.TIMER = {}
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(); run(); b.record(); torch.cuda.synchronize()
        timer, _torchabi.TIMER = _torchabi.TIMER, None
        tot = {name: sum(x.elapsed_time(y) for x, y in evs) for name, evs in timer.items()}
        ex["c4_chunk_ms"] = a.elapsed_time(b)
        ex["c4_entry_point_ms"] = tot
        if tot.get("indexer_scores"):
            ex["c4_indexer_tflops"] = 2.0 * T * HI * DI * R / (tot["indexer_scores"] * 1e-3) / 1e12
            ex["c4_indexer_frac_of_bf16_peak"] = ex["c4_indexer_tflops"] / tf_peak
        if tot.get("sparse_attn"):
            ex["c4_sparse_attn_tflops"] = 2.0 * T * H * kk * (DQK + DV) / (tot["sparse_attn"] * 1e-3) / 1e12
            ex["c4_sparse_attn_frac_of_bf16_peak"] = ex["c4_sparse_attn_tflops"] / tf_peak
            ex["c4_gathered_GBs"] = T * kk * DQK * 2 / (tot["sparse_attn"] * 1e-3) / 1e9
    except Exception as e:
        ex["c4_error"] = repr(e)
    return ex


if __name__ == "__main__":
    main()
