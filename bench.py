#!/usr/bin/env python
"""Benchmark of the sparse-decode attention hot path (and, as extras, the other configurations).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload ...]

Headline workload (N = 1): the batched DS-V4-shaped sparse decode step — batch 32,
context ~ U[32K, 128K] per sequence, top-k 2048, bf16 queries over an int8 latent KV
cache with per-token fp16 scales, FP8-E4M3 index keys, 64 heads x 576 (V = first 512),
indexer 16 heads x 64, seed 1.  One "step" = indexer score -> top-k -> indexed sparse
attention for the whole batch (one decoded token per sequence), so tokens/s = batch /
step time.  With N > 1 every rank holds its own batch of 32 sequences (sequence
sharding, no collective on the data path): weak scaling.

Prints ONE JSON line on rank 0.  `value` is timed with the inputs resident in HBM;
`e2e` goes through the public Python operator with the step's inputs in pinned host
memory and the result read back to the host inside the timed region.  The latent KV
and index-key tables are the decode cache (state that lives on the device between
steps, like weights); the per-step inputs are the queries, indexer queries and
head weights.
"""
from __future__ import annotations

import argparse
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


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return float(d["hbm_gbs"]), float(d["bf16_tflops"]), "measured"
    return 6650.0, 1590.0, "fallback"


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
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.gpu)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([x.strip() for x in line.split(",")])

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, smax, reasons = [], [], set()
        for r in self.rows:
            try:
                sm.append(float(r[1])); smax.append(float(r[2]))
            except Exception:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(smax) if smax else None,
                "reasons": sorted(reasons), "samples": len(sm)}


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
        "config": {"workload": WORKLOAD, "batch": B, "topk": int(c["k"]), "rows_total": int(c["lens"].sum())},
        "cpu_baseline": {"value": val, "unit": UNIT, "cores": cores, "kind": "port",
                         "sample": f"all {B} sequences of the batch per step, NumPy float32 (BLAS threads = {cores})"},
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
    ap.add_argument("--no-extras", action="store_true", help="skip the secondary workloads (c1, c2)")
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
    from moespresso_b200.deepseek_v4.decode_step import LatentCache
    from moespresso_b200.deepseek_v4.indexed_attention_kernel import indexer_scores, sparse_attention

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: there is no CPU path for the product kernels")
    _abi.load()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    W = max(args.warmup, 3)
    K = args.steps

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
    out_h = torch.empty((B, 64, d_v), dtype=torch.bfloat16).pin_memory()   # the step's result in the activation type

    from moespresso_b200 import _torchabi
    from moespresso_b200.deepseek_v4.decode_step import SparseDecodePlan, sparse_decode_step

    plan = SparseDecodePlan(cache, heads=64, d_qk=576, idx_heads=16, idx_dim=64, k=kk, scale=scale, d_v=d_v,
                            q_dtype=torch.bfloat16, out_dtype=torch.bfloat16, graph=not args.no_graph)
    plan.load_inputs(q_d, iq_d, iw_d)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(x: float) -> float:
        if world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    sampler = ClockSampler(local)
    sampler.start()
    for _ in range(W):
        plan.launch()
    barrier()
    # ---- timed region: K steps, inputs resident in HBM
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(K):
        plan.launch()
    e1.record()
    barrier()
    ms_step = max_over_ranks(e0.elapsed_time(e1) / K)

    # ---- per-stage device time: each entry point captured as its own CUDA graph and replayed K times between two
    # events (no host gaps inside the timed region; the 167 MB key table alone exceeds L2 between replays)
    lib = _abi.load()
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
        for _ in range(K):
            g.replay()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / K * 1e3

    stage = {
        "indexer_scores": stage_us(lambda: indexer_scores(
            iq_d[:, :, None, :], iw_d[:, None, :].contiguous(), cache.idx_keys, n_rows=cache.max_rows,
            row_start=cache.row_start, row_count=cache.row_count)),
        "topk_select": stage_us(lambda: topk_select(sc_e, kk, valid=cache.row_count, row_start=cache.row_start,
                                                    n=cache.max_rows)),
        "sparse_attn": stage_us(lambda: sparse_attention(
            q_d[:, :, None, :], cache.kv, ids_e[:, None, :], None, pos0=0, window=0, ratio=0, scale=scale, d_v=d_v,
            kv_scales=cache.kv_scales, comp_row_start=cache.row_start, comp_row_count=cache.row_count,
            n_comp=cache.max_rows, out_dtype=torch.bfloat16)),
    }

    # ---- end to end: pinned host inputs -> device -> step -> result back on the host, every step
    in_h, (qv, iqv, iwv) = plan.host_buffer()   # the step's inputs live in one pinned buffer: one H2D copy
    qv.copy_(q_h)
    iqv.copy_(iq_h)
    iwv.copy_(iw_h)
    for _ in range(2):
        out_h.copy_(plan.run_packed(in_h), non_blocking=True)
    barrier()
    f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    f0.record()
    for _ in range(K):
        out_h.copy_(plan.run_packed(in_h), non_blocking=True)
        torch.cuda.current_stream().synchronize()   # the caller consumes the result of every step
    f1.record()
    barrier()
    ms_e2e = max_over_ranks(f0.elapsed_time(f1) / K)
    # keep the device busy with the same step until the clock sampler has seen it under load
    t_end = time.time() + 1.5
    while time.time() < t_end and len(sampler.rows) < 8:
        for _ in range(50):
            plan.launch()
        torch.cuda.synchronize()
    clocks = sampler.stop()
    if K * ms_step < 500:
        clocks["note"] = ("timed region shorter than the 100 ms sampling period: samples span warm-up, the timed "
                          "region and an untimed repeat of the same step")

    hbm, tf, which = measured_peaks()
    # algorithmic bytes of the dominant kernel (indexer score scan): FP8 keys read once, fp32 scores written once
    idx_bytes = total * 64 + total * 4 + B * (16 * 64 * 2 + 16 * 4)
    achieved = idx_bytes / (stage["indexer_scores"] * 1e-6) / 1e9
    # DRAM traffic of the same kernel from one ncu capture on the --small case (profiles/): 65.0 B read and
    # 4.8 B written per key row against 68 B algorithmic; scaled to this launch by its row count
    traffic = total * (65.0 + 4.8)
    step_bytes = idx_bytes + total * 4 + B * (kk * (576 + 2) + 64 * 576 * 2 + 64 * d_v * 2 + kk * 4 * 2)

    line = {
        "metric": METRIC, "value": world * B / (ms_step * 1e-3), "unit": UNIT, "n_gpus": world, "steps": K,
        "warmup": W, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic",
        "config": {"workload": WORKLOAD if not args.small else WORKLOAD + "_SMALL", "batch_per_gpu": B,
                   "rows_total_per_gpu": total, "topk": kk, "heads": 64, "d_qk": 576, "d_v": d_v,
                   "indexer": "16x64 fp8-e4m3 keys", "kv": "int8 + fp16 per-token scale",
                   "parallelism": f"sequence-sharded x{world}, no collective",
                   "l2": "inputs (1.7 GB per GPU) exceed L2, no flush needed"},
        "e2e": {"value": world * B / (ms_e2e * 1e-3), "unit": UNIT,
                "h2d_bytes_per_step": int(in_h.numel()),
                "d2h_bytes_per_step": int(out_h.numel() * out_h.element_size()), "ms_per_step": ms_e2e},
        "gpu_launches": kernels_per_step * K,
        "launch": (f"one CUDA graph per step ({kernels_per_step} kernels of this library)" if not args.no_graph
                   else f"eager ({kernels_per_step} kernels of this library per step)"),
        "stage_us": stage,
        "roofline": {"bound": "hbm", "kernel": "indexer_decode_kernel<64, 16 heads>", "achieved": achieved, "peak": hbm,
                     "unit": "GB/s", "frac": achieved / hbm, "peak_source": which, "traffic": traffic,
                     "algorithmic_bytes": idx_bytes, "launch_us": stage["indexer_scores"],
                     "frac_of_nominal_8TBs": achieved / 8000.0,
                     "whole_step_GBs": step_bytes / (ms_step * 1e-3) / 1e9},
        "clocks": clocks,
    }

    if rank == 0 and world == 1 and not args.no_extras and not args.small:
        line["extras"] = run_extras(torch, dev, tf)
    if rank == 0 and world == 1 and not args.no_cpu:
        cores = len(os.sched_getaffinity(0))
        seqs = list(range(B))
        t = cpu_decode_batch(c, seqs)
        line["cpu_baseline"] = {"value": len(seqs) / t, "unit": UNIT, "cores": cores, "kind": "port",
                                "sample": f"one pass over all {len(seqs)} sequences of the batch, NumPy float32"}
    if rank == 0:
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def run_extras(torch, dev, tf_peak) -> dict:
    """Secondary workloads, single GPU: config 1 (fp32 decode, latency) and config 2 (Qwen prefill)."""
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
        ex["c1_fp32_decode_step_us"] = ms * 1e3
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
        # config 4: 4096-token chunk over 32768 ratio-4 compressed rows, top-k 2048 per token, bf16.
        # Inputs are generated on the device (same shapes and N(0,1) distributions as synth.config4).
        from moespresso_b200 import _torchabi
        from moespresso_b200.deepseek_v4.prefill_step import sparse_prefill_step
        T, R, H, Dqk, Dv, Hi, Di, kk = 4096, 32768, 64, 576, 512, 16, 64, 2048
        g = torch.Generator(device=dev).manual_seed(2)
        rn = lambda *sh: torch.randn(*sh, generator=g, device=dev, dtype=torch.float32)
        kv, q = rn(R, Dqk).to(torch.bfloat16), rn(T, H, Dqk).to(torch.bfloat16)
        iq, ik, iw = rn(T, Hi, Di).to(torch.bfloat16), rn(R, Di).to(torch.bfloat16), rn(T, Hi) / 4
        run = lambda: sparse_prefill_step(q, kv, iq, ik, iw, pos0=131072 - T, ratio=4, k=kk, scale=Dqk ** -0.5,
                                          d_v=Dv, window=0)
        run(); torch.cuda.synchronize()
        _torchabi.TIMER = {}
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(); run(); b.record(); torch.cuda.synchronize()
        timer, _torchabi.TIMER = _torchabi.TIMER, None
        tot = {name: sum(x.elapsed_time(y) for x, y in evs) for name, evs in timer.items()}
        ex["c4_chunk_ms"] = a.elapsed_time(b)
        ex["c4_entry_point_ms"] = tot
        if tot.get("indexer_scores"):
            ex["c4_indexer_tflops"] = 2.0 * T * Hi * Di * R / (tot["indexer_scores"] * 1e-3) / 1e12
        if tot.get("sparse_attn"):
            ex["c4_sparse_attn_tflops"] = 2.0 * T * H * kk * (Dqk + Dv) / (tot["sparse_attn"] * 1e-3) / 1e12
            ex["c4_gathered_GBs"] = T * kk * Dqk * 2 / (tot["sparse_attn"] * 1e-3) / 1e9
    except Exception as e:
        ex["c4_error"] = repr(e)
    return ex


if __name__ == "__main__":
    main()
