"""KV-range sharding of one long sequence with the CUDA operators.

* On one GPU the ranks are emulated in turn (same phases, candidates and partials stacked in rank order where the
  collective would gather them), which exercises the CUDA operators behind the driver.
* With two or more GPUs the driver itself runs as NCCL ranks (one process per GPU, NVLS off).
Both must reproduce the single-device result: bit-exact selection, output within the 16-bit tolerance.
"""
import datetime
import os
import socket

import numpy as np
import pytest
import torch

from moespresso_b200 import dist as mdist
from moespresso_b200 import synth
from oracle import ds4
from tests.gpu_util import need_gpu

pytestmark = pytest.mark.gpu


def _case(R, seed):
    c = synth.config3(seed=seed, lens=[R])
    keys = synth.e4m3_bits_to_f32(c["idx_key_bits"])
    scores = ds4.indexer_scores(c["idx_q"][0][None], keys, c["idx_w"][0][None])[0]
    return c, scores


def _shard(c, lo, hi, device):
    t = lambda x: torch.from_numpy(np.ascontiguousarray(x)).to(device)  # noqa: E731
    return mdist.RangeShard(kv=t(c["kv"][lo:hi]), kv_scales=t(c["kv_scales"][lo:hi]),
                            idx_keys=t(c["idx_key_bits"][lo:hi]).view(torch.float8_e4m3fn), row_lo=lo)


def _check(c, scores_ref, ids, out):
    k = int(c["k"])
    ids = np.sort(np.asarray(ids))
    ref_ids = ds4.topk_ids(scores_ref, k)[0]
    diff = np.setxor1d(ids, ref_ids[ref_ids >= 0])
    if diff.size:   # device and oracle round the scores differently: only near-ties of the k-th score may swap
        kth = np.sort(scores_ref)[::-1][k - 1]
        assert np.all(np.abs(scores_ref[diff] - kth) <= 1e-3 * max(1.0, abs(kth)))
    ref = ds4.indexed_mixed_attention_decode(c["q"][0], None, c["kv"][ids], np.arange(ids.size), None, pos0=0,
                                             window=0, ratio=0, scale=c["scale"], d_v=c["d_v"],
                                             kv_scales=c["kv_scales"][ids])
    assert np.abs(out - ref).max() <= 2e-2


@pytest.mark.parametrize("world,R", [(2, 70000), (4, 9000), (3, 2500), (8, 1048576)])   # the last: one 1 M-row sequence over 8 ranks
def test_range_sharded_step_emulated_ranks(world, R):
    need_gpu()
    c, scores_ref = _case(R, seed=world)
    dev = torch.device("cuda")
    ops = mdist.CudaOps()
    k = int(c["k"])
    q = torch.from_numpy(c["q"][0]).to(dev).to(torch.bfloat16)
    iq = torch.from_numpy(c["idx_q"][0]).to(dev).to(torch.bfloat16)
    iw = torch.from_numpy(c["idx_w"][0]).to(dev)
    shards = [_shard(c, *mdist.row_range(R, world, r, align=128), dev) for r in range(world)]
    cands = [mdist.range_step_candidates(iq, iw, s, k=k, ops=ops) for s in shards]
    all_scores = torch.stack([x[0] for x in cands])
    all_ids = torch.stack([x[1] for x in cands])
    parts = [mdist.range_step_partial(q, s, all_scores, all_ids, k=k, scale=c["scale"], d_v=c["d_v"], ops=ops)
             for s in shards]
    out = ops.merge(torch.stack([p[0] for p in parts]), torch.stack([p[1] for p in parts]), None)
    ids = torch.cat([p[2] for p in parts]).cpu().numpy()
    assert ids.size == min(k, R) and np.unique(ids).size == ids.size
    # the sharded selection is the single-device selection, bit for bit
    from moespresso_b200.deepseek_v4.decode_step import LatentCache, sparse_decode_step
    whole = _shard(c, 0, R, dev)
    cache = LatentCache(kv=whole.kv, kv_scales=whole.kv_scales, idx_keys=whole.idx_keys,
                        row_start=torch.zeros(1, dtype=torch.int64, device=dev),
                        row_count=torch.tensor([R], dtype=torch.int32, device=dev), max_rows=R)
    one_out, one_ids = sparse_decode_step(q[None], iq[None], iw[None], cache, k=k, scale=c["scale"], d_v=c["d_v"],
                                          return_ids=True)
    one = one_ids[0].cpu().numpy()
    np.testing.assert_array_equal(np.sort(ids), one[one >= 0])
    assert (out - one_out[0]).abs().max().item() <= 2e-3
    _check(c, scores_ref, ids, out.float().cpu().numpy())


def _nccl_worker(rank, world, port, R, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    torch.distributed.init_process_group("nccl", rank=rank, world_size=world, device_id=dev,
                                         timeout=datetime.timedelta(seconds=120))
    try:
        c, _ = _case(R, seed=world)
        lo, hi = mdist.row_range(R, world, rank, align=128)
        out, mine = mdist.range_sharded_decode_step(
            torch.from_numpy(c["q"][0]).to(dev).to(torch.bfloat16), torch.from_numpy(c["idx_q"][0]).to(dev).to(torch.bfloat16),
            torch.from_numpy(c["idx_w"][0]).to(dev), _shard(c, lo, hi, dev), k=int(c["k"]), scale=c["scale"],
            d_v=c["d_v"], return_ids=True)
        torch.cuda.synchronize()
        np.save(os.path.join(out_dir, f"out{rank}.npy"), out.float().cpu().numpy())
        np.save(os.path.join(out_dir, f"ids{rank}.npy"), mine.cpu().numpy())
    finally:
        torch.distributed.destroy_process_group()


def test_range_sharded_step_nccl_ranks(tmp_path):
    need_gpu()
    world = min(torch.cuda.device_count(), 4)
    if world < 2:
        pytest.skip("needs two or more GPUs")
    R = 70000
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    torch.multiprocessing.spawn(_nccl_worker, args=(world, port, R, str(tmp_path)), nprocs=world, join=True)
    c, scores_ref = _case(R, seed=world)
    ids = np.concatenate([np.load(tmp_path / f"ids{r}.npy") for r in range(world)])
    outs = [np.load(tmp_path / f"out{r}.npy") for r in range(world)]
    for o in outs[1:]:
        np.testing.assert_array_equal(o, outs[0])          # every rank holds the same merged output
    _check(c, scores_ref, ids, outs[0])


def _plan_worker(rank, world, port, R, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    torch.distributed.init_process_group("nccl", rank=rank, world_size=world, device_id=dev,
                                         timeout=datetime.timedelta(seconds=120))
    try:
        c, _ = _case(R, seed=5)
        lo, hi = mdist.row_range(R, world, rank, align=128)
        shard = _shard(c, lo, hi, dev)
        H, Dqk = c["q"][0].shape
        Hi, Di = c["idx_q"][0].shape
        plan = mdist.RangeDecodePlan(shard, heads=H, d_qk=Dqk, idx_heads=Hi, idx_dim=Di, k=int(c["k"]),
                                     scale=c["scale"], d_v=c["d_v"])
        rng = np.random.default_rng(3)
        same = True
        for step in range(3):   # fresh inputs every step: the graphs must read the plan's buffers, not stale copies
            q = torch.from_numpy(synth.to_bf16_f32(rng.standard_normal((H, Dqk), dtype=np.float32))).to(dev).to(torch.bfloat16)
            iq = torch.from_numpy(synth.to_bf16_f32(rng.standard_normal((Hi, Di), dtype=np.float32))).to(dev).to(torch.bfloat16)
            iw = torch.from_numpy((rng.standard_normal(Hi) / 4).astype(np.float32)).to(dev)
            eager = mdist.range_sharded_decode_step(q, iq, iw, shard, k=int(c["k"]), scale=c["scale"], d_v=c["d_v"])
            got = plan.step(q, iq, iw).clone()
            torch.cuda.synchronize()
            same = same and bool(torch.equal(got, eager))
        with open(os.path.join(out_dir, f"same{rank}.txt"), "w") as f:
            f.write("1" if same else "0")
    finally:
        torch.distributed.destroy_process_group()


def test_range_plan_matches_eager_step(tmp_path):
    """The graph-captured plan (three graphs, two collectives per step) returns the eager driver's result bit for
    bit, over several steps with new inputs; one NCCL rank per GPU, a single rank when there is one GPU."""
    need_gpu()
    world = min(torch.cuda.device_count(), 2)
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    torch.multiprocessing.spawn(_plan_worker, args=(world, port, 50000, str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        assert (tmp_path / f"same{r}.txt").read_text() == "1"
