"""Host-side logic of the multi-GPU drivers on CPU ranks (gloo, world size 2 and 3):
sequence assignment, row ranges, and the KV-range-sharded decode step with the device
operators replaced by the NumPy oracle."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from moespresso_b200 import dist as mdist
from oracle import ds4


class OracleOps:
    """NumPy stand-ins with the CudaOps interface (CPU tensors in and out)."""

    def scores(self, idx_q, idx_w, keys):
        s = ds4.indexer_scores(idx_q.numpy()[None], keys.numpy(), idx_w.numpy()[None])[0]
        return torch.from_numpy(s.astype(np.float32))

    def topk(self, scores, k):
        return torch.from_numpy(ds4.topk_ids(scores.numpy(), k)[0].astype(np.int32))

    def attend_partial(self, q, kv, kv_scales, ids, scale, d_v):
        rows = ds4.dequant_rows(kv.numpy(), None if kv_scales is None else kv_scales.numpy())
        sel = ids.numpy(); sel = sel[sel >= 0]
        H = q.shape[0]
        if sel.size == 0:
            return torch.zeros(H, d_v), torch.stack([torch.full((H,), float("-inf")), torch.zeros(H)], 1)
        s = (q.numpy().astype(np.float64) @ rows[sel].T) * scale
        m = s.max(axis=1); p = np.exp(s - m[:, None])
        return (torch.from_numpy((p @ rows[sel][:, :d_v]).astype(np.float32)),
                torch.from_numpy(np.stack([m, p.sum(axis=1)], 1).astype(np.float32)))

    def merge(self, o_parts, ml_parts, sinks):
        out = ds4.merge_partials(o_parts.numpy(), ml_parts[..., 0].numpy(), ml_parts[..., 1].numpy(),
                                 None if sinks is None else sinks.numpy())
        return torch.from_numpy(out.astype(np.float32))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _case(seed=0, R=1000, H=8, Dqk=48, Dv=32, Hi=4, Di=16, k=64, ties=False):
    rng = np.random.default_rng(seed)
    keys = rng.standard_normal((R, Di)).astype(np.float32)
    if ties:
        keys = np.round(keys)           # integer keys and queries: many exactly equal scores
    return dict(q=rng.standard_normal((H, Dqk)).astype(np.float32), kv=rng.standard_normal((R, Dqk)).astype(np.float32),
                idx_q=(np.round(rng.standard_normal((Hi, Di))) if ties else rng.standard_normal((Hi, Di))).astype(np.float32),
                idx_keys=keys, idx_w=(np.ones(Hi) if ties else rng.standard_normal(Hi) / 4).astype(np.float32),
                sinks=rng.standard_normal(H).astype(np.float32), k=k, scale=Dqk ** -0.5, d_v=Dv)


def _worker(rank, world, port, c, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        R = c["kv"].shape[0]
        lo, hi = mdist.row_range(R, world, rank, align=128)
        shard = mdist.RangeShard(kv=torch.from_numpy(c["kv"][lo:hi]), kv_scales=None,
                                 idx_keys=torch.from_numpy(c["idx_keys"][lo:hi]), row_lo=lo)
        out, mine = mdist.range_sharded_decode_step(
            torch.from_numpy(c["q"]), torch.from_numpy(c["idx_q"]), torch.from_numpy(c["idx_w"]), shard, k=c["k"],
            scale=c["scale"], d_v=c["d_v"], sinks=torch.from_numpy(c["sinks"]), ops=OracleOps(), return_ids=True)
        np.save(os.path.join(out_dir, f"out{rank}.npy"), out.numpy())
        np.save(os.path.join(out_dir, f"ids{rank}.npy"), mine.numpy())
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,R,ties", [(2, 1000, False), (3, 700, True), (2, 100, False)])
def test_range_sharded_step_equals_single_device(tmp_path, world, R, ties):
    c = _case(seed=world + R, R=R, ties=ties)
    mp.spawn(_worker, args=(world, _free_port(), c, str(tmp_path)), nprocs=world, join=True)
    scores = ds4.indexer_scores(c["idx_q"][None], c["idx_keys"], c["idx_w"][None])[0].astype(np.float32)
    ref_ids = ds4.topk_ids(scores, c["k"])[0]
    ref = ds4.indexed_mixed_attention_decode(c["q"], None, c["kv"], ref_ids, c["sinks"], pos0=0, window=0, ratio=0,
                                             scale=c["scale"], d_v=c["d_v"])
    got_ids = np.sort(np.concatenate([np.load(tmp_path / f"ids{r}.npy") for r in range(world)]))
    np.testing.assert_array_equal(got_ids, ref_ids[ref_ids >= 0])          # bit-exact selection, ties to lower id
    for r in range(world):
        np.testing.assert_allclose(np.load(tmp_path / f"out{r}.npy"), ref, rtol=1e-4, atol=1e-5)


def test_assign_sequences_and_ranges():
    lens = [100, 900, 300, 300, 50, 700]
    parts = mdist.assign_sequences(lens, 3)
    assert sorted(sum(parts, [])) == list(range(6))
    loads = [sum(lens[i] for i in p) for p in parts]
    assert max(loads) - min(loads) <= 300 and max(loads) <= 900
    assert mdist.assign_sequences(lens, 1) == [list(range(6))]
    assert mdist.assign_sequences([5, 5], 4) == [[0], [1], [], []]
    for world in (1, 2, 4, 8):
        rs = [mdist.row_range(1048576, world, r) for r in range(world)]
        assert rs[0][0] == 0 and rs[-1][1] == 1048576
        assert all(a[1] == b[0] for a, b in zip(rs, rs[1:])) and all(lo % 128 == 0 for lo, _ in rs)
    assert [mdist.row_range(300, 4, r) for r in range(4)] == [(0, 128), (128, 256), (256, 300), (300, 300)]


def test_numpy_lens_to_tables():
    from moespresso_b200 import synth
    c = synth.config3(seed=2, lens=[10, 20, 30])
    sub = mdist.numpy_lens_to_tables(c, [2, 0])
    assert sub["lens"].tolist() == [30, 10] and sub["row_start"].tolist() == [0, 30]
    np.testing.assert_array_equal(sub["kv"][:30], c["kv"][30:60])
    np.testing.assert_array_equal(sub["kv"][30:], c["kv"][:10])
    assert sub["q"].shape[0] == 2


def test_all_winners_in_one_shard(tmp_path):
    """Every one of the k best rows lies in rank 0's range: the other ranks attend nothing and contribute
    (m = -inf, l = 0) partials; selection and output still equal the single-device result."""
    world, R = 3, 900
    c = _case(seed=5, R=R, k=64)
    lo, hi = mdist.row_range(R, world, 0, align=128)
    c["idx_keys"][hi:] *= 1e-3                       # rows outside rank 0's range score ~0 ...
    c["idx_keys"][lo:lo + 200] = np.abs(c["idx_keys"][lo:lo + 200]) + 1.0
    c["idx_q"] = np.abs(c["idx_q"]) + 0.5            # ... rows inside it score high (all weights positive)
    c["idx_w"] = np.abs(c["idx_w"]) + 0.1
    mp.spawn(_worker, args=(world, _free_port(), c, str(tmp_path)), nprocs=world, join=True)
    scores = ds4.indexer_scores(c["idx_q"][None], c["idx_keys"], c["idx_w"][None])[0].astype(np.float32)
    ref_ids = ds4.topk_ids(scores, c["k"])[0]
    assert ref_ids.max() < hi
    assert np.load(tmp_path / "ids1.npy").size == 0 and np.load(tmp_path / "ids2.npy").size == 0
    np.testing.assert_array_equal(np.sort(np.load(tmp_path / "ids0.npy")), ref_ids)
    ref = ds4.indexed_mixed_attention_decode(c["q"], None, c["kv"], ref_ids, c["sinks"], pos0=0, window=0, ratio=0,
                                             scale=c["scale"], d_v=c["d_v"])
    for r in range(world):
        np.testing.assert_allclose(np.load(tmp_path / f"out{r}.npy"), ref, rtol=1e-4, atol=1e-5)


def _failing_worker(rank, world, port, c, out_dir, bad_rank, timeout_s):
    """One rank raises before the candidate exchange; the others must get an error out of the collective (not
    hang) within the process group's timeout, and record it."""
    import datetime
    import time
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=timeout_s))
    R = c["kv"].shape[0]
    lo, hi = mdist.row_range(R, world, rank, align=128)
    shard = mdist.RangeShard(kv=torch.from_numpy(c["kv"][lo:hi]), kv_scales=None,
                             idx_keys=torch.from_numpy(c["idx_keys"][lo:hi]), row_lo=lo)

    class Ops(OracleOps):
        def scores(self, idx_q, idx_w, keys):
            if rank == bad_rank:
                raise RuntimeError("injected failure before the candidate exchange")
            return super().scores(idx_q, idx_w, keys)

    t0 = time.time()
    try:
        mdist.range_sharded_decode_step(torch.from_numpy(c["q"]), torch.from_numpy(c["idx_q"]),
                                        torch.from_numpy(c["idx_w"]), shard, k=c["k"], scale=c["scale"], d_v=c["d_v"],
                                        ops=Ops())
        msg = "completed"
    except Exception as e:   # noqa: BLE001 - the kind of error is the backend's business
        msg = f"error after {time.time() - t0:.1f}s: {type(e).__name__}"
    with open(os.path.join(out_dir, f"rank{rank}.txt"), "w") as f:
        f.write(msg)
    os._exit(1 if rank == bad_rank else 0)   # no clean shutdown of a broken group


def test_rank_failure_surfaces_as_error_on_the_survivors(tmp_path):
    import time
    world, bad, timeout_s = 3, 1, 8
    c = _case(seed=9, R=600)
    ctx = mp.get_context("spawn")
    port = _free_port()
    procs = [ctx.Process(target=_failing_worker, args=(r, world, port, c, str(tmp_path), bad, timeout_s))
             for r in range(world)]
    t0 = time.time()
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=90)
    hung = [p for p in procs if p.is_alive()]
    for p in hung:
        p.kill()
    assert not hung, "a surviving rank hung instead of failing"
    assert time.time() - t0 < 80
    for r in range(world):
        text = (tmp_path / f"rank{r}.txt").read_text()
        assert text.startswith("error"), (r, text)
