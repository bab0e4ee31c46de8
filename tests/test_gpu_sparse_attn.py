"""Indexed mixed (sparse) attention against the CPU oracle.

Tolerances (max-abs): 1e-4 for float32 inputs, 2e-2 for 16-bit / int8 inputs."""
import numpy as np
import pytest
import torch

from moespresso_b200 import synth
from moespresso_b200.deepseek_v4 import indexed_attention_kernel as iak
from oracle import ds4
from tests.gpu_util import bf16_round, dev, f16_round, max_abs, need_gpu

pytestmark = pytest.mark.gpu
TOL_F32 = 1e-4
TOL_16 = 2e-2


def test_config1_decode_fp32():
    need_gpu()
    c = synth.config1()
    ids = ds4.topk_ids(ds4.indexer_scores(c["idx_q"][None], c["idx_keys"], c["idx_w"][None]), c["k"])[0]
    out = iak.indexed_mixed_attention_decode(dev(c["q"]), None, dev(c["kv"]), dev(ids.astype(np.int32)), None,
                                             pos0=0, window=0, ratio=0, scale=c["scale"], d_v=c["d_v"])
    ref = ds4.indexed_mixed_attention_decode(c["q"], None, c["kv"], ids, None, pos0=0, window=0, ratio=0,
                                             scale=c["scale"], d_v=c["d_v"])
    assert out.shape == (64, 512) and out.dtype == torch.float32
    assert max_abs(out, ref) <= TOL_F32


def test_reference_probe_shape_with_window_and_sinks():
    """Seeded like the reference's own probe: q N(0,1) [H,512] fp32, raw 128x512 fp16,
    comp Rx512 fp16, topk = arange(512), sinks N(0,1)."""
    need_gpu()
    rng = np.random.default_rng(123)
    H, D, R = 64, 512, 961
    q = rng.standard_normal((H, D)).astype(np.float32)
    raw = f16_round(rng.standard_normal((128, D)))
    comp = f16_round(rng.standard_normal((R, D)))
    sinks = rng.standard_normal(H).astype(np.float32)
    ids = np.arange(512, dtype=np.int32)
    pos0 = 128 + R * 4 - 1
    for raw_start in (0, 37):
        out = iak.indexed_mixed_attention_decode(dev(q), dev(raw, torch.float16), dev(comp, torch.float16), dev(ids),
                                                 dev(sinks), pos0=pos0, raw_start=raw_start)
        ref = ds4.indexed_mixed_attention_decode(q, raw, comp, ids, sinks, pos0=pos0, raw_start=raw_start)
        assert max_abs(out, ref) <= 2e-3   # the reference's own tolerance for this probe


def test_skip_break_and_empty():
    need_gpu()
    rng = np.random.default_rng(1)
    H, D, R = 8, 64, 40
    q = rng.standard_normal((H, D)).astype(np.float32)
    comp = rng.standard_normal((R, D)).astype(np.float32)
    sinks = rng.standard_normal(H).astype(np.float32)
    # visible = (19+1)//4 = 5 : -1 skipped, 7 ends the walk, 1 after it is never visited
    ids = np.array([0, -1, 3, 4, 7, 1], np.int32)
    out = iak.indexed_mixed_attention_decode(dev(q), None, dev(comp), dev(ids), dev(sinks), pos0=19, ratio=4)
    ref = ds4.indexed_mixed_attention_decode(q, None, comp, ids, sinks, pos0=19, ratio=4)
    assert max_abs(out, ref) <= TOL_F32
    # nothing visible: with a sink the output is zero, without one it is zero as well
    none = np.full(6, -1, np.int32)
    for sk in (dev(sinks), None):
        out = iak.indexed_mixed_attention_decode(dev(q), None, dev(comp), dev(none), sk, pos0=19, ratio=4)
        assert float(out.abs().max()) == 0.0
    # -inf sink == no sink
    a = iak.indexed_mixed_attention_decode(dev(q), None, dev(comp), dev(ids), None, pos0=19, ratio=4)
    b = iak.indexed_mixed_attention_decode(dev(q), None, dev(comp), dev(ids),
                                           dev(np.full(H, -np.inf, np.float32)), pos0=19, ratio=4)
    assert torch.equal(a, b)


@pytest.mark.parametrize("kvkind", ["bf16", "int8"])
def test_batched_ragged_decode_16bit(kvkind):
    need_gpu()
    lens = [700, 129, 4096, 33]
    c = synth.config3(seed=7, lens=lens, k=256)
    rng = np.random.default_rng(0)
    B = len(lens)
    ids = np.stack([np.sort(rng.choice(n, size=256, replace=n < 256))[:256] if n >= 256 else
                    np.concatenate([np.arange(n), np.full(256 - n, -1)]) for n in lens]).astype(np.int32)
    if kvkind == "int8":
        kv_t, sc_t = dev(c["kv"]), dev(c["kv_scales"])
        rows = c["kv"].astype(np.float64) * c["kv_scales"].astype(np.float64)[:, None]
    else:
        rows32 = bf16_round(c["kv"].astype(np.float32) * c["kv_scales"].astype(np.float32)[:, None])
        kv_t, sc_t, rows = dev(rows32, torch.bfloat16), None, rows32.astype(np.float64)
    out = iak.sparse_attention(dev(c["q"], torch.bfloat16)[:, :, None, :], kv_t, dev(ids)[:, None, :], None,
                               pos0=0, window=0, ratio=0, scale=c["scale"], d_v=c["d_v"], kv_scales=sc_t,
                               comp_row_start=dev(c["row_start"]), comp_row_count=dev(c["lens"].astype(np.int32)),
                               n_comp=max(lens))
    assert out.shape == (B, 64, 1, 512)
    for b in range(B):
        s = c["row_start"][b]
        ref = ds4.indexed_mixed_attention_decode(c["q"][b], None, rows[s:s + lens[b]], ids[b], None, pos0=0,
                                                 window=0, ratio=0, scale=c["scale"], d_v=c["d_v"])
        assert max_abs(out[b, :, 0], ref) <= TOL_16
    # bf16 output
    out16 = iak.sparse_attention(dev(c["q"], torch.bfloat16)[:, :, None, :], kv_t, dev(ids)[:, None, :], None,
                                 pos0=0, window=0, ratio=0, scale=c["scale"], d_v=c["d_v"], kv_scales=sc_t,
                                 comp_row_start=dev(c["row_start"]), comp_row_count=dev(c["lens"].astype(np.int32)),
                                 n_comp=max(lens), out_dtype=torch.bfloat16)
    assert out16.dtype == torch.bfloat16
    assert max_abs(out16, out) <= float(out.abs().max()) * 2 ** -8 + 1e-6


@pytest.mark.parametrize("qdt", ["f32", "f16", "bf16"])
def test_prefill_live_matches_oracle(qdt):
    need_gpu()
    rng = np.random.default_rng(21)
    B, H, T, D, R, k, raw_cap = 2, 16, 13, 64, 50, 12, 9
    pos0 = 100
    tdt = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}[qdt]
    rnd = {"f32": lambda x: x.astype(np.float32), "f16": f16_round, "bf16": bf16_round}[qdt]
    kvdt = torch.float16 if qdt != "bf16" else torch.bfloat16
    kvr = f16_round if qdt != "bf16" else bf16_round
    q = rnd(rng.standard_normal((B, H, T, D)))
    raw = kvr(rng.standard_normal((B, 1, raw_cap, D)))
    comp = kvr(rng.standard_normal((B, R, D)))
    sinks = rng.standard_normal(H).astype(np.float32)
    ids = np.sort(rng.integers(0, R, size=(B, T, k)), axis=-1).astype(np.int32)
    ids[0, 3, :4] = -1
    fn = iak.indexed_mixed_attention_prefill_live_f32 if qdt == "f32" else iak.indexed_mixed_attention_prefill_live_f16
    out = fn(dev(q, tdt), dev(raw, kvdt), dev(comp, kvdt), dev(ids), dev(sinks), pos0=pos0, window=5, ratio=4,
             raw_start=2)
    assert out.shape == (B, H, T, D) and out.dtype == torch.float32
    for b in range(B):
        ref = ds4.indexed_mixed_attention_prefill(q[b].transpose(1, 0, 2), raw[b, 0], comp[b], ids[b], sinks,
                                                  pos0=pos0, window=5, ratio=4, raw_start=2)
        assert max_abs(out[b].permute(1, 0, 2), ref) <= (TOL_F32 if qdt == "f32" else 2e-3)
    # chunk invariance: the second half of the chunk computed alone gives the same bits
    h = T // 2
    raw_half = raw  # raw buffer ends at the chunk's last token in both calls
    out2 = fn(dev(q[:, :, h:], tdt), dev(raw_half, kvdt), dev(comp, kvdt), dev(ids[:, h:]), dev(sinks),
              pos0=pos0 + h, window=5, ratio=4, raw_start=2)
    assert torch.equal(out2, out[:, :, h:])
    before = iak.prefill_consumer_call_counts()["prefill"]
    fn(dev(q, tdt), dev(raw, kvdt), dev(comp, kvdt), dev(ids), dev(sinks), pos0=pos0, window=5, ratio=4)
    assert iak.prefill_consumer_call_counts()["prefill"] == before + 1


def test_splits_and_partials_merge():
    need_gpu()
    rng = np.random.default_rng(3)
    H, D, Dv, R, k = 16, 96, 64, 3000, 700
    q = rng.standard_normal((1, H, 1, D)).astype(np.float32)
    comp = rng.standard_normal((R, D)).astype(np.float32)
    sinks = rng.standard_normal(H).astype(np.float32)
    ids = np.sort(rng.choice(R, size=k, replace=False)).astype(np.int32)
    ref = ds4.indexed_mixed_attention_decode(q[0, :, 0], None, comp, ids, sinks, pos0=0, window=0, ratio=0, d_v=Dv)
    outs = []
    for ns in (1, 2, 7, 16):
        o = iak.sparse_attention(dev(q), dev(comp), dev(ids)[None, None], dev(sinks), pos0=0, window=0, ratio=0,
                                 d_v=Dv, n_splits=ns)
        assert max_abs(o[0, :, 0], ref) <= TOL_F32
        outs.append(o)
    # two disjoint id ranges as partials, merged with the sink joining once
    parts_o, parts_ml = [], []
    for sub in (ids[:300], ids[300:]):
        for ns in (1, 3):
            pass
        o, ml = iak.sparse_attention(dev(q), dev(comp), dev(sub)[None, None], None, pos0=0, window=0, ratio=0,
                                     d_v=Dv, partial=True, out_layout="bthd", n_splits=3)
        parts_o.append(o); parts_ml.append(ml)
    merged = iak.merge_partials(torch.stack(parts_o), torch.stack(parts_ml), dev(sinks))
    assert max_abs(merged[0, 0], ref) <= TOL_F32
    # an empty partial (no rows) contributes nothing
    o, ml = iak.sparse_attention(dev(q), dev(comp), dev(np.full(4, -1, np.int32))[None, None], None, pos0=0,
                                 window=0, ratio=0, d_v=Dv, partial=True, out_layout="bthd")
    merged = iak.merge_partials(torch.stack(parts_o + [o]), torch.stack(parts_ml + [ml]), dev(sinks))
    assert max_abs(merged[0, 0], ref) <= TOL_F32


def test_contract_errors():
    need_gpu()
    z = lambda *s, dt=torch.float32: torch.zeros(*s, dtype=dt, device="cuda")
    with pytest.raises(ValueError, match="rank-2"):
        iak.indexed_mixed_attention_decode(z(2, 8, 64), None, z(4, 64), z(4, dt=torch.int32), None, pos0=0)
    with pytest.raises(ValueError, match="width must match"):
        iak.indexed_mixed_attention_decode(z(8, 64), None, z(4, 32), z(4, dt=torch.int32), None, pos0=0)
    with pytest.raises(ValueError, match="sinks must have shape"):
        iak.indexed_mixed_attention_decode(z(8, 64), None, z(4, 64), z(4, dt=torch.int32), z(7), pos0=0)
    with pytest.raises(ValueError, match="raw_start must be inside"):
        iak.indexed_mixed_attention_decode(z(8, 64), z(4, 64), z(4, 64), z(4, dt=torch.int32), None, pos0=9,
                                           raw_start=4)
    with pytest.raises(ValueError, match="divisible by 8"):
        iak.indexed_mixed_attention_prefill_live_f32(z(1, 12, 2, 64), None, z(1, 4, 64), z(1, 2, 4, dt=torch.int32),
                                                     None, pos0=0)
    with pytest.raises(ValueError, match="float16"):
        iak.indexed_mixed_attention_prefill_live_f16(z(1, 16, 2, 64), None, z(1, 4, 64),
                                                     z(1, 2, 4, dt=torch.int32), None, pos0=0)
    with pytest.raises(ValueError, match="positive window and ratio"):
        iak.banded_prefill_attention_live(z(1, 16, 2, 64), None, z(1, 4, 64), z(1, 2, 4, dt=torch.int32), None,
                                          pos0=0, window=0, ratio=4)
    with pytest.raises(ValueError, match="mma consumer"):
        iak.banded_prefill_attention_live(z(1, 8, 2, 64), None, z(1, 4, 64), z(1, 2, 4, dt=torch.int32), None,
                                          pos0=0, window=128, ratio=4)
    with pytest.raises(ValueError, match="at least one compressed row"):
        iak.indexer_scores_tiled_live(z(1, 16, 2, 64), z(1, 2, 16), z(1, 0, 64), pos0=0)
    with pytest.raises(ValueError, match="head_dim=128"):
        iak.indexer_scores_tiled_live(z(1, 16, 2, 32), z(1, 2, 16), z(1, 4, 32), pos0=0)
    with pytest.raises(ValueError, match="float16"):
        iak.indexer_scores_tiled_live(z(1, 16, 2, 64, dt=torch.float16), z(1, 2, 16), z(1, 4, 64), pos0=0)
    with pytest.raises(RuntimeError, match="CUDA tensors only"):
        iak.indexed_mixed_attention_decode(torch.zeros(8, 64), None, torch.zeros(4, 64),
                                           torch.zeros(4, dtype=torch.int32), None, pos0=0)


@pytest.mark.parametrize("kvkind,qkind", [("f16", "f32"), ("bf16", "bf16"), ("int8", "bf16"), ("f16", "f16")])
@pytest.mark.parametrize("Dqk,Dv,H", [(576, 512, 64), (512, 512, 64), (192, 128, 16)])
def test_tensor_core_kernel_decode(kvkind, qkind, Dqk, Dv, H):
    """tcgen05 kernel: raw window + selected rows + sinks + skipped ids, several splits,
    against the oracle and against the fp32 CUDA-core kernel."""
    need_gpu()
    rng = np.random.default_rng(Dqk + H)
    R, k, raw_cap = 3000, 700, 128
    qr = {"f32": lambda x: x.astype(np.float32), "f16": f16_round, "bf16": bf16_round}[qkind]
    qt = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}[qkind]
    q = qr(rng.standard_normal((H, Dqk)))
    sinks = rng.standard_normal(H).astype(np.float32)
    ids = np.sort(rng.choice(R, size=k, replace=False)).astype(np.int32)
    ids[5] = -1; ids[300] = -1
    if kvkind == "int8":
        comp_i = rng.integers(-127, 128, size=(R, Dqk), dtype=np.int8)
        raw_i = rng.integers(-127, 128, size=(raw_cap, Dqk), dtype=np.int8)
        cs = np.exp(rng.uniform(np.log(1e-3), np.log(1e-1), size=R)).astype(np.float16)
        rs = np.exp(rng.uniform(np.log(1e-3), np.log(1e-1), size=raw_cap)).astype(np.float16)
        comp_t, raw_t, cs_t, rs_t = dev(comp_i), dev(raw_i), dev(cs), dev(rs)
        comp, raw = comp_i, raw_i
        okw = dict(kv_scales=cs, raw_scales=rs)
    else:
        rnd = f16_round if kvkind == "f16" else bf16_round
        kt = torch.float16 if kvkind == "f16" else torch.bfloat16
        comp, raw = rnd(rng.standard_normal((R, Dqk))), rnd(rng.standard_normal((raw_cap, Dqk)))
        comp_t, raw_t, cs_t, rs_t = dev(comp, kt), dev(raw, kt), None, None
        okw = {}
    pos0 = 128 + R * 4 - 1
    scale = Dqk ** -0.5 * (20.0 if kvkind == "int8" else 1.0)   # int8 rows are ~0.3 rms: sharpen the softmax a bit
    ref = ds4.indexed_mixed_attention_decode(q if kvkind != "f16" or qkind != "f32" else f16_round(q), raw, comp, ids,
                                             sinks, pos0=pos0, raw_start=37, scale=scale, d_v=Dv, **okw)
    tol = 2e-3 if kvkind == "f16" else TOL_16
    outs = []
    for ns in (0, 1, 3):
        o = iak.indexed_mixed_attention_decode(dev(q, qt), raw_t, comp_t, dev(ids), dev(sinks), pos0=pos0,
                                               raw_start=37, scale=scale, d_v=Dv, kv_scales=cs_t, raw_scales=rs_t)
        o = iak.sparse_attention(dev(q, qt)[None, :, None, :], comp_t, dev(ids)[None, None], dev(sinks), pos0=pos0,
                                 window=128, ratio=4, raw_kv=raw_t[None], raw_start=37, scale=scale, d_v=Dv,
                                 kv_scales=cs_t, raw_scales=rs_t, n_splits=ns, check=True)[0, :, 0]
        assert max_abs(o, ref) <= tol, (ns, max_abs(o, ref))
        outs.append(o)
    exact = iak.sparse_attention(dev(q, qt)[None, :, None, :], comp_t, dev(ids)[None, None], dev(sinks), pos0=pos0,
                                 window=128, ratio=4, raw_kv=raw_t[None], raw_start=37, scale=scale, d_v=Dv,
                                 kv_scales=cs_t, raw_scales=rs_t, exact_fp32=True)[0, :, 0]
    assert max_abs(exact, ref) <= 2e-3
    assert max_abs(outs[0], exact) <= tol


@pytest.mark.parametrize("kvkind", ["bf16", "f16", "int8"])
@pytest.mark.parametrize("window,raw_cap", [(101, 128), (6, 128), (128, 127), (63, 64)])
def test_tensor_core_kernel_raw_window_boundary(kvkind, window, raw_cap):
    """Raw windows whose length is not a multiple of four: with 16-bit tables a group of four gathered rows then
    holds rows of both tables (fetched from the compressed one, raw rows patched in afterwards)."""
    need_gpu()
    Dqk, Dv, H, R, k = 576, 512, 64, 2000, 515
    rng = np.random.default_rng(window * 131 + raw_cap)
    q = bf16_round(rng.standard_normal((H, Dqk)))
    sinks = rng.standard_normal(H).astype(np.float32)
    ids = np.sort(rng.choice(R, size=k, replace=False)).astype(np.int32)
    ids[0] = -1; ids[2] = -1; ids[77] = -1
    if kvkind == "int8":
        comp = rng.integers(-127, 128, size=(R, Dqk), dtype=np.int8)
        raw = rng.integers(-127, 128, size=(raw_cap, Dqk), dtype=np.int8)
        cs = np.exp(rng.uniform(np.log(1e-3), np.log(1e-1), size=R)).astype(np.float16)
        rs = np.exp(rng.uniform(np.log(1e-3), np.log(1e-1), size=raw_cap)).astype(np.float16)
        comp_t, raw_t, cs_t, rs_t = dev(comp), dev(raw), dev(cs), dev(rs)
        okw = dict(kv_scales=cs, raw_scales=rs)
        qt, scale = torch.bfloat16, Dqk ** -0.5 * 20.0
    else:
        rnd = f16_round if kvkind == "f16" else bf16_round
        kt = torch.float16 if kvkind == "f16" else torch.bfloat16
        comp, raw = rnd(rng.standard_normal((R, Dqk))), rnd(rng.standard_normal((raw_cap, Dqk)))
        comp_t, raw_t, cs_t, rs_t = dev(comp, kt), dev(raw, kt), None, None
        okw = {}
        qt, scale = kt, Dqk ** -0.5
        q = rnd(q)
    pos0 = 128 + R * 4 - 1
    ref = ds4.indexed_mixed_attention_decode(q, raw, comp, ids, sinks, pos0=pos0, window=window, ratio=4, raw_start=11,
                                             scale=scale, d_v=Dv, **okw)
    for ns in (1, 2, 5):
        o = iak.sparse_attention(dev(q, qt)[None, :, None, :], comp_t, dev(ids)[None, None], dev(sinks), pos0=pos0,
                                 window=window, ratio=4, raw_kv=raw_t[None], raw_start=11, scale=scale, d_v=Dv,
                                 kv_scales=cs_t, raw_scales=rs_t, n_splits=ns, check=True)[0, :, 0]
        assert max_abs(o, ref) <= (2e-3 if kvkind == "f16" else TOL_16), (ns, max_abs(o, ref))


@pytest.mark.parametrize("H,kvkind", [(8, "f32"), (64, "bf16"), (64, "int8")])
@pytest.mark.parametrize("pos0,T", [(40, 1), (0, 1), (100, 20)])
def test_raw_buffer_that_is_not_full_yet(H, kvkind, pos0, T):
    """pos0 + T < raw_cap: outside the reference's domain (its uint32 first_raw_pos wraps and it attends no raw row;
    its callers pass the rows held, not the capacity).  Pinned here: the valid rows are the last pos0 + T slots in
    ring order.  Both the scalar kernel (H = 8, float32) and the tensor-core kernel take this path."""
    need_gpu()
    Dqk, Dv, R, k, raw_cap = 576, 512, 600, 32, 128
    rng = np.random.default_rng(pos0 * 7 + T + H)
    sinks = rng.standard_normal(H).astype(np.float32)
    # few compressed rows are visible this early ((qpos + 1) // 4): ids beyond them end the walk
    ids = np.stack([np.sort(rng.choice(40, size=k, replace=False)) for _ in range(T)]).astype(np.int32)
    cs_t, rs_t = None, None
    if kvkind == "int8":
        comp = rng.integers(-127, 128, size=(R, Dqk), dtype=np.int8)
        raw = rng.integers(-127, 128, size=(raw_cap, Dqk), dtype=np.int8)
        cs = np.exp(rng.uniform(np.log(1e-3), np.log(1e-1), size=R)).astype(np.float16)
        rs = np.exp(rng.uniform(np.log(1e-3), np.log(1e-1), size=raw_cap)).astype(np.float16)
        comp_t, raw_t, cs_t, rs_t = dev(comp), dev(raw), dev(cs), dev(rs)
        comp, raw = ds4.dequant_rows(comp, cs), ds4.dequant_rows(raw, rs)
        # values reach 127 x 0.1: the 16-bit bound is taken relative to them (2e-2 at values of magnitude <= 4)
        q, qt, scale = bf16_round(rng.standard_normal((H, T, Dqk))), torch.bfloat16, Dqk ** -0.5 * 20.0
        tol = TOL_16 * max(1.0, float(np.abs(raw).max()) / 4.0)
    elif kvkind == "bf16":
        comp, raw = bf16_round(rng.standard_normal((R, Dqk))), bf16_round(rng.standard_normal((raw_cap, Dqk)))
        comp_t, raw_t = dev(comp, torch.bfloat16), dev(raw, torch.bfloat16)
        q, qt, scale, tol = bf16_round(rng.standard_normal((H, T, Dqk))), torch.bfloat16, Dqk ** -0.5, TOL_16
    else:
        comp = rng.standard_normal((R, Dqk)).astype(np.float32)
        raw = rng.standard_normal((raw_cap, Dqk)).astype(np.float32)
        comp_t, raw_t = dev(comp), dev(raw)
        q, qt, scale, tol = rng.standard_normal((H, T, Dqk)).astype(np.float32), torch.float32, Dqk ** -0.5, TOL_F32
    ref = ds4.indexed_mixed_attention_prefill(q.transpose(1, 0, 2), raw, comp, ids, sinks, pos0=pos0, window=128,
                                              ratio=4, raw_start=5, scale=scale, d_v=Dv)
    o = iak.sparse_attention(dev(q, qt)[None], comp_t, dev(ids)[None], dev(sinks), pos0=pos0, window=128, ratio=4,
                             raw_kv=raw_t[None], raw_start=5, scale=scale, d_v=Dv, kv_scales=cs_t, raw_scales=rs_t,
                             check=True)[0]
    assert max_abs(o.permute(1, 0, 2), ref) <= tol, max_abs(o.permute(1, 0, 2), ref)


@pytest.mark.parametrize("kvkind", ["bf16", "int8"])
@pytest.mark.parametrize("B,ns,Dqk,Dv,H", [(3, 4, 576, 512, 64), (2, 3, 576, 512, 64), (5, 2, 576, 512, 40),
                                            (2, 4, 256, 256, 16), (2, 2, 192, 128, 16), (8, 4, 576, 512, 64)])
def test_tensor_core_kernel_splits_merged_inside_a_cluster(kvkind, B, ns, Dqk, Dv, H):
    """Two to four splits of a token run as one thread-block cluster and merge through shared memory (no partials,
    no merge kernel); shapes whose blocks do not fit the idle operand buffers keep the partials path.  The result
    must be the oracle's, with a sink, ragged sequences, and an empty split."""
    need_gpu()
    rng = np.random.default_rng(B * 100 + ns * 10 + Dv)
    k, R = 700, 3000
    lens = rng.integers(900, R, size=B)
    lens[0] = 70                                   # fewer visible rows than k: most splits of this sequence are empty
    row_start = np.concatenate([[0], np.cumsum(lens)[:-1]]).astype(np.int64)
    total = int(lens.sum())
    q = bf16_round(rng.standard_normal((B, H, Dqk)))
    sinks = rng.standard_normal(H).astype(np.float32)
    ids = np.stack([np.sort(rng.choice(int(n), size=min(k, int(n)), replace=False)).tolist() + [-1] * (k - min(k, int(n)))
                    for n in lens]).astype(np.int32)
    if kvkind == "int8":
        kv = rng.integers(-127, 128, size=(total, Dqk), dtype=np.int8)
        sc = np.exp(rng.uniform(np.log(1e-3), np.log(3e-2), size=total)).astype(np.float16)
        kv_t, sc_t, okw = dev(kv), dev(sc), dict(kv_scales=None)
    else:
        kv = bf16_round(rng.standard_normal((total, Dqk)))
        kv_t, sc_t, okw = dev(kv, torch.bfloat16), None, {}
    from moespresso_b200 import _abi
    before = int(_abi.load().mxb_kernel_launches())
    o = iak.sparse_attention(dev(q, torch.bfloat16)[:, :, None, :], kv_t, dev(ids)[:, None, :], dev(sinks), pos0=0,
                             window=0, ratio=0, scale=Dqk ** -0.5, d_v=Dv, kv_scales=sc_t,
                             comp_row_start=dev(row_start), comp_row_count=dev(lens.astype(np.int32)),
                             n_comp=int(lens.max()), n_splits=ns, out_dtype=torch.bfloat16, check=True)[:, :, 0]
    launches = int(_abi.load().mxb_kernel_launches()) - before
    # one kernel when the cluster merges, kernel + merge kernel otherwise (more clusters than fit at once; blocks
    # that do not fit the idle operand buffers of a narrow shape)
    assert launches in (1, 2)
    if Dqk == 576:
        assert launches == 1
    for b in range(B):
        s, n = int(row_start[b]), int(lens[b])
        rows = kv[s:s + n]
        ref = ds4.indexed_mixed_attention_decode(q[b], None, rows, ids[b], sinks, pos0=0, window=0, ratio=0,
                                                 scale=Dqk ** -0.5, d_v=Dv,
                                                 **(dict(kv_scales=sc[s:s + n]) if kvkind == "int8" else {}))
        assert max_abs(o[b], ref) <= TOL_16, (b, max_abs(o[b], ref))


def test_tensor_core_kernel_peaked_softmax_and_empty_tiles():
    """Logits spread over hundreds of units force reference-maximum updates and O rescales;
    a list with long runs of skipped ids gives tiles without any valid row."""
    need_gpu()
    rng = np.random.default_rng(77)
    H, Dqk, Dv, R, k = 64, 576, 512, 4000, 1024
    q = bf16_round(rng.standard_normal((H, Dqk)) * 4)
    comp = bf16_round(rng.standard_normal((R, Dqk)) * np.linspace(0.2, 3.0, R)[:, None])   # late rows dominate
    ids = np.sort(rng.choice(R, size=k, replace=False)).astype(np.int32)
    ids[100:400] = -1
    ref = ds4.indexed_mixed_attention_decode(q, None, comp, ids, None, pos0=0, window=0, ratio=0, scale=Dqk ** -0.5,
                                             d_v=Dv)
    for ns in (1, 2):
        o = iak.sparse_attention(dev(q, torch.bfloat16)[None, :, None, :], dev(comp, torch.bfloat16),
                                 dev(ids)[None, None], None, pos0=0, window=0, ratio=0, d_v=Dv, n_splits=ns,
                                 check=True)[0, :, 0]
        assert max_abs(o, ref) <= 2.5e-2, max_abs(o, ref)   # |v| reaches ~10 here
    none = np.full(256, -1, np.int32)
    o = iak.sparse_attention(dev(q, torch.bfloat16)[None, :, None, :], dev(comp, torch.bfloat16),
                             dev(none)[None, None], None, pos0=0, window=0, ratio=0, d_v=Dv, check=True)
    assert float(o.abs().max()) == 0.0


@pytest.mark.parametrize("ns", [1, 2, 4])
def test_tensor_core_kernel_int8_scales_that_rise_and_rows_of_zeros(ns):
    """Int8 rows whose dequantisation scales rise through the list by three decades (the reference maxima, which
    follow logit + log2(scale), keep moving, and O is rescaled each time), with all-zero rows (scale 0) in between:
    those carry no value but count in the denominator with logit 0."""
    need_gpu()
    rng = np.random.default_rng(5)
    H, Dqk, Dv, R, k = 64, 576, 512, 3000, 1024
    q = bf16_round(rng.standard_normal((H, Dqk)) * 0.5)
    kv = rng.integers(-127, 128, size=(R, Dqk), dtype=np.int8)
    sc = (np.exp(np.linspace(np.log(2e-4), np.log(0.2), R)) * rng.uniform(0.5, 1.0, R)).astype(np.float16)
    zero = rng.choice(R, size=300, replace=False)
    sc[zero] = 0
    kv[zero[:150]] = 0                      # a quantiser writes zeros there; the other half keeps stale bytes
    rows = kv.astype(np.float64) * sc.astype(np.float64)[:, None]
    ids = np.sort(rng.choice(R, size=k, replace=False)).astype(np.int32)
    ref = ds4.indexed_mixed_attention_decode(q, None, rows, ids, None, pos0=0, window=0, ratio=0, scale=Dqk ** -0.5,
                                             d_v=Dv)
    o = iak.sparse_attention(dev(q, torch.bfloat16)[None, :, None, :], dev(kv), dev(ids)[None, None], None, pos0=0,
                             window=0, ratio=0, scale=Dqk ** -0.5, d_v=Dv, kv_scales=dev(sc), n_splits=ns,
                             check=True)[0, :, 0]
    assert max_abs(o, ref) <= TOL_16 * max(1.0, float(np.abs(ref).max()) / 4), max_abs(o, ref)
    # a list of nothing but zero rows: uniform weights over zero values
    only = np.sort(zero[:150])[:128].astype(np.int32)
    o = iak.sparse_attention(dev(q, torch.bfloat16)[None, :, None, :], dev(kv), dev(only)[None, None], None, pos0=0,
                             window=0, ratio=0, scale=Dqk ** -0.5, d_v=Dv, kv_scales=dev(sc), check=True)
    assert float(o.abs().max()) == 0.0 and bool(torch.isfinite(o).all())


@pytest.mark.parametrize("kvkind", ["bf16", "int8"])
def test_tensor_core_kernel_more_tokens_than_sms(kvkind):
    """More (sequence, token) items than the device has SMs: the tensor-core kernel is issued one wave at a time
    (at most one CTA per SM per launch), and every item comes out the same as on its own."""
    need_gpu()
    from moespresso_b200 import _abi
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    B = sms + 37
    rng = np.random.default_rng(11)
    H, Dqk, Dv, R, k = 64, 576, 512, 700, 192
    q = bf16_round(rng.standard_normal((B, H, Dqk)))
    if kvkind == "int8":
        kv = rng.integers(-127, 128, size=(R, Dqk), dtype=np.int8)
        sc = np.exp(rng.uniform(np.log(1e-3), np.log(1e-1), size=R)).astype(np.float16)
        rows = kv.astype(np.float64) * sc.astype(np.float64)[:, None]
        kv_t, sc_t = dev(kv), dev(sc)
    else:
        rows32 = bf16_round(rng.standard_normal((R, Dqk)))
        rows, kv_t, sc_t = rows32.astype(np.float64), dev(rows32, torch.bfloat16), None
    ids = np.stack([np.sort(rng.choice(R, size=k, replace=False)) for _ in range(B)]).astype(np.int32)
    zero = torch.zeros(B, dtype=torch.int64, device="cuda")      # every sequence reads the same table
    count = torch.full((B,), R, dtype=torch.int32, device="cuda")
    before = int(_abi.load().mxb_kernel_launches())
    out = iak.sparse_attention(dev(q, torch.bfloat16)[:, :, None, :], kv_t, dev(ids)[:, None, :], None, pos0=0, window=0,
                               ratio=0, scale=Dqk ** -0.5, d_v=Dv, kv_scales=sc_t, comp_row_start=zero,
                               comp_row_count=count, n_comp=R, n_splits=1, check=True)
    assert int(_abi.load().mxb_kernel_launches()) - before == 2      # two waves
    for b in (0, 1, sms - 1, sms, sms + 1, B - 1):
        ref = ds4.indexed_mixed_attention_decode(q[b], None, rows, ids[b], None, pos0=0, window=0, ratio=0,
                                                 scale=Dqk ** -0.5, d_v=Dv)
        assert max_abs(out[b, :, 0], ref) <= TOL_16 * max(1.0, float(np.abs(ref).max()) / 4), (b, max_abs(out[b, :, 0], ref))
    alone = iak.sparse_attention(dev(q[sms:sms + 1], torch.bfloat16)[:, :, None, :], kv_t, dev(ids[sms:sms + 1])[:, None, :],
                                 None, pos0=0, window=0, ratio=0, scale=Dqk ** -0.5, d_v=Dv, kv_scales=sc_t,
                                 comp_row_start=zero[:1], comp_row_count=count[:1], n_comp=R, n_splits=1)
    assert torch.equal(alone[0], out[sms])


def test_tensor_core_kernel_prefill_form():
    need_gpu()
    rng = np.random.default_rng(8)
    B, H, T, Dqk, Dv, R, k = 2, 64, 5, 576, 512, 600, 256
    pos0 = 2000
    q = bf16_round(rng.standard_normal((B, H, T, Dqk)))
    comp = bf16_round(rng.standard_normal((B, R, Dqk)))
    ids = np.sort(rng.integers(0, R, size=(B, T, k)), axis=-1).astype(np.int32)
    sinks = rng.standard_normal(H).astype(np.float32)
    out = iak.indexed_mixed_attention_prefill_live_f16(dev(q, torch.bfloat16), None, dev(comp, torch.bfloat16),
                                                       dev(ids), dev(sinks), pos0=pos0, ratio=4, d_v=Dv)
    assert out.shape == (B, H, T, Dv)
    for b in range(B):
        ref = ds4.indexed_mixed_attention_prefill(q[b].transpose(1, 0, 2), None, comp[b], ids[b], sinks, pos0=pos0,
                                                  ratio=4, d_v=Dv)
        assert max_abs(out[b].permute(1, 0, 2), ref) <= TOL_16
