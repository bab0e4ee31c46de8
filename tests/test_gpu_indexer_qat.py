"""Indexer QAT, fused QAT score row and score tail through the C ABI against the oracle.

Distributions follow the reference's own adversarial cases for this operator (described in its
tests/test_deepseek_v4_indexer_score_kernel.py:38-75): plain normal rows, rows scaled by 2^30 and 2^-30, group
maxima within a few ulp of 6 * 2^k (the ceil boundary of the group scale), exact midpoints between lattice
values (ties go to the lower value), zeros and denormals.
"""
import numpy as np
import pytest
import torch

from moespresso_b200.deepseek_v4 import indexer_score_kernel as isk
from moespresso_b200.deepseek_v4.indexed_attention_kernel import indexer_q_qat_live
from oracle import ds4
from tests.gpu_util import dev, need_gpu

pytestmark = pytest.mark.gpu


def _qat_case_rows(name, rng):
    if name == "normal":
        return rng.standard_normal((1024, 128)).astype(np.float32)
    if name == "scaled_2p30":
        return (rng.standard_normal((1024, 128)) * 2.0 ** 30).astype(np.float32)
    if name == "scaled_2m30":
        return (rng.standard_normal((1024, 128)) * 2.0 ** -30).astype(np.float32)
    if name == "amax_near_lattice_boundary":
        groups = rng.standard_normal((1024, 4, 32)).astype(np.float32)
        amax = np.abs(groups).max(axis=-1, keepdims=True)
        target = 6.0 * (2.0 ** rng.integers(-40, 40, size=(1024, 4, 1)))
        jitter = 1.0 + rng.integers(-4, 5, size=(1024, 4, 1)) * np.float32(1.1920929e-07)
        return (groups / amax * target * jitter).astype(np.float32).reshape(1024, 128)
    if name == "lattice_midpoints":
        mids = np.array([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0], dtype=np.float32)
        signs = np.where(rng.random((256, 128)) < 0.5, 1.0, -1.0)
        return (rng.choice(mids, size=(256, 128)) * signs).astype(np.float32)
    if name == "zeros_and_denormals":
        rows = np.zeros((8, 128), dtype=np.float32)
        rows[1] = -0.0
        rows[2] = 1e-39
        rows[3] = rng.standard_normal(128) * 1e-38
        rows[4] = rng.standard_normal(128) * 1e-44
        return rows
    raise AssertionError(name)


@pytest.mark.parametrize("case", ["normal", "scaled_2p30", "scaled_2m30", "amax_near_lattice_boundary",
                                  "lattice_midpoints", "zeros_and_denormals"])
def test_indexer_qat_rows_bitexact_float32(case):
    need_gpu()
    rows = _qat_case_rows(case, np.random.default_rng(1234))
    got = isk.indexer_qat_rows(dev(rows))
    assert got.dtype == torch.float32 and tuple(got.shape) == rows.shape
    exp = ds4.indexer_qat(rows)
    np.testing.assert_array_equal(got.cpu().numpy().view(np.uint32), exp.view(np.uint32))


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_indexer_qat_rows_low_precision_query(dtype):
    need_gpu()
    rng = np.random.default_rng(77)
    q = dev(rng.standard_normal((1, 64, 1, 128), dtype=np.float32)).to(dtype)
    got = isk.indexer_qat_rows(q)
    assert got.shape == q.shape and got.dtype == torch.float32
    exp = ds4.indexer_qat(q.float().cpu().numpy())
    np.testing.assert_array_equal(got.cpu().numpy().view(np.uint32), exp.view(np.uint32))
    live = indexer_q_qat_live(q.float())
    assert torch.equal(live, got)


def test_qat_and_tail_reject_bad_inputs():
    need_gpu()
    with pytest.raises(ValueError, match="128-wide"):
        isk.indexer_qat_rows(torch.zeros((4, 64), device="cuda"))
    with pytest.raises(ValueError, match="float32, float16, or bfloat16"):
        isk.indexer_qat_rows(torch.zeros((4, 128), device="cuda", dtype=torch.float64))
    q = torch.zeros((1, 8, 1, 128), device="cuda")
    p = torch.zeros((1, 16, 128), device="cuda")
    w = torch.zeros((1, 1, 8), device="cuda")
    with pytest.raises(ValueError, match="one decode token"):
        isk.fused_qat_indexer_scores(torch.zeros((1, 8, 2, 128), device="cuda"), p, w, 0.1)
    with pytest.raises(ValueError, match="head_dim=128"):
        isk.fused_qat_indexer_scores(torch.zeros((1, 8, 1, 64), device="cuda"), p, w, 0.1)
    with pytest.raises(ValueError, match="between 1 and 64 heads"):
        isk.fused_qat_indexer_scores(torch.zeros((1, 65, 1, 128), device="cuda"), p,
                                     torch.zeros((1, 1, 65), device="cuda"), 0.1)
    with pytest.raises(ValueError, match="at least one row"):
        isk.fused_qat_indexer_scores(q, torch.zeros((1, 0, 128), device="cuda"), w, 0.1)
    s = torch.zeros((1, 32, 1, 40), device="cuda")
    params = torch.tensor([0, 40], dtype=torch.int32, device="cuda")
    with pytest.raises(ValueError, match="32 to 64 index heads"):
        isk.fused_score_tail(torch.zeros((1, 16, 1, 40), device="cuda"), torch.zeros((1, 1, 16), device="cuda"),
                             params, scale=0.1)
    with pytest.raises(ValueError, match="row count at index 1"):
        isk.fused_score_tail(s, torch.zeros((1, 1, 32), device="cuda"), params[:1], scale=0.1)
    with pytest.raises(RuntimeError, match="CUDA tensors only"):
        isk.indexer_qat_rows(torch.zeros((4, 128)))


@pytest.mark.parametrize("n_heads,n_rows,dtype", [(64, 961, torch.float32), (64, 4097, torch.bfloat16),
                                                   (16, 130, torch.float16), (1, 1, torch.float32)])
def test_fused_qat_indexer_scores(n_heads, n_rows, dtype):
    need_gpu()
    rng = np.random.default_rng(n_heads * 1000 + n_rows)
    q = dev(rng.standard_normal((1, n_heads, 1, 128), dtype=np.float32)).to(dtype)
    pooled = ds4.indexer_qat(rng.standard_normal((n_rows, 128), dtype=np.float32))[None]
    weights = (rng.standard_normal((1, 1, n_heads), dtype=np.float32) * n_heads ** -0.5).astype(np.float32)
    got = isk.fused_qat_indexer_scores(q, dev(pooled), dev(weights), 128 ** -0.5)
    assert got.dtype == torch.float32 and tuple(got.shape) == (n_rows,)
    exp = ds4.fused_qat_indexer_scores(q.float().cpu().numpy(), pooled, weights, 128 ** -0.5)
    np.testing.assert_allclose(got.cpu().numpy(), exp, rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("n_heads,cap,valid,wdtype", [(64, 4096, 961, torch.float32), (32, 300, 300, torch.bfloat16),
                                                       (48, 1025, 0, torch.float16), (64, 1, 1, torch.float32)])
def test_fused_score_tail_bitexact(n_heads, cap, valid, wdtype):
    need_gpu()
    rng = np.random.default_rng(cap + n_heads)
    s = rng.standard_normal((1, n_heads, 1, cap), dtype=np.float32) * 7
    s[0, 3, 0, : min(cap, 5)] = np.nan if cap > 4 else 1.0
    w = dev(rng.standard_normal((1, 1, n_heads), dtype=np.float32)).to(wdtype)
    params = torch.tensor([12345, valid], dtype=torch.int32, device="cuda")
    got = isk.fused_score_tail(dev(s), w, params, scale=128 ** -0.5)
    assert tuple(got.shape) == (1, 1, cap) and got.dtype == torch.float32
    exp = ds4.score_tail(s[0, :, 0, :], w.float().cpu().numpy().reshape(-1), valid, 128 ** -0.5)
    g = got.cpu().numpy().reshape(-1)
    np.testing.assert_array_equal(np.isnan(g), np.isnan(exp))                  # NaN scores pass through (payload free)
    ok = ~np.isnan(exp)
    np.testing.assert_array_equal(g[ok].view(np.uint32), exp[ok].view(np.uint32))


def test_pooled_qat_appends_in_place_and_padded_scores_match_the_valid_prefix():
    """The fixed-capacity derived cache of the indexer (reference: model.py:905-944 with
    fixed_decode_state.aux_fixed_update): rows appended over several decode steps equal the QAT of the whole pool
    bit for bit, the buffer never moves, and scoring the full capacity then masking past the valid count gives the
    concat-layout scores bitwise and the same top-k (its tests/test_deepseek_v4_fixed_decode_state.py:337-375)."""
    need_gpu()
    from moespresso_b200.deepseek_v4 import fixed_decode_state as fds
    from moespresso_b200.deepseek_v4.attention import topk_select
    rng = np.random.default_rng(37)
    n_rows, capacity, heads, topk = 961, 1024, 64, 512
    pool = dev(rng.standard_normal((1, n_rows, 128)).astype(np.float32))
    branch, state = fds.FixedBranch(pool_capacity=capacity), {}
    addr = None
    for rows in (1, 640, 641, 960, 961):
        view, prior = fds.pooled_qat_update(branch, state, pool[:, :rows])
        cap = fds.aux_capacity_buffer(branch, "pooled_qat")
        addr = addr or cap.data_ptr()
        assert cap.data_ptr() == addr and tuple(cap.shape) == (1, capacity, 128)
    assert prior == 960 and state["pooled_qat_rows"] == n_rows
    assert torch.equal(view, isk.indexer_qat_rows(pool))
    np.testing.assert_array_equal(view[0].cpu().numpy(), ds4.indexer_qat(pool[0].cpu().numpy()))
    assert torch.all(cap[:, n_rows:] == 0)
    q = dev(rng.standard_normal((1, heads, 1, 128)).astype(np.float32))
    w = dev(rng.standard_normal((1, 1, heads)).astype(np.float32))
    scale = 128 ** -0.5
    valid = isk.fused_qat_indexer_scores(q, view, w, scale)
    params = fds.decode_step_params(offset=3844, pool_rows=n_rows)
    padded = fds.pad_scores_to_capacity(isk.fused_qat_indexer_scores(q, cap, w, scale), params)
    assert torch.equal(padded[:n_rows], valid) and torch.all(torch.isneginf(padded[n_rows:]))
    assert torch.equal(topk_select(padded[None], topk), topk_select(valid[None], topk))
