"""Indexer score kernels against the CPU oracle (float64)."""
import numpy as np
import pytest
import torch

from moespresso_b200 import synth
from moespresso_b200.deepseek_v4 import indexed_attention_kernel as iak
from oracle import ds4
from tests.gpu_util import bf16_round, dev, f16_round, fp8_from_bits, need_gpu

pytestmark = pytest.mark.gpu


def _case(rng, B, H, T, D, R):
    q = rng.standard_normal((B, H, T, D)).astype(np.float32)
    keys = rng.standard_normal((B, R, D)).astype(np.float32)
    w = (rng.standard_normal((B, T, H)) / 4).astype(np.float32)
    return q, keys, w


def _oracle(q, keys, w, pos0, ratio):
    return np.stack([ds4.indexer_scores(q[b].transpose(1, 0, 2), keys[b], w[b], pos0=pos0, ratio=ratio)
                     for b in range(q.shape[0])])


@pytest.mark.parametrize("B,H,T,D,R,pos0,ratio", [
    (1, 16, 1, 64, 4096, 0, 0),          # config-1 shape
    (2, 64, 5, 128, 333, 1200, 4),       # reference head shape, ragged tile, causal mask
    (1, 3, 2, 64, 1, 7, 4),              # single row, odd head count
    (1, 8, 9, 64, 130, 300, 4),          # masked tail inside the chunk
])
def test_exact_fp32_matches_oracle(B, H, T, D, R, pos0, ratio):
    need_gpu()
    rng = np.random.default_rng(5)
    q, keys, w = _case(rng, B, H, T, D, R)
    got = iak.indexer_scores_tiled_live(dev(q), dev(w), dev(keys), pos0=pos0, ratio=ratio).cpu().numpy()
    ref = _oracle(q, keys, w, pos0, ratio)
    assert np.array_equal(np.isneginf(got), np.isneginf(ref))
    fin = np.isfinite(ref)
    np.testing.assert_allclose(got[fin], ref[fin], rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("form", ["bf16", "f16", "fp8_bf16", "fp8_f16"])
@pytest.mark.parametrize("B,H,T,D,R,pos0,ratio", [
    (1, 16, 1, 64, 4096, 0, 0),
    (2, 16, 40, 64, 1000, 3000, 4),      # token tiles (16 tokens x 16 heads = 256 columns), ragged last tile
    (1, 64, 7, 128, 700, 2500, 4),       # D = 128 (two swizzle slabs), 64 heads
    (3, 32, 1, 64, 129, 0, 0),
    (2, 16, 1, 64, 1000, 1500, 4),       # one token WITH the causal row mask: rows >= (1500 + 1) // 4 are -inf
])
def test_tensor_core_path_matches_oracle(form, B, H, T, D, R, pos0, ratio):
    need_gpu()
    rng = np.random.default_rng(11)
    q, keys, w = _case(rng, B, H, T, D, R)
    if form.startswith("fp8"):
        bits = synth.to_e4m3_bits(keys)
        keys_r = synth.e4m3_bits_to_f32(bits)
        kt = fp8_from_bits(bits)
        qdt = torch.bfloat16 if form.endswith("bf16") else torch.float16
    else:
        qdt = torch.bfloat16 if form == "bf16" else torch.float16
        keys_r = bf16_round(keys) if form == "bf16" else f16_round(keys)
        kt = dev(keys_r, qdt)
    q_r = bf16_round(q) if qdt == torch.bfloat16 else f16_round(q)
    before = iak.indexer_scores_call_counts()
    got = iak.indexer_scores_tiled_live(dev(q_r, qdt), dev(w), kt, pos0=pos0, ratio=ratio, check=True).cpu().numpy()
    ref = _oracle(q_r, keys_r, w, pos0, ratio)
    assert np.array_equal(np.isneginf(got), np.isneginf(ref))
    fin = np.isfinite(ref)
    np.testing.assert_allclose(got[fin], ref[fin], rtol=2e-4, atol=2e-3)
    if form.startswith("fp8"):   # the direct FP8 tensor-core mode: reduced-precision accumulation
        got3 = iak.indexer_scores_tiled_live(dev(q_r, qdt), dev(w), kt, pos0=pos0, ratio=ratio, fp8_mma=True,
                                             check=True).cpu().numpy()
        np.testing.assert_allclose(got3[fin], ref[fin], rtol=5e-3, atol=5e-2)
        before["fp8"] += 1
    # the explicit fp32 mode agrees as well
    got2 = iak.indexer_scores_tiled_live(dev(q_r, qdt), dev(w), kt, pos0=pos0, ratio=ratio,
                                         exact_fp32=True).cpu().numpy()
    np.testing.assert_allclose(got2[fin], ref[fin], rtol=1e-5, atol=1e-4)
    after = iak.indexer_scores_call_counts()
    assert sum(after.values()) == sum(before.values()) + 2


def test_ragged_batch_fp8_scores():
    need_gpu()
    c = synth.config3(seed=3, lens=[700, 129, 4096, 1, 2500])
    keys_r = synth.e4m3_bits_to_f32(c["idx_key_bits"])
    rs = dev(c["row_start"]); rc = dev(c["lens"].astype(np.int32))
    got = iak.indexer_scores(dev(c["idx_q"], torch.bfloat16)[:, :, None, :], dev(c["idx_w"])[:, None, :].contiguous(),
                             fp8_from_bits(c["idx_key_bits"]), n_rows=int(c["lens"].max()), row_start=rs,
                             row_count=rc, check=True).cpu().numpy()
    for b, (s, n) in enumerate(zip(c["row_start"], c["lens"])):
        ref = ds4.indexer_scores(c["idx_q"][b][None], keys_r[s:s + n], c["idx_w"][b][None])[0]
        np.testing.assert_allclose(got[s:s + n], ref, rtol=2e-4, atol=2e-3)


def test_scan_counts_the_first_digit_of_the_selection():
    """The decode scan leaves, per sequence, the histogram of the top 11 bits of the selection keys of exactly the
    scores it wrote; a call the scan does not take refuses the histogram."""
    need_gpu()
    from tests.gpu_util import first_digit_hist
    c = synth.config3(seed=4, lens=[70000, 129, 33000, 1, 2500, 5000])
    B = int(c["lens"].size)
    rs = dev(c["row_start"]); rc = dev(c["lens"].astype(np.int32))
    q = dev(c["idx_q"], torch.bfloat16)[:, :, None, :]
    w = dev(c["idx_w"])[:, None, :].contiguous()
    keys = fp8_from_bits(c["idx_key_bits"])
    assert iak.scan_counts_digits(q, keys, n_tokens=1, ratio=0)
    hist = torch.zeros((B, iak.DIGIT_BINS), dtype=torch.int32, device="cuda")
    got = iak.indexer_scores(q, w, keys, n_rows=int(c["lens"].max()), row_start=rs, row_count=rc, digit_hist=hist)
    plain = iak.indexer_scores(q, w, keys, n_rows=int(c["lens"].max()), row_start=rs, row_count=rc)
    assert torch.equal(got, plain)                         # the same score bits with and without the counting
    sc, h = got.cpu().numpy(), hist.cpu().numpy()
    for b, (s, n) in enumerate(zip(c["row_start"], c["lens"])):
        np.testing.assert_array_equal(h[b], first_digit_hist(sc[s:s + n]))
        assert int(h[b].sum()) == int(n)
    # a second call adds on top (the selection is what clears the counters)
    iak.indexer_scores(q, w, keys, n_rows=int(c["lens"].max()), row_start=rs, row_count=rc, digit_hist=hist)
    np.testing.assert_array_equal(hist.cpu().numpy(), 2 * h)
    with pytest.raises(ValueError):                        # wrong shape
        iak.indexer_scores(q, w, keys, n_rows=int(c["lens"].max()), row_start=rs, row_count=rc, digit_hist=hist[:, :100])
    from moespresso_b200 import _abi
    with pytest.raises((_abi.MxbError, RuntimeError)):     # float32 keys: not the scan
        iak.indexer_scores(q.float(), w, dev(synth.e4m3_bits_to_f32(c["idx_key_bits"])), n_rows=int(c["lens"].max()),
                           row_start=rs, row_count=rc, digit_hist=hist)


def test_score_is_independent_of_row_partition():
    """A row's score bits do not depend on where the row sits in the table
    (needed for bit-exact top-k under KV-range sharding)."""
    need_gpu()
    rng = np.random.default_rng(2)
    q, keys, w = _case(rng, 1, 16, 1, 64, 5000)
    bits = synth.to_e4m3_bits(keys[0])
    qd, wd = dev(bf16_round(q), torch.bfloat16), dev(w)
    full = iak.indexer_scores_tiled_live(qd, wd, fp8_from_bits(bits)[None], pos0=0, ratio=0)[0, 0]
    for lo, hi in [(0, 1000), (1000, 1777), (1777, 5000)]:
        part = iak.indexer_scores_tiled_live(qd, wd, fp8_from_bits(bits[lo:hi])[None], pos0=0, ratio=0)[0, 0]
        assert torch.equal(part, full[lo:hi])
