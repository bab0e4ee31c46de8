"""Top-k selection: bit-exact against the CPU oracle, ties to the lower index."""
import numpy as np
import pytest
import torch

from moespresso_b200.deepseek_v4.attention import causal_indexer_topk, topk_select
from oracle import ds4
from tests.gpu_util import dev, need_gpu

pytestmark = pytest.mark.gpu


def _check(scores, k, valid=None):
    got = topk_select(dev(scores), k, valid=None if valid is None else dev(np.asarray(valid, np.int32))).cpu().numpy()
    ref = ds4.topk_ids(scores, k, valid=valid)
    np.testing.assert_array_equal(got.reshape(ref.shape), ref)


@pytest.mark.parametrize("n", [1, 3, 31, 32, 33, 511, 512, 513, 4096, 32768, 45056])
@pytest.mark.parametrize("k", [1, 16, 512, 2048])
def test_random_rows(n, k):
    need_gpu()
    rng = np.random.default_rng(n * 7 + k)
    _check(rng.standard_normal((3, n)).astype(np.float32), k)


def test_ties_and_specials():
    need_gpu()
    rng = np.random.default_rng(0)
    s = np.round(rng.standard_normal((4, 5000)) * 2).astype(np.float32)      # heavy ties
    _check(s, 512)
    s = np.ones((2, 4096), np.float32)                                        # all equal -> arange(k)
    got = topk_select(dev(s), 512).cpu().numpy()
    np.testing.assert_array_equal(got, np.tile(np.arange(512), (2, 1)))
    s = rng.standard_normal((2, 300)).astype(np.float32)
    s[:, ::3] = -np.inf; s[0, 5] = np.nan; s[1, 7] = np.inf; s[0, 10] = -0.0; s[0, 11] = 0.0
    _check(s, 64)
    _check(s, 299)                                                            # fewer finite than k -> -1 padding
    _check(np.full((1, 77), -np.inf, np.float32), 8)                          # nothing selectable
    s = rng.standard_normal((3, 1000)).astype(np.float32)
    _check(s, 100, valid=[1000, 7, 0])                                        # valid prefixes
    # denormals, huge, negative-only rows
    s = np.concatenate([rng.standard_normal((1, 500)) * 1e-41, -np.abs(rng.standard_normal((1, 500))) * 1e38], 0)
    _check(s.astype(np.float32), 33)


@pytest.mark.parametrize("n,k,rows", [(45057, 2048, 2), (131072, 2048, 3), (1048576, 2048, 1), (200000, 512, 2)])
def test_long_rows(n, k, rows):
    need_gpu()
    rng = np.random.default_rng(n + k)
    _check(rng.standard_normal((rows, n)).astype(np.float32), k)


@pytest.mark.parametrize("n,k,rows", [(16384, 1, 1), (16385, 2048, 1), (100003, 8192, 2), (360448, 2048, 1),
                                      (360449, 2048, 1), (20000, 512, 80)])
def test_kernel_boundaries(n, k, rows):
    """Shapes either side of the switches between the one-CTA, cluster and multi-launch kernels."""
    need_gpu()
    rng = np.random.default_rng(n * 3 + k)
    s = rng.standard_normal((rows, n)).astype(np.float32)
    s[:, ::97] = s[:, 5:6]                                                    # a value repeated across all parts
    _check(s, k)


@pytest.mark.parametrize("n,k,rows", [(32768, 2048, 160), (24576, 512, 150), (45056, 2048, 80), (30001, 2048, 60),
                                      (32768, 1, 75), (40000, 4096, 38)])
def test_many_rows_small_clusters(n, k, rows):
    """Row batches that run as clusters of two or four CTAs: random rows, then rows made of a few distinct values."""
    rng = np.random.default_rng(n + rows)
    _check(rng.standard_normal((rows, n)).astype(np.float32), k)
    _check(np.round(rng.standard_normal((rows, n)) * 2).astype(np.float32), k)


def test_long_rows_ties():
    need_gpu()
    rng = np.random.default_rng(4)
    n = 150000
    _check(np.round(rng.standard_normal((2, n))).astype(np.float32), 2048)    # ~38% of rows tie at each value
    _check(np.zeros((1, n), np.float32), 2048)                                # all equal
    s = rng.standard_normal((2, n)).astype(np.float32); s[:, 1000:] = -np.inf
    _check(s, 2048)                                                           # fewer finite than k
    _check(rng.standard_normal((3, n)).astype(np.float32), 2048, valid=[n, 50000, 5])


def test_ragged_flat_rows():
    need_gpu()
    rng = np.random.default_rng(9)
    lens = np.array([70000, 129, 131072, 1, 46000], np.int64)
    start = np.concatenate([[0], np.cumsum(lens)[:-1]])
    flat = rng.standard_normal(int(lens.sum())).astype(np.float32)
    got = topk_select(dev(flat), 2048, valid=dev(lens.astype(np.int32)), row_start=dev(start),
                      n=int(lens.max())).cpu().numpy()
    for b, (s, n) in enumerate(zip(start, lens)):
        np.testing.assert_array_equal(got[b], ds4.topk_ids(flat[s:s + n], 2048)[0])


@pytest.mark.parametrize("kind", ["normal", "ties", "specials"])
def test_selection_from_a_precounted_first_digit(kind):
    """With the rows' first-digit histograms handed in (as the decode scan leaves them) the selection is the same,
    bit for bit, and the counters are zero afterwards — on the cluster kernel, which uses them, and on the kernels
    that only clear them."""
    need_gpu()
    from tests.gpu_util import first_digit_hist
    rng = np.random.default_rng(11)
    lens = np.array([70000, 129, 131072, 1, 46000, 0, 24000], np.int64)
    start = np.concatenate([[0], np.cumsum(lens)[:-1]])
    flat = rng.standard_normal(int(lens.sum())).astype(np.float32)
    if kind == "ties":
        flat = np.round(flat * 2).astype(np.float32)
    if kind == "specials":
        flat[::7] = -np.inf; flat[5] = np.nan; flat[70001] = np.inf; flat[3] = -0.0; flat[4] = 0.0
        flat[200000:200100] = 1e-40
    hist = np.stack([first_digit_hist(flat[s:s + n]) for s, n in zip(start, lens)])
    for k in (2048, 16):
        h = dev(hist.copy())
        got = topk_select(dev(flat), k, valid=dev(lens.astype(np.int32)), row_start=dev(start), n=int(lens.max()),
                          digit_hist=h).cpu().numpy()
        for b, (s, n) in enumerate(zip(start, lens)):
            ref = ds4.topk_ids(flat[s:s + n], k)[0] if n else np.full(k, -1)
            np.testing.assert_array_equal(got[b], ref)
        assert int(h.abs().sum()) == 0
    # short rows go to the one-CTA kernel, very long ones to the multi-launch one: both ignore and clear the counters
    for n in (5000, 400000):
        s2 = rng.standard_normal((2, n)).astype(np.float32)
        h = dev(np.stack([first_digit_hist(r) for r in s2]))
        got = topk_select(dev(s2), 512, digit_hist=h).cpu().numpy()
        np.testing.assert_array_equal(got, ds4.topk_ids(s2, 512))
        assert int(h.abs().sum()) == 0


def test_causal_indexer_topk_known_answers(golden):
    need_gpu()
    raw = np.array([[[1.0, 20.0, 1000.0, 1000.0], [2.0, 10.0, 1000.0, 1000.0]],
                    [[1.0, 9.0, 1000.0, 1000.0], [2.0, 8.0, 1000.0, 1000.0]]])
    got = causal_indexer_topk(dev(raw), dev(np.ones((2, 2))), [3, 7], np.arange(4), 4, topk=3,
                              index_head_dim=128, n_heads=2).cpu().numpy()
    np.testing.assert_array_equal(got, [[0, -1, -1], [1, 0, -1]])
    for i in range(3):
        raw, w, qp = golden[f"idx{i}_raw"], golden[f"idx{i}_w"], golden[f"idx{i}_qpos"]
        D, H, k, ratio = (int(x) for x in golden[f"idx{i}_meta"])
        if i == 1:
            continue  # float64 reference scores; float32 rounding may reorder near-ties
        got = causal_indexer_topk(dev(raw), dev(w), qp, np.arange(raw.shape[2]), ratio, topk=k,
                                  index_head_dim=D, n_heads=H).cpu().numpy()
        np.testing.assert_array_equal(got, golden[f"idx{i}_topk"])
