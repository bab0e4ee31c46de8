"""CPU checks of the oracle's indexer QAT and score tail (no GPU, no reference import)."""
import numpy as np

from oracle import ds4


def _hadamard_matrix(n):
    h = np.array([[1.0]])
    while h.shape[0] < n:
        h = np.block([[h, h], [h, -h]])
    return h


def test_hadamard128_matches_the_matrix_product():
    rng = np.random.default_rng(0)
    x = rng.standard_normal((16, 128)).astype(np.float32)
    ref = (x.astype(np.float64) @ _hadamard_matrix(128)) * 128 ** -0.5
    np.testing.assert_allclose(ds4.indexer_hadamard128(x), ref, rtol=0, atol=2e-6)
    # orthonormal: applying it twice returns the input
    np.testing.assert_allclose(ds4.indexer_hadamard128(ds4.indexer_hadamard128(x)), x, rtol=0, atol=5e-6)


def test_e2m1_round_trip_lattice_and_ties():
    mids = np.array([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0], np.float32)
    g = np.zeros((1, 128), np.float32)
    g[0, :7] = mids
    g[0, 7] = 6.0            # group amax 6 -> scale 1
    g[0, 8:15] = -mids
    out = ds4.indexer_fp4_act_roundtrip(g)[0]
    np.testing.assert_array_equal(out[:8], [0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0])      # ties -> lower value
    np.testing.assert_array_equal(out[8:15], [-0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0])
    # a group of zeros stays zero; outputs are lattice values times the group scale
    assert not np.any(ds4.indexer_fp4_act_roundtrip(np.zeros((2, 128), np.float32)))
    rng = np.random.default_rng(1)
    x = rng.standard_normal((64, 128)).astype(np.float32) * 3.0
    y = ds4.indexer_fp4_act_roundtrip(x).reshape(64, 4, 32)
    amax = np.abs(x.reshape(64, 4, 32)).max(-1, keepdims=True)
    scale = 2.0 ** np.ceil(np.log2(amax / 6.0))
    lattice = np.abs(y) / scale
    assert np.all(np.min(np.abs(lattice[..., None] - ds4._E2M1), axis=-1) < 1e-6)
    assert np.all(np.abs(y) <= np.abs(x.reshape(64, 4, 32)).max(-1, keepdims=True) * 2.0 + 1e-6)


def test_score_tail_against_float64():
    rng = np.random.default_rng(2)
    for H in (32, 48, 64):
        s = rng.standard_normal((H, 300)).astype(np.float32) * 5
        w = rng.standard_normal(H).astype(np.float32)
        got = ds4.score_tail(s, w, 257, 128 ** -0.5)
        ref = -(np.maximum(s.astype(np.float64), 0) * 128 ** -0.5 * (w.astype(np.float64) * H ** -0.5)[:, None]).sum(0)
        np.testing.assert_allclose(got[:257], ref[:257], rtol=1e-5, atol=1e-5)
        assert np.all(np.isposinf(got[257:]))
