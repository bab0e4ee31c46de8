"""The CPU oracle against vectors produced by the reference's own NumPy code
(tests/golden/make_golden.py) and against the known-answer values of the
reference's tests/test_deepseek_v4_attention.py."""
import math

import numpy as np

from oracle import ds4


def test_visibility_tables(golden):
    qpos, pool = golden["vis_qpos"], golden["vis_pool"]
    for ratio in (4, 128):
        np.testing.assert_array_equal(ds4.compressed_visibility(qpos, pool, ratio), golden[f"vis_r{ratio}"])
        np.testing.assert_array_equal(ds4.visible_compressed_count(qpos, ratio), golden[f"viscount_r{ratio}"])


def test_visibility_known_answers():
    # tests/test_deepseek_v4_attention.py:163-189
    vis4 = ds4.compressed_visibility([2, 3, 4, 127, 128], np.arange(34), 4)
    assert not vis4[0, 0] and vis4[1, 0] and vis4[2, 0]
    assert vis4[3, 31] and not vis4[3, 32] and vis4[4, 31] and not vis4[4, 32]
    vis128 = ds4.compressed_visibility([126, 127, 128], np.arange(2), 128)
    assert not vis128[0, 0] and vis128[1, 0] and vis128[2, 0] and not vis128[2, 1]
    np.testing.assert_array_equal(
        ds4.visible_compressed_count([3, 4, 65535, 65536, 1048575], 4),
        np.array([1, 1, 16384, 16384, 262144]))


def test_sink_softmax(golden):
    for i in range(3):
        out = ds4.sink_softmax_attention(golden[f"sink{i}_scores"], golden[f"sink{i}_values"],
                                         golden[f"sink{i}_sinks"])
        np.testing.assert_allclose(out, golden[f"sink{i}_out"], rtol=1e-13, atol=1e-14)


def test_sink_known_answer():
    # tests/test_deepseek_v4_attention.py:146-160
    scores = np.array([[0.25]]); values = np.array([[[8.0, -4.0]]]); sinks = np.array([1.25])
    out = ds4.sink_softmax_attention(scores, values, sinks)
    den = math.exp(0.25 - 1.25) + 1.0
    np.testing.assert_allclose(out, values[:, 0, :] * (math.exp(0.25 - 1.25) / den))
    assert np.allclose(ds4.sink_softmax_attention(scores, values, np.array([-np.inf])), values[:, 0, :])


def test_indexer_scores_and_topk(golden):
    for i in range(3):
        raw, w, qp = golden[f"idx{i}_raw"], golden[f"idx{i}_w"], golden[f"idx{i}_qpos"]
        D, H, k, ratio = (int(x) for x in golden[f"idx{i}_meta"])
        R = raw.shape[2]
        np.testing.assert_allclose(
            ds4.indexer_weighted_scores(raw, w, index_head_dim=D, n_heads=H),
            golden[f"idx{i}_weighted"], rtol=1e-13)
        got = ds4.causal_indexer_topk(raw, w, qp, np.arange(R), ratio, topk=k,
                                      index_head_dim=D, n_heads=H)
        np.testing.assert_array_equal(got, golden[f"idx{i}_topk"])
        # the masked score matrix through the q.k formulation: use identity keys so that
        # q[t,h,:] . key[r,:] reproduces raw[t,h,r]
        scale = (D ** -0.5) * (H ** -0.5)
        s = ds4.indexer_scores(raw, np.eye(R), w * scale, pos0=int(qp[0]), ratio=ratio)
        np.testing.assert_allclose(s, golden[f"idx{i}_causal"], rtol=1e-12)
        # index-ordered form selects the same set
        ids = ds4.topk_ids(golden[f"idx{i}_causal"], k, order="index")
        for a, b in zip(ids, golden[f"idx{i}_topk"]):
            assert sorted(a[a >= 0]) == sorted(b[b >= 0])
            assert list(a[a >= 0]) == sorted(a[a >= 0])


def test_topk_known_answer():
    # tests/test_deepseek_v4_attention.py:206-244
    raw = np.array([[[1.0, 20.0, 1000.0, 1000.0], [2.0, 10.0, 1000.0, 1000.0]],
                    [[1.0, 9.0, 1000.0, 1000.0], [2.0, 8.0, 1000.0, 1000.0]]])
    got = ds4.causal_indexer_topk(raw, np.ones((2, 2)), np.array([3, 7]), np.arange(4), 4,
                                  topk=3, index_head_dim=128, n_heads=2)
    np.testing.assert_array_equal(got, np.array([[0, -1, -1], [1, 0, -1]]))


def test_topk_tie_rule_and_specials():
    s = np.array([[1.0, 1.0, 1.0, 1.0, 1.0]])
    np.testing.assert_array_equal(ds4.topk_ids(s, 3), [[0, 1, 2]])      # all ties -> arange(k)
    s = np.array([[0.0, -0.0, np.nan, -np.inf, 0.0, 5.0]])
    np.testing.assert_array_equal(ds4.topk_ids(s, 3), [[0, 1, 5]])      # -0 == +0, NaN/-inf never
    np.testing.assert_array_equal(ds4.topk_ids(s, 6), [[0, 1, 4, 5, -1, -1]])
    np.testing.assert_array_equal(ds4.topk_ids(s, 2, valid=[2]), [[0, 1]])


def test_raw_window_attention_matches_reference_numpy(golden):
    for i in range(3):
        q, kv, sk = golden[f"raw{i}_q"], golden[f"raw{i}_kv"], golden[f"raw{i}_sinks"]
        window = int(golden[f"raw{i}_meta"][0])
        T, H, D = q.shape
        out = ds4.indexed_mixed_attention_prefill(
            q, kv, np.zeros((0, D)), np.zeros((T, 0), dtype=np.int64), sk,
            pos0=0, window=window, ratio=4)
        np.testing.assert_allclose(out, golden[f"raw{i}_out"], rtol=2e-5, atol=2e-6)


def test_decode_skip_break_and_merge():
    rng = np.random.default_rng(0)
    H, D, R = 4, 16, 12
    q = rng.normal(size=(H, D)); comp = rng.normal(size=(R, D)); sk = rng.normal(size=H)
    # visible = (pos0+1)//4 = 5: ids 7.. stop the walk, -1 is skipped
    ids = np.array([0, -1, 3, 4, 7, 1])
    out = ds4.indexed_mixed_attention_decode(q, None, comp, ids, sk, pos0=19, ratio=4)
    ref = ds4.sink_softmax_attention((q @ comp[[0, 3, 4]].T) * D ** -0.5, comp[[0, 3, 4]], sk)
    np.testing.assert_allclose(out, ref, rtol=1e-12)
    # split the rows in two partials and merge with the sink
    parts_o, parts_m, parts_l = [], [], []
    for rows in ([0], [3, 4]):
        s = (q @ comp[rows].T) * D ** -0.5
        m = s.max(axis=1); p = np.exp(s - m[:, None])
        parts_o.append(p @ comp[rows]); parts_m.append(m); parts_l.append(p.sum(axis=1))
    merged = ds4.merge_partials(np.stack(parts_o), np.stack(parts_m), np.stack(parts_l), sk)
    np.testing.assert_allclose(merged, ref, rtol=1e-12)


def test_e4m3_round_trip():
    codes = np.arange(256, dtype=np.uint8)
    vals = ds4.e4m3_decode(codes)
    ok = ~np.isnan(vals)
    back = ds4.e4m3_encode(vals[ok])
    np.testing.assert_array_equal(ds4.e4m3_decode(back), vals[ok])
    assert ds4.e4m3_decode(ds4.e4m3_encode(np.array([1000.0, -1000.0]))).tolist() == [448.0, -448.0]
    try:
        import torch
    except Exception:
        return
    x = np.random.default_rng(1).normal(size=4096) * 3
    t = torch.tensor(x, dtype=torch.float32).to(torch.float8_e4m3fn)
    np.testing.assert_array_equal(t.view(torch.uint8).numpy(), ds4.e4m3_encode(x.astype(np.float32)))


def _fp8kv_golden():
    import os
    return np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "fp8kv_golden.npz"))


def test_fp8_kv_replay_form_matches_reference_vectors():
    """oracle.ds4.fp8_kv_round_replay / e4m3fn_dequant against outputs of the reference's own NumPy functions
    (tests/golden/make_golden_fp8kv.py)."""
    g = _fp8kv_golden()
    np.testing.assert_array_equal(ds4.E4M3FN_VALUES, g["table"])
    np.testing.assert_array_equal(ds4.e4m3fn_dequant(g["dequant_in"]).view(np.uint32), g["dequant_out"].view(np.uint32))
    np.testing.assert_array_equal(ds4.fp8_kv_round_replay(g["rows"]).view(np.uint32), g["rounded"].view(np.uint32))


def test_fp8_kv_served_form_stays_within_scale_rounding_of_the_replay_form():
    g = _fp8kv_golden()
    served = ds4.fp8_kv_prefix_rows(g["rows"])
    np.testing.assert_array_equal(served[:, 448:], g["rows"][:, 448:])            # rotary tail untouched
    np.testing.assert_allclose(served, g["rounded"], rtol=1e-6, atol=0)          # float32 exp(k ln 2) vs 2**k


def test_rope_matches_reference_vectors():
    """oracle.ds4 rope functions and the host-side frequency helper of the package against outputs of the
    reference's NumPy functions (tests/golden/make_golden_rope.py)."""
    import os
    g = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "rope_golden.npz"))
    yarn = {"factor": float(g["yarn_factor"]), "original_seq_len": float(g["yarn_original_seq_len"]),
            "beta_fast": float(g["yarn_beta_fast"]), "beta_slow": float(g["yarn_beta_slow"])}
    np.testing.assert_array_equal(ds4.rope_inverse_frequencies(64, float(g["swa_base"])), g["inv_freq_swa"])
    np.testing.assert_array_equal(ds4.rope_inverse_frequencies(64, float(g["compress_base"]), yarn), g["inv_freq_yarn"])
    np.testing.assert_array_equal(ds4.apply_rope_tail(g["x"], g["pos"], base=float(g["compress_base"]), yarn=yarn),
                                  g["fwd_yarn"])
    np.testing.assert_array_equal(ds4.apply_rope_tail(g["fwd_yarn"], g["pos"], base=float(g["compress_base"]),
                                                      yarn=yarn, inverse=True), g["inv_yarn"])
    np.testing.assert_array_equal(ds4.apply_rope_tail(g["x"], g["pos"], base=float(g["swa_base"])), g["fwd_swa"])
    from moespresso_b200.deepseek_v4 import attention as pkg
    np.testing.assert_array_equal(pkg.rope_inverse_frequencies(64, pkg.DS4_COMPRESS_ROPE_BASE, pkg.DS4_YARN),
                                  g["inv_freq_yarn"])
    np.testing.assert_array_equal(pkg.rope_inverse_frequencies(64, pkg.DS4_SWA_ROPE_BASE), g["inv_freq_swa"])
    assert pkg.DS4_YARN == yarn


def test_raw_rows_of_a_buffer_that_is_not_full_yet():
    """Pinned convention outside the reference's domain.  The reference's kernels take n_raw = the rows the buffer
    holds and compute first_raw_pos = last_pos + 1 - n_raw in uint32 (indexed_attention_kernel.py:120-130,
    :243-251): with n_raw > last_pos + 1 that wraps and no raw row is attended, so its callers never pass it.  Here
    raw_cap may exceed last_pos + 1 (a pre-allocated ring that is still filling): the valid rows are the LAST
    last_pos + 1 slots in ring order, position p at (raw_start + p + raw_cap - last_pos - 1) mod raw_cap."""
    raw_cap, raw_start, last_pos = 128, 11, 40
    rows, comp = ds4._visit_rows(raw_cap, 0, [], qpos=40, last_pos=last_pos, window=128, ratio=4, raw_start=raw_start)
    assert rows == [(raw_start + p + raw_cap - last_pos - 1) % raw_cap for p in range(41)] and comp == []
    rows, _ = ds4._visit_rows(raw_cap, 0, [], qpos=30, last_pos=last_pos, window=8, ratio=4, raw_start=raw_start)
    assert rows == [(raw_start + p + raw_cap - last_pos - 1) % raw_cap for p in range(23, 31)]
    # inside the reference's domain (raw_cap <= last_pos + 1) the same formula is the reference's own
    rows, _ = ds4._visit_rows(16, 0, [], qpos=40, last_pos=40, window=0, ratio=4, raw_start=3)
    assert rows == [(3 + i) % 16 for i in range(16)]
