"""Parity at the full sizes of the benchmark configurations, through checks whose cost does not grow with the
size: the selection property of top-k over every row, and the oracle on a sample of rows / sequences / heads."""
import numpy as np
import pytest
import torch

from moespresso_b200 import synth
from moespresso_b200.deepseek_v4.decode_step import LatentCache, sparse_decode_step
from moespresso_b200.qwen.full_attention import sdpa_fa_prefill
from oracle import ds4
from tests.gpu_util import dev, fp8_from_bits, max_abs, need_gpu

pytestmark = pytest.mark.gpu


def test_batched_decode_step_at_full_size():
    """Batch 32, contexts U[32K, 128K], top-k 2048, int8 KV + FP8 index keys: 2.6 M rows."""
    need_gpu()
    c = synth.config3(seed=1)
    B, k = int(c["lens"].size), int(c["k"])
    cache = LatentCache(kv=dev(c["kv"]), kv_scales=dev(c["kv_scales"]), idx_keys=fp8_from_bits(c["idx_key_bits"]),
                        row_start=dev(c["row_start"]), row_count=dev(c["lens"].astype(np.int32)),
                        max_rows=int(c["lens"].max()))
    hist = torch.zeros((B, 2048), dtype=torch.int32, device="cuda")   # the scan counts the selection's first digit
    out, ids, scores = sparse_decode_step(dev(c["q"], torch.bfloat16), dev(c["idx_q"], torch.bfloat16),
                                          dev(c["idx_w"]), cache, k=k, scale=c["scale"], d_v=c["d_v"],
                                          return_ids=True, return_scores=True, digit_hist=hist)
    assert int(hist.abs().sum()) == 0                                  # ... and the selection leaves it clear
    out_b, ids_b = sparse_decode_step(dev(c["q"], torch.bfloat16), dev(c["idx_q"], torch.bfloat16), dev(c["idx_w"]),
                                      cache, k=k, scale=c["scale"], d_v=c["d_v"], return_ids=True)
    assert torch.equal(ids, ids_b) and torch.equal(out, out_b)        # same step without the fused counting
    # --- top-k over EVERY row, on the device: ascending distinct valid ids, and nothing left out beats anything taken
    rs, ln = dev(c["row_start"]), dev(c["lens"])
    assert ids.dtype == torch.int32 and tuple(ids.shape) == (B, k)
    assert torch.all(ids[:, 1:] > ids[:, :-1]) and torch.all(ids >= 0) and torch.all(ids < ln[:, None])
    taken = torch.gather(scores, 0, (rs[:, None] + ids.long()).reshape(-1)).reshape(B, k)
    for b in range(B):
        row = scores[int(rs[b]): int(rs[b]) + int(ln[b])].clone()
        kth = taken[b].min()
        row[ids[b].long()] = -float("inf")
        rest = row.max()
        assert rest <= kth
        if rest == kth:   # a tie at the boundary goes to the lower id
            tied_out = torch.nonzero(row == kth).reshape(-1)
            tied_in = ids[b][taken[b] == kth]
            assert tied_in.max() < tied_out.min()
    # --- scores of EVERY sequence against the oracle; the selection against the oracle's, swaps allowed only among
    # near-ties of the k-th score (the two sides round the scores differently); attention of every fourth sequence
    sc = scores.cpu().numpy()
    idn = ids.cpu().numpy()
    margins = []
    for b in range(B):
        s, n = int(c["row_start"][b]), int(c["lens"][b])
        kb = synth.e4m3_bits_to_f32(c["idx_key_bits"][s:s + n])
        ref_scores = ds4.indexer_scores(c["idx_q"][b][None], kb, c["idx_w"][b][None])[0]
        np.testing.assert_allclose(sc[s:s + n], ref_scores, rtol=2e-4, atol=2e-3)
        order = np.sort(ref_scores)[::-1]
        kth = order[k - 1]
        margins.append(float(kth - order[k]) / max(1.0, abs(float(kth))))   # relative gap at the k-th boundary
        diff = np.setxor1d(idn[b], ds4.topk_ids(ref_scores, k)[0])
        if diff.size:
            assert np.all(np.abs(ref_scores[diff] - kth) <= 1e-3 * max(1.0, abs(kth))), (b, diff)
        if b % 4:
            continue
        sel = idn[b].astype(np.int64)
        ref = ds4.indexed_mixed_attention_decode(c["q"][b], None, c["kv"][s:s + n][sel], np.arange(k), None, pos0=0,
                                                 window=0, ratio=0, scale=c["scale"], d_v=c["d_v"],
                                                 kv_scales=c["kv_scales"][s:s + n][sel])
        assert max_abs(out[b], ref) <= 2e-2
    print(f"k-th boundary margins (relative): min {min(margins):.2e}, median {float(np.median(margins)):.2e}")


def test_qwen_prefill_at_full_size():
    """S = 8192, 16 query heads over 2 KV heads, head_dim 256, bf16: every head of four query tiles (first, two in
    the middle, last) against a float64 evaluation of those rows."""
    need_gpu()
    c = synth.config2()
    t = lambda x: torch.from_numpy(x).cuda().to(torch.bfloat16)  # noqa: E731
    q, k, v, g = t(c["q"]), t(c["k"]), t(c["v"]), t(c["gate"])
    out = sdpa_fa_prefill(q, k, v, c["scale"], gate=g, layout="lhd").float().cpu().numpy()
    S, Hq, D = c["q"].shape
    group = Hq // c["k"].shape[1]
    for h in range(Hq):
        kk = c["k"][:, h // group].astype(np.float64)
        vv = c["v"][:, h // group].astype(np.float64)
        for r0 in (0, 2688, 4032, S - 128):
            rows = np.arange(r0, r0 + 128)
            n_keys = r0 + 128                      # later keys are masked for every row of the tile
            s = (c["q"][rows, h].astype(np.float64) @ kk[:n_keys].T) * c["scale"]
            s[np.arange(n_keys)[None, :] > rows[:, None]] = -np.inf
            p = np.exp(s - s.max(axis=1, keepdims=True))
            ref = (p @ vv[:n_keys]) / p.sum(axis=1, keepdims=True)
            ref = ref / (1.0 + np.exp(-c["gate"][rows, h].astype(np.float64)))
            assert np.abs(out[rows, h] - ref).max() <= 2e-2


def test_chunked_sparse_prefill_at_full_size():
    """One 4096-token chunk at the end of a 131072-token context over 32768 ratio-4 compressed rows, top-k 2048 per
    token, bf16: 64 tokens spread over the chunk (and its first and last) against the oracle (scores -> selection ->
    attention)."""
    need_gpu()
    from moespresso_b200.deepseek_v4.prefill_step import sparse_prefill_step
    c = synth.config4()
    T, H, Dqk = c["q"].shape
    R, k = c["kv"].shape[0], int(c["k"])
    bf = lambda x: torch.from_numpy(x).cuda().to(torch.bfloat16)  # noqa: E731
    out, ids = sparse_prefill_step(bf(c["q"]), bf(c["kv"]), bf(c["idx_q"]), bf(c["idx_keys"]), dev(c["idx_w"]),
                                   pos0=int(c["pos0"]), ratio=int(c["ratio"]), k=k, scale=c["scale"], d_v=c["d_v"],
                                   window=0, return_ids=True)
    assert tuple(out.shape) == (T, H, c["d_v"]) and tuple(ids.shape) == (T, k)
    vis = (int(c["pos0"]) + torch.arange(T, device="cuda") + 1) // int(c["ratio"])
    assert torch.all(ids[:, 1:] > ids[:, :-1]) and torch.all(ids >= 0) and torch.all(ids < vis[:, None])
    ids_n = ids.cpu().numpy()
    for t in sorted(set(range(0, T, 65)) | {1, T - 1}):
        v = int(vis[t])
        ref_scores = ds4.indexer_scores(c["idx_q"][t][None], c["idx_keys"][:v], c["idx_w"][t][None])[0]
        ref_ids = ds4.topk_ids(ref_scores, k)[0]
        diff = np.setxor1d(ids_n[t], ref_ids)
        if diff.size:   # the two sides round the scores differently: only near-ties of the k-th score may swap
            kth = np.sort(ref_scores)[::-1][k - 1]
            assert np.all(np.abs(ref_scores[diff] - kth) <= 2e-3 * max(1.0, abs(kth)))
        sel = ids_n[t].astype(np.int64)
        ref = ds4.indexed_mixed_attention_decode(c["q"][t], None, c["kv"][sel], np.arange(k), None, pos0=0, window=0,
                                                 ratio=0, scale=c["scale"], d_v=c["d_v"])
        assert max_abs(out[t], ref) <= 2e-2
