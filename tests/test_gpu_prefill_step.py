"""Chunked ratio-4 sparse prefill (scores -> top-k -> attention) against the oracle."""
import numpy as np
import pytest
import torch

from moespresso_b200.deepseek_v4.prefill_step import sparse_prefill_step
from oracle import ds4
from tests.gpu_util import bf16_round, dev, max_abs, need_gpu
from tests.test_gpu_decode_step import boundary_exact

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("T,R,k,chunk", [(40, 700, 64, 16), (9, 50, 512, 256)])
def test_prefill_step_bf16(T, R, k, chunk):
    need_gpu()
    rng = np.random.default_rng(T + R)
    H, Dqk, Dv, Hi, Di, ratio = 64, 576, 512, 16, 64, 4
    pos0 = R * ratio - T          # the chunk ends at the frontier of the compressed pool
    q = bf16_round(rng.standard_normal((T, H, Dqk)))
    kv = bf16_round(rng.standard_normal((R, Dqk)))
    iq = bf16_round(rng.standard_normal((T, Hi, Di)))
    ik = bf16_round(rng.standard_normal((R, Di)))
    iw = (rng.standard_normal((T, Hi)) / 4).astype(np.float32)
    sinks = rng.standard_normal(H).astype(np.float32)
    bf = torch.bfloat16
    out, ids = sparse_prefill_step(dev(q, bf), dev(kv, bf), dev(iq, bf), dev(ik, bf), dev(iw), pos0=pos0, ratio=ratio,
                                   k=k, scale=Dqk ** -0.5, d_v=Dv, sinks=dev(sinks), window=0, token_chunk=chunk,
                                   return_ids=True)
    ids = ids.cpu().numpy()
    scores = ds4.indexer_scores(iq, ik, iw, pos0=pos0, ratio=ratio)
    if R > k:
        from moespresso_b200.deepseek_v4.indexed_attention_kernel import indexer_scores_tiled_live
        got_scores = indexer_scores_tiled_live(dev(iq, bf).permute(1, 0, 2)[None], dev(iw)[None], dev(ik, bf)[None],
                                               pos0=pos0, ratio=ratio)[0].cpu().numpy()
        for t in range(T):
            boundary_exact(ids[t], got_scores[t], scores[t], k)
    ref = ds4.indexed_mixed_attention_prefill(q, None, kv, ids, sinks, pos0=pos0, window=0, ratio=ratio,
                                              scale=Dqk ** -0.5, d_v=Dv)
    assert out.shape == (T, H, Dv)
    assert max_abs(out, ref) <= 2e-2


def test_prefill_step_fp8_keys_one_token_tail_chunk():
    """FP8 index keys and T % token_chunk == 1: the last score launch holds a single token and must still carry
    the causal row mask (rows >= (pos + 1) // ratio never selected)."""
    need_gpu()
    from moespresso_b200 import synth
    from tests.gpu_util import fp8_from_bits
    rng = np.random.default_rng(5)
    T, R, k, chunk = 17, 600, 64, 16
    H, Dqk, Dv, Hi, Di, ratio = 64, 576, 512, 16, 64, 4
    pos0 = 1200                      # visible rows 300 .. 304 of 600: half of the pool is masked
    q = bf16_round(rng.standard_normal((T, H, Dqk)))
    kv = bf16_round(rng.standard_normal((R, Dqk)))
    iq = bf16_round(rng.standard_normal((T, Hi, Di)))
    bits = synth.to_e4m3_bits(rng.standard_normal((R, Di)).astype(np.float32))
    ik = synth.e4m3_bits_to_f32(bits)
    iw = (rng.standard_normal((T, Hi)) / 4).astype(np.float32)
    bf = torch.bfloat16
    out, ids = sparse_prefill_step(dev(q, bf), dev(kv, bf), dev(iq, bf), fp8_from_bits(bits), dev(iw), pos0=pos0,
                                   ratio=ratio, k=k, scale=Dqk ** -0.5, d_v=Dv, window=0, token_chunk=chunk,
                                   return_ids=True)
    ids = ids.cpu().numpy()
    for t in range(T):
        vis = (pos0 + t + 1) // ratio
        assert ids[t].max() < vis and ids[t].min() >= 0
    ref = ds4.indexed_mixed_attention_prefill(q, None, kv, ids, None, pos0=pos0, window=0, ratio=ratio,
                                              scale=Dqk ** -0.5, d_v=Dv)
    assert max_abs(out, ref) <= 2e-2
    scores = ds4.indexer_scores(iq, ik, iw, pos0=pos0, ratio=ratio)
    for t in range(T):               # t = T - 1 is the one-token launch
        assert np.all(np.isfinite(scores[t][ids[t]]))
