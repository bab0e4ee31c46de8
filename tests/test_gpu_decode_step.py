"""Whole sparse decode step (indexer score -> top-k -> sparse attention) against the oracle."""
import numpy as np
import pytest
import torch

from moespresso_b200 import synth
from moespresso_b200.deepseek_v4.decode_step import LatentCache, sparse_decode_step
from oracle import ds4
from tests.gpu_util import dev, fp8_from_bits, max_abs, need_gpu

pytestmark = pytest.mark.gpu


def boundary_exact(ids_gpu, scores_gpu, scores_ref, k):
    """Top-k parity when the two sides computed scores with different rounding: the GPU
    selection must be the exact top-k of the GPU's own score bits, and every row on which
    it differs from the oracle's selection must sit within rounding distance of the k-th
    boundary of the oracle's scores."""
    own = ds4.topk_ids(scores_gpu, k)[0]
    np.testing.assert_array_equal(ids_gpu, own)
    ref = ds4.topk_ids(scores_ref, k)[0]
    diff = np.setxor1d(ids_gpu[ids_gpu >= 0], ref[ref >= 0])
    if diff.size:
        kth = np.sort(scores_ref[np.isfinite(scores_ref)])[::-1][min(k, np.isfinite(scores_ref).sum()) - 1]
        assert np.all(np.abs(scores_ref[diff] - kth) <= 1e-3 * max(1.0, abs(kth)))
    return diff.size


def test_config1_step_fp32():
    need_gpu()
    c = synth.config1()
    cache = LatentCache(kv=dev(c["kv"]), kv_scales=None, idx_keys=dev(c["idx_keys"]),
                        row_start=dev(np.zeros(1, np.int64)), row_count=dev(np.array([4096], np.int32)),
                        max_rows=4096)
    out, ids, scores = sparse_decode_step(dev(c["q"])[None], dev(c["idx_q"])[None], dev(c["idx_w"])[None], cache,
                                          k=c["k"], scale=c["scale"], d_v=c["d_v"], return_ids=True,
                                          return_scores=True)
    ref_scores, ref_ids, ref_out = ds4.sparse_decode_step(c["q"], c["kv"], c["idx_q"], c["idx_keys"], c["idx_w"],
                                                          k=c["k"], scale=c["scale"], d_v=c["d_v"])
    np.testing.assert_allclose(scores.cpu().numpy(), ref_scores, rtol=1e-5, atol=1e-5)
    ndiff = boundary_exact(ids[0].cpu().numpy(), scores.cpu().numpy(), ref_scores, c["k"])
    if ndiff == 0:
        assert max_abs(out[0], ref_out) <= 1e-4
    else:  # attention over the GPU's own selection
        ref2 = ds4.indexed_mixed_attention_decode(c["q"], None, c["kv"], ids[0].cpu().numpy(), None, pos0=0,
                                                  window=0, ratio=0, scale=c["scale"], d_v=c["d_v"])
        assert max_abs(out[0], ref2) <= 1e-4


@pytest.mark.parametrize("lens", [[5000, 2049, 40000, 300], [50000, 47000]])
def test_config3_shaped_step(lens):
    need_gpu()
    c = synth.config3(seed=1, lens=lens)
    cache = LatentCache(kv=dev(c["kv"]), kv_scales=dev(c["kv_scales"]), idx_keys=fp8_from_bits(c["idx_key_bits"]),
                        row_start=dev(c["row_start"]), row_count=dev(c["lens"].astype(np.int32)),
                        max_rows=int(max(lens)))
    out, ids, scores = sparse_decode_step(dev(c["q"], torch.bfloat16), dev(c["idx_q"], torch.bfloat16),
                                          dev(c["idx_w"]), cache, k=c["k"], scale=c["scale"], d_v=c["d_v"],
                                          return_ids=True, return_scores=True)
    keys = synth.e4m3_bits_to_f32(c["idx_key_bits"])
    scores = scores.cpu().numpy(); ids = ids.cpu().numpy()
    for b, n in enumerate(lens):
        s = int(c["row_start"][b])
        ref_scores = ds4.indexer_scores(c["idx_q"][b][None], keys[s:s + n], c["idx_w"][b][None])[0]
        np.testing.assert_allclose(scores[s:s + n], ref_scores, rtol=2e-4, atol=2e-3)
        boundary_exact(ids[b], scores[s:s + n], ref_scores, c["k"])
        ref = ds4.indexed_mixed_attention_decode(c["q"][b], None, c["kv"][s:s + n], ids[b], None, pos0=0, window=0,
                                                 ratio=0, scale=c["scale"], d_v=c["d_v"],
                                                 kv_scales=c["kv_scales"][s:s + n])
        assert max_abs(out[b], ref) <= 2e-2


@pytest.mark.parametrize("graph", [True, False])
def test_plan_matches_eager_step(graph):
    """The CUDA-graph plan returns the bits of the eager step, from device or pinned-host inputs."""
    need_gpu()
    from moespresso_b200.deepseek_v4.decode_step import SparseDecodePlan
    c = synth.config3(seed=3, lens=[3000, 2500, 6000])
    cache = LatentCache(kv=dev(c["kv"]), kv_scales=dev(c["kv_scales"]), idx_keys=fp8_from_bits(c["idx_key_bits"]),
                        row_start=dev(c["row_start"]), row_count=dev(c["lens"].astype(np.int32)), max_rows=6000)
    q, iq, iw = dev(c["q"], torch.bfloat16), dev(c["idx_q"], torch.bfloat16), dev(c["idx_w"])
    eager = sparse_decode_step(q, iq, iw, cache, k=c["k"], scale=c["scale"], d_v=c["d_v"], out_dtype=torch.bfloat16)
    plan = SparseDecodePlan(cache, heads=64, d_qk=576, idx_heads=16, idx_dim=64, k=c["k"], scale=c["scale"],
                            d_v=c["d_v"], q_dtype=torch.bfloat16, out_dtype=torch.bfloat16, graph=graph)
    out = plan.run(q, iq, iw)
    torch.cuda.synchronize()
    assert torch.equal(out, eager)
    plan.q.zero_()
    out = plan.run(q.cpu().pin_memory(), iq.cpu().pin_memory(), iw.cpu().pin_memory())
    torch.cuda.synchronize()
    assert torch.equal(out, eager)
    plan.packed.zero_()
    host, (qv, iqv, iwv) = plan.host_buffer()
    qv.copy_(q.cpu())
    iqv.copy_(iq.cpu())
    iwv.copy_(iw.cpu())
    out = plan.run_packed(host)
    torch.cuda.synchronize()
    assert torch.equal(out, eager)


def test_plan_with_16bit_cache():
    """bf16 latent cache: the attention kernel gathers rows by TMA (tensor maps passed as kernel parameters); the
    captured graph must replay to the eager step's bits and stay within the 16-bit bound of the oracle."""
    need_gpu()
    from moespresso_b200.deepseek_v4.decode_step import SparseDecodePlan
    lens = [3000, 2500, 6000]
    c = synth.config3(seed=4, lens=lens)
    kv = synth.to_bf16_f32(c["kv"].astype(np.float32) * c["kv_scales"].astype(np.float32)[:, None])   # dequantised rows
    cache = LatentCache(kv=dev(kv, torch.bfloat16), kv_scales=None, idx_keys=fp8_from_bits(c["idx_key_bits"]),
                        row_start=dev(c["row_start"]), row_count=dev(c["lens"].astype(np.int32)), max_rows=6000)
    q, iq, iw = dev(c["q"], torch.bfloat16), dev(c["idx_q"], torch.bfloat16), dev(c["idx_w"])
    eager, ids = sparse_decode_step(q, iq, iw, cache, k=c["k"], scale=c["scale"], d_v=c["d_v"], return_ids=True)
    plan = SparseDecodePlan(cache, heads=64, d_qk=576, idx_heads=16, idx_dim=64, k=c["k"], scale=c["scale"],
                            d_v=c["d_v"], q_dtype=torch.bfloat16)
    for _ in range(2):
        out = plan.run(q, iq, iw)
        torch.cuda.synchronize()
        assert torch.equal(out, eager)
    ids = ids.cpu().numpy()
    # The 2e-2 bound is stated for unit-scale values.  These rows reach |v| = 12.7 (int8 x scale), where bf16 itself
    # resolves 0.0625 and the bf16 softmax weights (8 significant bits) move an output by up to |v| * 2^-9: the
    # bound scales with the table's magnitude.
    tol = 2e-2 * max(1.0, float(np.abs(kv).max()) / 4.0)
    for b, n in enumerate(lens):
        s = int(c["row_start"][b])
        ref = ds4.indexed_mixed_attention_decode(c["q"][b], None, kv[s:s + n], ids[b], None, pos0=0, window=0, ratio=0,
                                                 scale=c["scale"], d_v=c["d_v"])
        assert max_abs(eager[b], ref) <= tol
