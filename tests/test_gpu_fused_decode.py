"""The reference-named fused decode operators (composed here from the package's operators) against the oracle."""
import numpy as np
import pytest
import torch

from moespresso_b200.deepseek_v4 import attention as att
from moespresso_b200.deepseek_v4.decode_attention_kernel import fused_decode_prep, fused_decode_sdpa
from oracle import ds4
from tests.gpu_util import dev, need_gpu

pytestmark = pytest.mark.gpu


def _inv_freq():
    return att.rope_inverse_frequencies(64, att.DS4_COMPRESS_ROPE_BASE, att.DS4_YARN).astype(np.float32)


@pytest.mark.parametrize("n_heads,n_rows,topk,pos,qdtype", [(64, 961, 512, 3843, torch.float32),
                                                             (64, 4000, 512, 65535, torch.bfloat16),
                                                             (16, 300, 64, 7, torch.float16)])
def test_fused_decode_prep(n_heads, n_rows, topk, pos, qdtype):
    need_gpu()
    rng = np.random.default_rng(n_rows + pos)
    q = dev(rng.standard_normal((n_heads, 128), dtype=np.float32)).to(qdtype)
    pooled = ds4.indexer_qat(rng.standard_normal((n_rows, 128), dtype=np.float32))
    weights = (rng.standard_normal(n_heads, dtype=np.float32) * n_heads ** -0.5).astype(np.float32)
    kv_row = (rng.standard_normal(512) * 2).astype(np.float16)
    inv = _inv_freq()
    params = torch.tensor([pos, 5], dtype=torch.int32, device="cuda")
    sel, row, scores = fused_decode_prep(q, dev(pooled), dev(weights), dev(kv_row), dev(inv), params,
                                         scale=128 ** -0.5, topk=topk)
    assert sel.dtype == torch.int32 and tuple(sel.shape) == (topk,)
    assert row.dtype == torch.float16 and tuple(row.shape) == (512,)
    exp_scores = ds4.fused_qat_indexer_scores(q.float().cpu().numpy(), pooled, weights, 128 ** -0.5)
    np.testing.assert_allclose(scores.cpu().numpy(), exp_scores, rtol=1e-5, atol=1e-5)
    # the selection is the exact top-k of the scores the device produced (ties to the lower row), ascending
    np.testing.assert_array_equal(sel.cpu().numpy(), ds4.topk_ids(scores.cpu().numpy(), topk)[0])
    np.testing.assert_array_equal(row.cpu().numpy().view(np.uint16),
                                  ds4.fused_decode_prep_row(kv_row, pos, inv).view(np.uint16))


@pytest.mark.parametrize("n_heads,window_rows,n_rows,topk,pos", [(64, 128, 961, 512, 3843), (8, 128, 200, 16, 130),
                                                                  (64, 128, 5000, 512, 20000)])
def test_fused_decode_sdpa(n_heads, window_rows, n_rows, topk, pos):
    need_gpu()
    rng = np.random.default_rng(n_rows * 7 + n_heads)
    q = rng.standard_normal((n_heads, 512)).astype(np.float16)
    window = rng.standard_normal((window_rows, 512)).astype(np.float16)
    row = rng.standard_normal(512).astype(np.float16)
    pooled = rng.standard_normal((n_rows, 512)).astype(np.float16)
    sel = np.sort(rng.choice(n_rows, size=topk, replace=False)).astype(np.int32)
    sinks = rng.standard_normal(n_heads).astype(np.float16)
    inv = _inv_freq()
    write_idx = pos % window_rows
    params = torch.tensor([pos, write_idx], dtype=torch.int32, device="cuda")
    got = fused_decode_sdpa(dev(q), dev(window), dev(row), dev(pooled), dev(sel), dev(sinks), dev(inv), params,
                            scale=512 ** -0.5)
    assert got.dtype == torch.float16 and tuple(got.shape) == (n_heads, 512)
    exp = ds4.fused_decode_sdpa(q, window, row, pooled, sel, sinks, inv, pos, write_idx, 512 ** -0.5)
    # the reference's own tolerance for its float16 attention kernels
    assert np.abs(got.float().cpu().numpy() - exp.astype(np.float32)).max() <= 2e-3


def test_fused_decode_rejects_bad_inputs():
    need_gpu()
    z = lambda *s, dt=torch.float32: torch.zeros(s, device="cuda", dtype=dt)  # noqa: E731
    params = torch.tensor([3, 1], dtype=torch.int32, device="cuda")
    with pytest.raises(ValueError, match="smaller than n_rows"):
        fused_decode_prep(z(8, 128), z(16, 128), z(8), z(512, dt=torch.float16), z(32), params, scale=0.1, topk=16)
    with pytest.raises(ValueError, match=r"float16 \[512\]"):
        fused_decode_prep(z(8, 128), z(16, 128), z(8), z(512), z(32), params, scale=0.1, topk=4)
    with pytest.raises(ValueError, match="between 1 and 64 heads"):
        fused_decode_prep(z(65, 128), z(16, 128), z(65), z(512, dt=torch.float16), z(32), params, scale=0.1, topk=4)
    with pytest.raises(ValueError, match=r"q must be float16"):
        fused_decode_sdpa(z(8, 512), z(128, 512, dt=torch.float16), z(512, dt=torch.float16),
                          z(16, 512, dt=torch.float16), torch.zeros(4, dtype=torch.int32, device="cuda"),
                          z(8, dt=torch.float16), z(32), params, scale=0.1)
