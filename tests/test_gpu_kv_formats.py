"""Cache-row formats through the C ABI: FP8 KV round trip (served and replay forms) and the int8 quantiser."""
import os

import numpy as np
import pytest
import torch

from moespresso_b200.deepseek_v4.decode_attention_kernel import fp8_kv_prefix_rows
from moespresso_b200.deepseek_v4.decode_step import quantize_kv_int8
from oracle import ds4
from tests.gpu_util import dev, need_gpu

pytestmark = pytest.mark.gpu


def _golden():
    return np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "fp8kv_golden.npz"))


def test_fp8_replay_form_matches_reference_vectors_bit_for_bit():
    """The reference's own NumPy outputs, through the CUDA kernel."""
    need_gpu()
    g = _golden()
    got = fp8_kv_prefix_rows(dev(g["rows"]), replay=True).cpu().numpy()
    np.testing.assert_array_equal(got.view(np.uint32), g["rounded"].view(np.uint32))


def _adversarial_rows(rng):
    rows = [rng.standard_normal((256, 512)), rng.standard_normal((64, 512)) * 2.0 ** 20,
            rng.standard_normal((64, 512)) * 2.0 ** -20, np.zeros((2, 512))]
    # block maxima within a few ulp of 448 * 2^k (the ceil boundary of the block scale)
    b = rng.standard_normal((128, 8, 64))
    b = b / np.abs(b).max(-1, keepdims=True) * 448.0 * 2.0 ** rng.integers(-20, 20, size=(128, 8, 1))
    b = b * (1.0 + rng.integers(-4, 5, size=(128, 8, 1)) * 1.1920929e-07)
    rows.append(b.reshape(128, 512))
    # exact midpoints between table values at scale 1 (one element pins the block maximum to 448)
    t = ds4.E4M3FN_VALUES.astype(np.float64)
    mids = (t[:-1] + t[1:]) / 2
    m = rng.choice(mids, size=(64, 512)) * np.where(rng.random((64, 512)) < 0.5, 1.0, -1.0)
    m[:, ::64] = 448.0
    rows.append(m)
    out = np.concatenate(rows).astype(np.float32)
    out[1, 7] = -0.0
    return out


@pytest.mark.parametrize("replay", [False, True])
def test_fp8_rows_bitexact_against_oracle(replay):
    need_gpu()
    rows = _adversarial_rows(np.random.default_rng(5))
    got = fp8_kv_prefix_rows(dev(rows).reshape(2, -1, 512), replay=replay).cpu().numpy().reshape(-1, 512)
    exp = ds4.fp8_kv_round_replay(rows) if replay else ds4.fp8_kv_prefix_rows(rows)
    np.testing.assert_array_equal(got.view(np.uint32), exp.view(np.uint32))
    np.testing.assert_array_equal(got[:, 448:].view(np.uint32), rows[:, 448:].view(np.uint32))


def test_fp8_rows_nan_and_errors():
    need_gpu()
    rows = np.random.default_rng(1).standard_normal((4, 512)).astype(np.float32)
    rows[2, 70] = np.nan
    got = fp8_kv_prefix_rows(dev(rows)).cpu().numpy()
    assert got[2, 70] == 0.0 and not np.isnan(got).any()        # a NaN element becomes 0; its block is not disturbed
    np.testing.assert_array_equal(got.view(np.uint32), ds4.fp8_kv_prefix_rows(rows).view(np.uint32))
    with pytest.raises(ValueError, match="512-wide"):
        fp8_kv_prefix_rows(torch.zeros((3, 576), device="cuda"))
    with pytest.raises(ValueError, match="must be float32"):
        fp8_kv_prefix_rows(torch.zeros((3, 512), device="cuda", dtype=torch.float16))
    with pytest.raises(ValueError, match="at least one row"):
        fp8_kv_prefix_rows(torch.zeros((0, 512), device="cuda"))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
def test_quantize_kv_int8(dtype):
    need_gpu()
    rng = np.random.default_rng(3)
    x = dev((rng.standard_normal((300, 576)) * np.exp(rng.uniform(-6, 2, size=(300, 1)))).astype(np.float32)).to(dtype)
    x[7] = 0
    q, s = quantize_kv_int8(x)
    eq, es = ds4.quantize_kv_int8(x.float().cpu().numpy())
    np.testing.assert_array_equal(s.cpu().numpy().view(np.uint16), es.view(np.uint16))
    np.testing.assert_array_equal(q.cpu().numpy(), eq)
    back = q.float() * s.float()[:, None]
    assert torch.all((back - x.float()).abs() <= 0.5 * s.float()[:, None] * 1.001 + 1e-30)
    # the decode operators read this format: a one-row sanity check through sparse attention happens elsewhere


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-7), (torch.bfloat16, 0.0), (torch.float16, 0.0)])
def test_rope_tail_against_reference_vectors(dtype, tol):
    """apply_rope_tail through the CUDA kernel against outputs of the reference's NumPy function."""
    need_gpu()
    from moespresso_b200.deepseek_v4 import attention as pkg
    g = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "rope_golden.npz"))
    x = dev(g["x"]).to(dtype)
    fwd = pkg.apply_rope_tail(x, g["pos"], base=pkg.DS4_COMPRESS_ROPE_BASE, yarn=pkg.DS4_YARN)
    assert fwd.dtype == dtype and fwd.shape == x.shape
    if dtype == torch.float32:
        np.testing.assert_allclose(fwd.cpu().numpy(), g["fwd_yarn"], rtol=0, atol=tol * 8)
        inv = pkg.apply_rope_tail(fwd, torch.as_tensor(g["pos"]), base=pkg.DS4_COMPRESS_ROPE_BASE, yarn=pkg.DS4_YARN,
                                  inverse=True)
        np.testing.assert_allclose(inv.cpu().numpy(), g["x"], rtol=0, atol=1e-5)
        swa = pkg.apply_rope_tail(x, g["pos"], base=pkg.DS4_SWA_ROPE_BASE)
        np.testing.assert_allclose(swa.cpu().numpy(), g["fwd_swa"], rtol=0, atol=tol * 8)
    else:
        exp = ds4.apply_rope_tail(x.float().cpu().numpy(), g["pos"], base=pkg.DS4_COMPRESS_ROPE_BASE, yarn=pkg.DS4_YARN)
        exp = torch.from_numpy(exp).to(dtype)                         # one rounding from float64 math
        diff = (fwd.float().cpu() - exp.float()).abs().max().item()
        assert diff <= 2 ** -7 * 8                                    # at most one unit in the last place of the 16-bit type
    np.testing.assert_array_equal(fwd[..., :448].float().cpu().numpy(), x[..., :448].float().cpu().numpy())
    same = x.clone()
    pkg.apply_rope_tail(same, g["pos"], base=pkg.DS4_COMPRESS_ROPE_BASE, yarn=pkg.DS4_YARN, out=same)   # in place
    assert torch.equal(same, fwd)
    with pytest.raises(ValueError, match="positions length"):
        pkg.apply_rope_tail(x, g["pos"][:3], base=10000.0)
    with pytest.raises(ValueError, match="positive even"):
        pkg.apply_rope_tail(x, g["pos"], base=10000.0, rope_dim=3)
