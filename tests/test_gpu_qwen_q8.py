"""Affine 8-bit KV format (group 64), the q8 prefill route and the q8 decode attention of the Qwen wrapper against
the CPU oracle.  Format: bit-exact packed words, scales and biases.  Attention: the reference's own bound for
this route, relative L2 1e-4 ... of its fp32 kernel against the composed path; here the operands are 16-bit, so
the bound is the 16-bit one (max-abs 2e-2) against the float64 composed path."""
import numpy as np
import pytest
import torch

from moespresso_b200.qwen import full_attention as fa
from oracle import qwen
from tests.gpu_util import bf16_round, dev, f16_round, max_abs, need_gpu
from tests.test_gpu_flash_prefill import _Inner

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("kind", ["bf16", "f16", "f32"])
def test_format_round_trip_is_bit_exact(kind):
    need_gpu()
    rng = np.random.default_rng(3)
    rnd = {"bf16": bf16_round, "f16": f16_round, "f32": lambda x: np.asarray(x, np.float32)}[kind]
    tdt = {"bf16": torch.bfloat16, "f16": torch.float16, "f32": torch.float32}[kind]
    x = rnd(rng.standard_normal((37, 2, 256)) * np.exp(rng.uniform(-3, 3, size=(37, 2, 1))))
    x[3, 0, :64] = 0.25            # a constant group: scale 0
    x[4, 1, 64:128] = 0.0
    p, s, b = fa.quantize_affine_q8(dev(x, tdt))
    rp, rs, rb = qwen.affine_q8_quantize(x, kind)
    assert p.shape == (37, 2, 64) and s.shape == (37, 2, 4)
    np.testing.assert_array_equal(s.float().cpu().numpy(), rs)
    np.testing.assert_array_equal(b.float().cpu().numpy(), rb)
    np.testing.assert_array_equal(p.cpu().numpy().view(np.uint32), rp)
    d = fa.dequantize_affine_q8(p, s, b, dtype=torch.float32)
    np.testing.assert_allclose(d.cpu().numpy(), qwen.affine_q8_dequantize(rp, rs, rb), rtol=0, atol=1e-6 * np.abs(x).max())
    # error of the format itself: half a step per element, plus up to 255 x 2^-9 steps where the step was rounded
    # to a 16-bit type (the top elements then land beyond 255 and clip)
    steps = 0.5 * 1.01 if kind == "f32" else 1.0
    assert np.all(np.abs(d.cpu().numpy() - x) <= steps * np.repeat(rs, 64, axis=-1) + 1e-7)


@pytest.mark.parametrize("L,P", [(256, 2065), (135, 700), (64, 1)])
def test_prefill_q8_matches_composed_path(L, P):
    """Past in the cache format, self chunk through the q8 round trip (the reference's contract for the route)."""
    need_gpu()
    rng = np.random.default_rng(L + P)
    Hq, Hkv, D = 16, 2, 256
    q = bf16_round(0.1 * rng.standard_normal((L, Hq, D)) * 5)
    kp = bf16_round(0.5 * rng.standard_normal((P, Hkv, D)))
    vp = bf16_round(0.5 * rng.standard_normal((P, Hkv, D)))
    ks = bf16_round(0.5 * rng.standard_normal((L, Hkv, D)))
    vs = bf16_round(0.5 * rng.standard_normal((L, Hkv, D)))
    g = bf16_round(rng.standard_normal((L, Hq, D)))
    bf = torch.bfloat16
    cache = fa.QuantizedKVCache(Hkv, D, P + L + 8)
    cache.update_and_fetch(dev(kp, bf).permute(1, 0, 2)[None], dev(vp, bf).permute(1, 0, 2)[None])
    assert cache.offset == P
    past_k, past_v = cache.state
    self_k = fa.dequantize_affine_q8(*fa.quantize_affine_q8(dev(ks, bf).permute(1, 0, 2)[None]))
    self_v = fa.dequantize_affine_q8(*fa.quantize_affine_q8(dev(vs, bf).permute(1, 0, 2)[None]))
    out = fa.sdpa_fa_prefill_q8(dev(q, bf).permute(1, 0, 2)[None], *past_k, *past_v, self_k, self_v, 1.0 / 16.0,
                                bq=64, bk=16, stage=2, check=True)
    assert out.shape == (1, Hq, L, D)
    rk, rv = qwen.affine_q8_quantize(kp, "bf16"), qwen.affine_q8_quantize(vp, "bf16")
    sk = bf16_round(qwen.affine_q8_dequantize(*qwen.affine_q8_quantize(ks, "bf16")))
    sv = bf16_round(qwen.affine_q8_dequantize(*qwen.affine_q8_quantize(vs, "bf16")))
    ref = qwen.prefill_q8(q, rk, rv, sk, sv, scale=1.0 / 16.0)
    assert max_abs(out[0].permute(1, 0, 2), ref) <= 2e-2
    fused = fa.sdpa_fa_prefill_q8(dev(q, bf).permute(1, 0, 2)[None], *past_k, *past_v, self_k, self_v, 1.0 / 16.0,
                                  gate=dev(g, bf).reshape(1, L, Hq * D))
    refg = qwen.prefill_q8(q, rk, rv, sk, sv, g, scale=1.0 / 16.0)
    assert max_abs(fused.reshape(L, Hq, D), refg) <= 2e-2


@pytest.mark.parametrize("P,splits,qdt", [(40000, 128, "f32"), (33000, 128, "bf16"), (700, 16, "f32"), (5, 128, "f32")])
def test_decode_q8_matches_composed_path(P, splits, qdt):
    need_gpu()
    rng = np.random.default_rng(P)
    Hq, Hkv, D = 16, 2, 256
    q = rng.standard_normal((Hq, D)).astype(np.float32)
    if qdt == "bf16":
        q = bf16_round(q)
    k = bf16_round(0.5 * rng.standard_normal((P, Hkv, D)))
    v = bf16_round(0.5 * rng.standard_normal((P, Hkv, D)))
    bf = torch.bfloat16
    cache = fa.QuantizedKVCache(Hkv, D, P + 64)
    qk, qv = cache.update_and_fetch(dev(k, bf).permute(1, 0, 2)[None], dev(v, bf).permute(1, 0, 2)[None])
    tq = dev(q, torch.float32 if qdt == "f32" else bf)[None, :, None, :]
    out = fa.sdpa_decode_q8(tq, *qk, *qv, 1.0 / 16.0, group_size=64, bits=8, splits=splits, stage=2, compute=1, tile_c=16)
    assert out.shape == (1, Hq, 1, D) and out.dtype == tq.dtype
    kd = qwen.affine_q8_dequantize(*qwen.affine_q8_quantize(k, "bf16"))
    vd = qwen.affine_q8_dequantize(*qwen.affine_q8_quantize(v, "bf16"))
    s = np.einsum("hd,phd->hp", q.astype(np.float64), np.repeat(kd, Hq // Hkv, axis=1).astype(np.float64)) / 16.0
    p = np.exp(s - s.max(axis=1, keepdims=True))
    ref = np.einsum("hp,phd->hd", p / p.sum(axis=1, keepdims=True), np.repeat(vd, Hq // Hkv, axis=1).astype(np.float64))
    # fp16 operands on the tensor cores (keys, values and P rounded to 11 bits), fp32 accumulation
    assert max_abs(out[0, :, 0], ref) <= (2e-3 if qdt == "f32" else 2e-2)


@torch.no_grad()
def test_wrapper_routes_q8_prefill_and_decode():
    need_gpu()
    torch.manual_seed(1)
    Hq, Hkv, D, E = 16, 2, 256, 128
    inner = _Inner(Hq, Hkv, D, E)
    attn = fa.FlashPrefillD256Attention(inner)
    cache = fa.QuantizedKVCache(Hkv, D, 1024)
    x = torch.randn(1, 300, E, dtype=torch.bfloat16, device="cuda") * 0.5
    # an empty quantised cache is not eligible (offset >= 1 required): the stock path takes the first chunk
    attn(x[:, :10], mask="causal", cache=cache)
    assert inner.stock_calls == 1 and attn.rejected["cache"] == 1
    # seed the cache the way the stock path would have
    k0 = inner.k_proj(x[:, :100]).reshape(1, 100, Hkv, D).transpose(1, 2)
    v0 = inner.v_proj(x[:, :100]).reshape(1, 100, Hkv, D).transpose(1, 2)
    cache.update_and_fetch(k0, v0)
    y = attn(x[:, 100:300], mask="causal", cache=cache)
    assert y.shape == (1, 200, E) and cache.offset == 300 and attn.flash_calls == 1
    # composed reference: the whole cache dequantised (the self chunk's values ARE the cache's), causal over 300
    kd = fa.dequantize_affine_q8(*cache.state[0], dtype=torch.float32)[0].permute(1, 0, 2).cpu().numpy()
    vd = fa.dequantize_affine_q8(*cache.state[1], dtype=torch.float32)[0].permute(1, 0, 2).cpu().numpy()
    qg = inner.q_proj(x[:, 100:300]).reshape(1, 200, Hq, 2 * D).float()
    ref = qwen.causal_gqa_prefill(qg[0, ..., :D].cpu().numpy(), kd, vd, qg[0, ..., D:].cpu().numpy(), scale=D ** -0.5,
                                  past_len=100)
    yref = inner.o_proj(torch.from_numpy(ref.reshape(1, 200, Hq * D)).to(torch.bfloat16).cuda())
    assert float((y.float() - yref.float()).norm() / yref.float().norm()) < 2e-2
    # decode below the long-context threshold goes to the stock path
    attn(x[:, :1], mask=None, cache=cache)
    assert inner.stock_calls == 2 and attn.decode_calls == 0
