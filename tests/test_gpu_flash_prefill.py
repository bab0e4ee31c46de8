"""Causal GQA flash prefill (head_dim 256) against the CPU oracle; max-abs 2e-2 for 16-bit inputs."""
import numpy as np
import pytest
import torch

from moespresso_b200.qwen import full_attention as fa
from oracle import qwen
from tests.gpu_util import bf16_round, dev, f16_round, max_abs, need_gpu

pytestmark = pytest.mark.gpu


def _inputs(rng, S, past, Hq, Hkv, rnd, amp=0.5):
    D = 256
    q = rnd(amp * rng.standard_normal((S, Hq, D)))
    k = rnd(amp * rng.standard_normal((past + S, Hkv, D)))
    v = rnd(amp * rng.standard_normal((past + S, Hkv, D)))
    g = rnd(rng.standard_normal((S, Hq, D)))
    return q, k, v, g


@pytest.mark.parametrize("S,past,Hq,Hkv", [
    (128, 0, 2, 1),       # one q tile, two key tiles
    (256, 0, 16, 2),      # GQA 16/2
    (135, 2065, 4, 2),    # ragged tile over a past (the reference's short-tail case shape)
    (1000, 0, 2, 2),      # many tiles, ragged tail
    (64, 0, 2, 1),        # shorter than one tile
])
@pytest.mark.parametrize("dt", ["bf16", "f16"])
def test_matches_oracle(S, past, Hq, Hkv, dt):
    need_gpu()
    rng = np.random.default_rng(S + past)
    tdt = torch.bfloat16 if dt == "bf16" else torch.float16
    rnd = bf16_round if dt == "bf16" else f16_round
    q, k, v, g = _inputs(rng, S, past, Hq, Hkv, rnd)
    out = fa.sdpa_fa_prefill(dev(q, tdt), dev(k, tdt), dev(v, tdt), 1.0 / 16.0, gate=dev(g, tdt), layout="lhd",
                             check=True)
    ref = qwen.causal_gqa_prefill(q, k, v, g, scale=1.0 / 16.0, past_len=past)
    assert out.shape == (S, Hq, 256) and out.dtype == tdt
    assert max_abs(out, ref) <= 2e-2
    out_ng = fa.sdpa_fa_prefill(dev(q, tdt), dev(k, tdt), dev(v, tdt), 1.0 / 16.0, layout="lhd", check=True)
    assert max_abs(out_ng, qwen.causal_gqa_prefill(q, k, v, None, scale=1.0 / 16.0, past_len=past)) <= 2e-2


def test_gate_layout_without_tensor_map():
    """A gate whose row stride is not a multiple of its head stride cannot be described by a tensor map: the drain
    then reads the gate and writes the output with per-thread accesses.  Same result as the tiled drain."""
    need_gpu()
    rng = np.random.default_rng(9)
    S, Hq, Hkv, D = 300, 4, 2, 256
    q, k, v, g = _inputs(rng, S, 0, Hq, Hkv, bf16_round)
    tq, tk, tv = (dev(x, torch.bfloat16) for x in (q, k, v))
    row = Hq * (D + 8) + 8
    store = torch.zeros(S * row, dtype=torch.bfloat16, device="cuda")
    tg = store.as_strided((S, Hq, D), (row, D + 8, 1))
    tg.copy_(dev(g, torch.bfloat16))
    odd = fa.sdpa_fa_prefill(tq, tk, tv, 1.0 / 16.0, gate=tg, layout="lhd", check=True)
    tiled = fa.sdpa_fa_prefill(tq, tk, tv, 1.0 / 16.0, gate=dev(g, torch.bfloat16), layout="lhd", check=True)
    ref = qwen.causal_gqa_prefill(q, k, v, g, scale=1.0 / 16.0, past_len=0)
    assert max_abs(odd, ref) <= 2e-2 and max_abs(tiled, ref) <= 2e-2
    assert (odd.float() - tiled.float()).abs().max().item() <= 1e-2


def test_bhld_layout_and_peaked_softmax():
    """[1,H,L,D] operands as the reference wrapper passes them; large logits exercise the
    running-maximum rescale."""
    need_gpu()
    rng = np.random.default_rng(5)
    S, Hq, Hkv = 384, 4, 2
    q, k, v, g = _inputs(rng, S, 0, Hq, Hkv, bf16_round, amp=2.0)
    tq = dev(q, torch.bfloat16).permute(1, 0, 2)[None]
    tk = dev(k, torch.bfloat16).permute(1, 0, 2)[None]
    tv = dev(v, torch.bfloat16).permute(1, 0, 2)[None]
    tg = dev(g, torch.bfloat16).reshape(1, S, Hq * 256)
    out = fa.sdpa_fa_prefill(tq, tk, tv, 1.0 / 16.0, gate=tg, check=True)
    assert out.shape == (1, S, Hq * 256)
    ref = qwen.causal_gqa_prefill(q, k, v, g, scale=1.0 / 16.0).reshape(1, S, Hq * 256)
    assert max_abs(out, ref) <= 4e-2      # |V| is 4x the benchmark's amplitude here


class _Inner(torch.nn.Module):
    """A stand-in for the stock attention module the wrapper decorates (Linear projections, identity norms and rope)."""

    def __init__(self, Hq, Hkv, D, E):
        super().__init__()
        mk = lambda o: torch.nn.Linear(E, o, bias=False, dtype=torch.bfloat16, device="cuda")
        self.q_proj, self.k_proj, self.v_proj = mk(Hq * 2 * D), mk(Hkv * D), mk(Hkv * D)
        self.o_proj = torch.nn.Linear(Hq * D, E, bias=False, dtype=torch.bfloat16, device="cuda")
        self.q_norm = self.k_norm = torch.nn.Identity()
        self.num_attention_heads, self.num_key_value_heads, self.head_dim, self.scale = Hq, Hkv, D, D ** -0.5
        self.stock_calls = 0

    def rope(self, x, offset):
        return x

    def forward(self, x, mask=None, cache=None):   # the stock path: only counted here
        self.stock_calls += 1
        return torch.zeros_like(x)


@torch.no_grad()
def test_wrapper_module_routes_counts_and_delegates():
    need_gpu()
    torch.manual_seed(0)
    Hq, Hkv, D, E = 4, 2, 256, 128
    inner = _Inner(Hq, Hkv, D, E)
    model = type("M", (), {})()
    model.layers = [type("L", (), {"self_attn": inner})()]
    assert fa.install_flash_prefill_attention(model) == 1
    attn = model.layers[0].self_attn
    x = torch.randn(1, 200, E, dtype=torch.bfloat16, device="cuda") * 0.5
    cache = fa.DenseKVCache(Hkv, D, 512)
    y = attn(x, mask="causal", cache=cache)
    assert y.shape == (1, 200, E) and cache.offset == 200
    # composed fp32 reference of the same module
    qg = inner.q_proj(x).reshape(1, 200, Hq, 2 * D).float()
    qq, gg = qg[..., :D], qg[..., D:]
    kk = inner.k_proj(x).reshape(1, 200, Hkv, D).float()
    vv = inner.v_proj(x).reshape(1, 200, Hkv, D).float()
    ref = qwen.causal_gqa_prefill(qq[0].cpu().numpy(), kk[0].cpu().numpy(), vv[0].cpu().numpy(),
                                  gg[0].cpu().numpy(), scale=D ** -0.5)
    ref = torch.from_numpy(ref.reshape(1, 200, Hq * D)).to(torch.bfloat16).cuda()
    yref = inner.o_proj(ref)
    rel = float((y.float() - yref.float()).norm() / yref.float().norm())
    assert rel < 2e-2
    # a second chunk appends in place and attends over the first
    y2 = attn(x[:, :100], mask="causal", cache=cache)
    assert y2.shape == (1, 100, E) and cache.offset == 300
    # calls the routes do not take go to the wrapped module, as the reference falls back to the stock path
    attn(x[:, :1], mask="causal", cache=None)
    attn(x, mask=None, cache=None)
    assert inner.stock_calls == 2
    st = fa.flash_prefill_attention_stats(model)
    assert st["layers"] == 1 and st["dense_flash_calls"] == 2 and st["flash_calls"] == 0
    assert st["rejected"]["single_token"] == 1 and st["rejected"]["mask"] == 1
