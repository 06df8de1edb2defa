"""Host-side checks of the Govuvik design (no GPU): configuration reader and registry, tensor names and shapes, synthetic
weights, and the oracle's mechanisms against closed forms written out in the tests themselves."""
import json
import math

import pytest
import torch

from moshi_b200.config import DECODER_ARCHITECTURES, DecoderLMConfig, GovuvikConfig
from moshi_b200.synth import iter_synth_decoder_tensors
from oracle import govuvik as G

F64 = torch.float64


def small_cfg():
    left = {"conv": 3, "dim": 6, "heads": 4, "kv_heads": 2, "mask": {"size": 5}, "scale": 0.4, "vdim": 5,
            "rot": {"base": 100.0, "dims": 4, "scaling": {"factor": 2.0, "low": 1.0, "high": 2.0, "original": 8}}}
    moe = {"expert": {"ff": 7}, "kind": "moe", "router": {"experts": 4, "top": 2}}
    return {"architecture": "Govuvik", "canon": {"taps": 2}, "logit_softcap": 5.0, "norm": {"eps": 1e-5}, "vocab": 31, "width": 12,
            "layers": [{"type": "parallel", "mixer": {"left": left, "right": {"dim": 3, "heads": 2, "tau": 3.0, "vdim": 4}}, "mlp": moe},
                       {"type": "mlstm", "mixer": {"dim": 5, "gate_cap": 4.0, "heads": 2, "vdim": 3}, "mlp": None}]}


def test_configuration_round_trip_and_registry():
    raw = small_cfg()
    cfg = DecoderLMConfig.from_dict(raw)
    assert isinstance(cfg, GovuvikConfig) and DECODER_ARCHITECTURES["Govuvik"] is GovuvikConfig
    assert cfg.block == "sandwich" and cfg.canon_taps == 2 and cfg.logit_softcap == 5.0
    assert cfg.layers[0].a.window == 5 and cfg.layers[0].a.rot_scaling["factor"] == 2.0 and cfg.layers[0].b.tau == 3.0
    assert cfg.layers[0].experts == 4 and cfg.layers[0].top == 2 and cfg.layers[1].mlp_kind is None
    assert json.loads(json.dumps(cfg.to_dict())) == raw
    from moshi_b200.models.loaders import model_class
    assert model_class(raw).__name__ == "DecoderLM"
    bad = small_cfg()
    bad["layers"][0]["type"] = "latent_attention"
    with pytest.raises((ValueError, KeyError)):
        DecoderLMConfig.from_dict(bad)


def test_tensor_names_and_synthetic_weights():
    cfg = DecoderLMConfig.from_dict(small_cfg())
    shapes = cfg.tensor_shapes()
    assert shapes["l0.mix.left.q"] == (24, 12) and shapes["l0.mix.left.k.conv"] == (12, 3) and shapes["l0.mix.left.talk"] == (4, 4)
    assert shapes["l0.mix.right.a2"] == (6, 16) and shapes["l0.mlp.e3.down"] == (12, 7) and shapes["l0.canon1"] == (12, 2)
    assert shapes["l1.mix.i"] == (2, 12) and shapes["l1.mix.norm"] == (6,) and "l1.norm2" not in shapes and "final.norm.b" not in shapes
    t = dict(iter_synth_decoder_tensors(cfg, seed=1))
    assert set(t) == set(shapes) and all(tuple(t[k].shape) == tuple(shapes[k]) for k in shapes)
    orc = G.GovuvikOracle(small_cfg(), t)
    lg, layers = orc.forward([1, 2, 3, 4, 5, 6, 7], return_layers=True)
    assert lg.shape == (7, 31) and layers.shape == (2, 7, 12) and torch.isfinite(lg).all() and float(lg.abs().max()) <= 5.0
    # state carried over a cut = the whole sequence
    st = orc.new_state()
    cut = torch.cat([orc.forward([1, 2, 3], st), orc.forward([4, 5, 6, 7], st)])
    assert torch.allclose(cut, lg, atol=1e-12)


def test_causal_convolution_against_the_sum():
    g = torch.Generator().manual_seed(0)
    u = torch.randn(9, 3, generator=g, dtype=F64)
    w = torch.randn(3, 4, generator=g, dtype=F64)
    hist, got = [], []
    for t in range(9):
        got.append(G.causal_conv_step(hist, u[t], w))
        hist.append(u[t])
        del hist[:-3]
    for t in range(9):
        want = sum(w[:, j] * u[t - 3 + j] for j in range(4) if t - 3 + j >= 0)
        assert torch.allclose(got[t], want, atol=1e-12)


def test_rotary_frequencies_in_all_three_bands():
    f = G.rope_frequencies(8, 500.0, {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 32})
    plain = [500.0 ** (-2.0 * i / 8) for i in range(4)]
    waves = [2 * math.pi / p for p in plain]
    assert waves[0] < 32 / 4 < waves[1] < 32 < waves[2]                    # kept | blended | divided
    assert f[0] == plain[0] and abs(float(f[2]) - plain[2] / 4) < 1e-15 and abs(float(f[3]) - plain[3] / 4) < 1e-15
    s = (32 / waves[1] - 1.0) / 3.0
    assert abs(float(f[1]) - ((1 - s) * plain[1] / 4 + s * plain[1])) < 1e-15
    assert torch.equal(G.rope_frequencies(8, 500.0, None), torch.tensor(plain, dtype=F64))
    # a rotation keeps the norm and leaves the unrotated tail alone
    u = torch.randn(2, 7, generator=torch.Generator().manual_seed(1), dtype=F64)
    r = G.rope_rotate(u, 13, G.rope_frequencies(4, 100.0, None))
    assert torch.allclose(r.norm(dim=-1), u.norm(dim=-1)) and torch.equal(r[:, 4:], u[:, 4:])
    assert torch.allclose(r[0, 0], u[0, 0] * math.cos(13.0) - u[0, 2] * math.sin(13.0))


def test_window_mask_sink_and_head_mix():
    g = torch.Generator().manual_seed(2)
    keys = [torch.randn(1, 3, generator=g, dtype=F64) for _ in range(6)]
    vals = [torch.randn(1, 2, generator=g, dtype=F64) for _ in range(6)]
    q = torch.randn(2, 3, generator=g, dtype=F64)
    temp, talk, sink = torch.tensor([1.0, 2.0], dtype=F64), torch.tensor([[1.0, 0.5], [0.0, 1.0]], dtype=F64), torch.tensor([0.3, -1.0], dtype=F64)
    out = G.mixed_window_attention(q, keys, vals, 5, 3, 0.5, temp, talk, sink)
    raw = torch.stack([torch.stack([(keys[j][0] @ q[h]) * 0.5 * temp[h] for j in (3, 4, 5)]) for h in range(2)])
    s0 = raw[0] + 0.5 * raw[1]
    e = torch.exp(s0)
    want0 = (e / (e.sum() + math.exp(0.3))) @ torch.stack([vals[j][0] for j in (3, 4, 5)])
    assert torch.allclose(out[0], want0, atol=1e-12)
    # a very large sink takes all the weight and gives nothing
    none = G.mixed_window_attention(q, keys, vals, 5, 3, 0.5, temp, talk, torch.tensor([60.0, 60.0], dtype=F64))
    assert float(none.abs().max()) < 1e-20


def test_gated_linear_attention_against_the_unrolled_sum():
    g = torch.Generator().manual_seed(3)
    T, H, d, v = 6, 2, 3, 4
    q, k, val = torch.randn(T, H, d, generator=g, dtype=F64), torch.randn(T, H, d, generator=g, dtype=F64), torch.randn(T, H, v, generator=g, dtype=F64)
    a = torch.rand(T, H, d, generator=g, dtype=F64)
    S = torch.zeros(H, d, v, dtype=F64)
    for t in range(T):
        S, o = G.gla_step(S, q[t], k[t], val[t], a[t])
        want = torch.zeros(H, v, dtype=F64)
        for j in range(t + 1):
            decay = torch.ones(H, d, dtype=F64)
            for l in range(j + 1, t + 1):
                decay = decay * a[l]
            want += ((q[t] * decay * k[j]).sum(-1))[:, None] * val[j]
        assert torch.allclose(o, want, atol=1e-12)


def test_mlstm_stabiliser_does_not_change_the_result():
    """With small gates the recurrence can be run without the running maximum: C_t = f C + i k v^T, o = C^T q / (max(|n.q|, 1) + ..)
    differs from the stabilised form only through the e^(-m) floor, which the unstabilised form writes as 1."""
    g = torch.Generator().manual_seed(4)
    T, H, d, v = 7, 2, 3, 2
    q, k, val = torch.randn(T, H, d, generator=g, dtype=F64), torch.randn(T, H, d, generator=g, dtype=F64), torch.randn(T, H, v, generator=g, dtype=F64)
    il, fl = torch.randn(T, H, generator=g, dtype=F64), torch.nn.functional.logsigmoid(torch.randn(T, H, generator=g, dtype=F64))
    S, n, m = torch.zeros(H, d, v, dtype=F64), torch.zeros(H, d, dtype=F64), torch.zeros(H, dtype=F64)
    C, nn = torch.zeros(H, d, v, dtype=F64), torch.zeros(H, d, dtype=F64)
    for t in range(T):
        S, n, m, o = G.mlstm_step(S, n, m, q[t], k[t], val[t], il[t], fl[t])
        C = torch.exp(fl[t])[:, None, None] * C + torch.exp(il[t])[:, None, None] * k[t][:, :, None] * val[t][:, None, :]
        nn = torch.exp(fl[t])[:, None] * nn + torch.exp(il[t])[:, None] * k[t]
        assert torch.allclose(S * torch.exp(m)[:, None, None], C, atol=1e-12)          # the true memory is e^m times the stored one
        num = torch.einsum("hdv,hd->hv", C, q[t])
        den = torch.maximum((nn * q[t]).sum(-1).abs(), torch.ones(H, dtype=F64)) * torch.exp(-m) + 1e-6
        assert torch.allclose(o, num * torch.exp(-m)[:, None] / den[:, None], atol=1e-12)
    assert float(G.capped(torch.tensor(100.0, dtype=F64), 4.0)) < 4.0 + 1e-12


def test_router_takes_the_largest_and_renormalises():
    h = torch.tensor([1.0, -2.0, 0.5], dtype=F64)
    router = torch.tensor([[1.0, 0, 0], [0, 1.0, 0], [0, 0, 4.0], [2.0, 0, 0]], dtype=F64)           # logits 1, -2, 2, 2 -> experts 2 and 3 (or 3 and 2)
    ups = [torch.eye(3, dtype=F64) * (e + 1) for e in range(4)]
    downs = [torch.eye(3, dtype=F64) for _ in range(4)]
    out = G.moe_relu2(h, router, ups, downs, 2)
    want = 0.5 * torch.relu(3 * h) ** 2 + 0.5 * torch.relu(4 * h) ** 2
    assert torch.allclose(out, want, atol=1e-12)
    one = G.moe_relu2(h, router[:3], ups[:3], downs[:3], 1)
    assert torch.allclose(one, torch.relu(3 * h) ** 2, atol=1e-12)
