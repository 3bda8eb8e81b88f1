"""Vikupel without a GPU: configuration, run order, tensor names, cache layout, and hand-worked
anchors of the plain implementation's functions."""
import copy
import math

import pytest
import torch

import plain_vikupel as P
from vikupel_configs import VIKUPEL, VIKUPEL_A, VIKUPEL_B, VIKUPEL_C, write_model

from ferrum_b200.config import registry
from ferrum_b200.config.vikupel import AttentionSpec, Mamba2Spec, VikupelConfig
from ferrum_b200.errors import ConfigError, WeightsError

F64 = torch.float64


def test_config_reads_every_size_and_constant():
    c = VikupelConfig.from_dict(VIKUPEL_A)
    assert (c.n_vocab, c.n_embd, c.norm_eps, c.residual_mult, c.side_dim) == (211, 60, 1e-5, 0.55, 6)
    a, m, r, r2 = (l.mixer for l in c.layers)
    assert isinstance(a, AttentionSpec) and (a.heads, a.kv_heads, a.dim, a.vdim, a.scale, a.window) == (3, 1, 10, 14, 0.3, 19)
    assert a.distance_penalty and a.gate and not a.unit_norm and not a.rotate_values and a.rot_dims == 0
    assert isinstance(m, Mamba2Spec) and (m.heads, m.vdim, m.state, m.groups, m.norm_groups, m.conv) == (4, 6, 20, 2, 3, 3)
    assert (r.rot_base, r.rot_dims, r.rot_scaling, r.value_layout, r.window) == (100.0, 8, None, "interleaved", 0)
    assert r.unit_norm and r.rotate_values and not r.gate and not r.distance_penalty
    s = r2.rot_scaling
    assert (s.rope_type, s.factor, s.low_freq_factor, s.high_freq_factor, s.original_max_position_embeddings) == ("llama3", 3.0, 1.0, 3.0, 24)
    assert c.layers[3].mlp is None and c.layers[0].mlp.ff == 100
    assert (c.loop.start, c.loop.stop, c.loop.times) == (1, 3, 3)
    assert c.run_order() == [0, 1, 2, 1, 2, 1, 2, 3]
    assert VikupelConfig.from_dict(VIKUPEL_B).run_order() == [0, 1, 2, 3]
    cc = VikupelConfig.from_dict(VIKUPEL_C)
    assert cc.run_order() == [0, 1, 2] and cc.side_dim == 0


@pytest.mark.parametrize("edit,message", [
    (lambda d: d["layers"][0].update(type="conv"), "not a mixer"),
    (lambda d: d["layers"][0]["mixer"]["mask"].update(size=0), "mask"),
    (lambda d: d["layers"][2]["mixer"].pop("rot"), "rot"),
    (lambda d: d["layers"][1]["mixer"].update(groups=3), "groups"),
    (lambda d: d["layers"][1]["mixer"].update(norm_groups=5), "norm_groups"),
    (lambda d: d["layers"][2]["mixer"]["rot"].update(dims=14), "rot.dims"),
    (lambda d: d["layers"][2]["mixer"].update(vdim=9), "even"),
    (lambda d: d["layers"][0]["mixer"].update(kv_heads=2), "kv_heads"),
    (lambda d: d["loop"].update(stop=9), "loop"),
    (lambda d: d["layers"][0]["mlp"].update(kind="routed"), "feed-forward"),
    (lambda d: d.pop("width"), "width"),
    (lambda d: d["layers"][3]["mixer"]["rot"]["scaling"].pop("high"), "high"),
])
def test_config_refusals(edit, message):
    d = copy.deepcopy(VIKUPEL_A)
    edit(d)
    with pytest.raises(ConfigError, match=message):
        VikupelConfig.from_dict(d)


def test_config_optional_window_and_rotation():
    d = copy.deepcopy(VIKUPEL_A)
    d["layers"][0]["mixer"].pop("mask")                       # no mask: every earlier key
    d["layers"][2]["mixer"]["mask"] = {"size": 7}             # a window on the rotary mixer
    c = VikupelConfig.from_dict(d)
    assert c.layers[0].mixer.window == 0 and c.layers[0].mixer.distance_penalty
    assert c.layers[2].mixer.window == 7 and c.layers[2].mixer.rotate_values


def test_registry_names_and_cache_layout():
    arch = registry.lookup(registry.architecture_name(VIKUPEL_A))
    assert arch.name == "Vikupel"
    cfg = arch.read_config(VIKUPEL_A)
    model = arch.build(cfg, torch.float32, "cpu", max_positions=8)
    names = arch.hf_names(cfg)
    assert names["l1.mix.conv.b"] == "blk.1.mix.conv.bias" and names["l0.mix.r1"] == "blk.0.mix.r1"
    assert names["side.embed"] == "side_embd.weight" and names["l3.side.norm"] == "blk.3.side.norm.weight"
    specs = model.weight_specs()
    assert set(names.values()) == set(specs)                   # every declared tensor has a name in the file and back
    assert specs["side_embd.weight"][0].shape == (211, 4 * 6)
    assert specs["blk.1.mix.in.weight"][0].shape == (2 * 24 + 2 * 2 * 20 + 4, 60)
    assert specs["blk.0.mix.g.weight"][0].shape == (3 * 14, 60) and "blk.2.mix.g.weight" not in specs
    assert "blk.3.mlp.gate.weight" not in specs
    # eight runs; every pass of the loop has planes and state rows of its own
    from ferrum_b200.cache.storage import CacheLayout
    lay = CacheLayout(model)
    assert [r.block for r in model.schedule] == [0, 1, 2, 1, 2, 1, 2, 3]
    assert lay.group_keys == [(1, 14, 19, 2), (2, 12, 0, 2), (2, 8, 0, 2)]          # (kv heads, max(dim, vdim), window, parts)
    assert lay.group_planes == [1, 3, 1]
    assert lay.run_state == [None, 0, None, 1, None, 2, None, None]
    assert lay.state_needs[0].shape == (24 * 20 + 2 * (24 + 2 * 2 * 20),)


def test_weights_are_checked(tmp_path):
    from ferrum_b200.weights.loader import check_weights, open_source
    folder = write_model(VIKUPEL_C, str(tmp_path / "c"), 1)
    arch, cfg = registry.read_config(folder)
    model = arch.build(cfg, torch.float32, "cpu", max_positions=4)
    src = open_source(folder)
    have = {n: e[0] for n, e in src.entries.items()}
    specs = {n: s for n, (s, _, _) in model.weight_specs().items()}
    assert len(check_weights(specs, have, arch.hf_names(cfg))) == len(specs)
    del have["l1.mix.A_log"]
    have["l0.mix.r2"] = (2,)
    have["l2.mix.g"] = (4, 32)
    with pytest.raises(WeightsError) as e:
        check_weights(specs, have, arch.hf_names(cfg))
    assert "l1.mix.A_log" in str(e.value) and "l0.mix.r2" in str(e.value) and "l2.mix.g" in str(e.value)


# --------------------------------------------------------------------------- anchors of the plain functions
def test_plain_small_functions():
    assert abs(float(P.gelu_tanh(torch.tensor(1.0, dtype=F64))) - 0.8411919906082768) < 1e-12
    assert abs(float(P.softplus(torch.tensor(0.0, dtype=F64))) - math.log(2.0)) < 1e-15
    assert abs(float(P.softplus(torch.tensor(50.0, dtype=F64))) - 50.0) < 1e-12
    v = torch.tensor([[3.0, 4.0]], dtype=F64)
    assert torch.allclose(P.rms(v, 0.0), v / math.sqrt(12.5))
    assert torch.allclose(P.rms(v, 12.5), v / 5.0)              # eps sits inside the root


def test_plain_frequencies_and_rotation():
    f = P.rotary_frequencies(100.0, 4)
    assert f == [1.0, 0.1]
    # wavelengths 6.28, 29.2, 135 against borders at 25 and 100: the first is kept, the last is divided, the middle one blended
    f = P.rotary_frequencies(100.0, 6, {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 100})
    base = [1.0, 100.0 ** (-1 / 3), 100.0 ** (-2 / 3)]
    assert f[0] == base[0] and abs(f[2] - base[2] / 4.0) < 1e-15
    s = (100 * base[1] / (2 * math.pi) - 1.0) / 3.0
    assert 0 < s < 1 and abs(f[1] - ((1 - s) * base[1] / 4 + s * base[1])) < 1e-15
    v = torch.tensor([[[1.0, 2.0, 3.0, 4.0, 9.0]]], dtype=F64)
    pos = torch.tensor([1])
    q = math.pi / 2
    halves = P.rotate(v, pos, [q, q], 4)                          # (1, 3) and (2, 4) turn by a quarter; 9 passes
    assert torch.allclose(halves, torch.tensor([[[-3.0, -4.0, 1.0, 2.0, 9.0]]], dtype=F64), atol=1e-12)
    inter = P.rotate(v, pos, [q, q], 4, layout="interleaved")     # (1, 2) and (3, 4)
    assert torch.allclose(inter, torch.tensor([[[-2.0, 1.0, -4.0, 3.0, 9.0]]], dtype=F64), atol=1e-12)
    assert torch.allclose(P.rotate(halves, pos, [q, q], 4, sign=-1.0), v, atol=1e-12)


def test_plain_window_and_distance_penalty():
    # one head, scores all zero: the weights follow the penalty alone, exp(-r1 ln(1 + r2 d)) = (1 + r2 d)^(-r1)
    T = 4
    q = torch.zeros(T, 1, 2, dtype=F64)
    k = torch.zeros(T, 1, 2, dtype=F64)
    v = torch.eye(T, dtype=F64).view(T, 1, T)
    i = torch.arange(T)
    dist = i[:, None] - i[None, :]
    allowed = (dist >= 0) & (dist < 3)
    bias = 2.0 * torch.log1p(0.5 * dist.clamp(min=0).to(F64))[None]
    out = P.softmax_attention(q, k, v, 1.0, allowed, bias)[:, 0]
    w = [1.0, 1.5 ** -2, 2.0 ** -2]
    assert torch.allclose(out[3], torch.tensor([0.0, w[2], w[1], w[0]], dtype=F64) / sum(w))     # key 0 has left the window
    assert torch.allclose(out[1], torch.tensor([w[1], w[0], 0.0, 0.0], dtype=F64) / (w[0] + w[1]))


def test_plain_convolution_and_recurrence():
    u = torch.tensor([[1.0], [2.0], [3.0]], dtype=F64)
    out = P.causal_conv(u, torch.tensor([[10.0, 1.0]], dtype=F64), torch.tensor([0.5], dtype=F64))
    assert out.flatten().tolist() == [1.5, 12.5, 23.5]           # the last tap is the current token's
    # one head, one state element, one value element, a convolution of one tap with weight 1: by hand
    w = {"p.in": torch.eye(5, dtype=F64), "p.conv": torch.ones(3, 1, dtype=F64), "p.conv.b": torch.zeros(3, dtype=F64),
         "p.dt_bias": torch.zeros(1, dtype=F64), "p.A_log": torch.zeros(1, dtype=F64), "p.D": torch.tensor([0.25], dtype=F64),
         "p.norm": torch.ones(1, dtype=F64), "p.o": torch.ones(1, 1, dtype=F64)}
    mc = {"heads": 1, "vdim": 1, "state": 1, "groups": 1, "norm_groups": 1}
    h = torch.tensor([[0.3, 1.0, 2.0, -1.0, 0.0], [0.3, 0.5, 1.0, 3.0, 1.0]], dtype=F64)        # z, x, B, C, dt
    sl = lambda t: t / (1 + math.exp(-t))
    ys, S = [], 0.0
    for z, x, B, C, dt in h.tolist():
        x, B, C = sl(x), sl(B), sl(C)
        d = math.log1p(math.exp(dt))
        S = math.exp(-d) * S + d * B * x
        y = (S * C + 0.25 * x) * sl(z)
        ys.append(y / math.sqrt(y * y + 1e-3))
    got = P.mixer_mamba2(h, w, "p.", mc, 1e-3, None)
    assert torch.allclose(got.flatten(), torch.tensor(ys, dtype=F64), atol=1e-12)


def test_plain_run_order_and_layer_sum(tmp_path):
    assert P.run_order({"layers": [0] * 5, "loop": {"start": 1, "stop": 3, "times": 2}}) == [0, 1, 2, 1, 2, 3, 4]
    assert P.run_order({"layers": [0] * 2}) == [0, 1]
    # residual_mult scales the sublayers' sum: with it at zero the logits are those of the embedding alone
    d = copy.deepcopy(VIKUPEL_C)
    d["residual_mult"] = 0.0
    folder = write_model(d, str(tmp_path / "z"), 2)
    cfg, w = P.load(folder)
    toks = [5, 9, 5]
    lg = P.forward(cfg, w, toks)
    x = w["embed"][toks]
    assert torch.allclose(lg, (P.rms(x, 1e-6) * w["final.norm"]) @ w["head"].T, atol=1e-12)
    assert torch.allclose(lg[0], lg[2])
