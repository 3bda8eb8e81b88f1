"""Ruperax without a GPU: configuration, tensor names, cache layout, random-weights folders, and
the plain implementation against numbers worked by hand."""
import copy
import json
import os

import numpy as np
import pytest
import torch

import plain_ruperax as P
from ruperax_configs import RUPERAX_A, RUPERAX_B, write_model


def test_config_reads_every_size_per_layer():
    from ferrum_b200.config import registry
    from ferrum_b200.config.ruperax import RuperaxConfig
    c = RuperaxConfig.from_dict(RUPERAX_A)
    assert (c.n_vocab, c.n_embd, c.n_ctx_train, c.norm_groups, c.embedding_scale) == (211, 60, 192, 4, 1.7)
    assert [l.mixer.heads for l in c.layers] == [3, 2, 1] and [l.mixer.window for l in c.layers] == [19, 7, 500]
    assert c.layers[1].mixer.kv_from == 0 and c.layers[1].mlp is None and c.layers[2].mlp.ff == 36
    assert registry.architecture_name(RUPERAX_A) == "Ruperax" and registry.lookup("Ruperax").read_config(RUPERAX_B).n_layer == 4


@pytest.mark.parametrize("edit,message", [
    (lambda d: d["layers"][1]["mixer"].update(kv_from=1), "earlier layer"),
    (lambda d: d["layers"][1]["mixer"].update(kv_rank=30), "must equal"),
    (lambda d: d["layers"][0].update(type="other"), "not a mixer"),
    (lambda d: d["layers"][0]["mlp"].update(kind="routed"), "not a feed-forward"),
    (lambda d: d["norm"].update(groups=7), "groups"),
    (lambda d: d["layers"][2]["mixer"].pop("vdim"), "vdim"),
    (lambda d: d.pop("width"), "width"),
])
def test_config_refusals(edit, message):
    from ferrum_b200 import ConfigError
    from ferrum_b200.config.ruperax import RuperaxConfig
    d = copy.deepcopy(RUPERAX_A)
    edit(d)
    with pytest.raises(ConfigError, match=message):
        RuperaxConfig.from_dict(d)


def test_a_reader_of_a_reader_is_refused():
    from ferrum_b200 import ConfigError
    from ferrum_b200.config.ruperax import RuperaxConfig
    d = copy.deepcopy(RUPERAX_B)
    d["layers"][3]["mixer"].update(kv_from=2, kv_rank=128, rot_dim=16, rot={"base": 500.0, "dims": 16})
    with pytest.raises(ConfigError, match="keeps no rows"):
        RuperaxConfig.from_dict(d)


def build(cfg_dict):
    from ferrum_b200.config import registry
    arch = registry.lookup("Ruperax")
    cfg = arch.read_config(cfg_dict)
    return arch, cfg, arch.build(cfg, torch.bfloat16, "cpu", max_positions=32)


def test_tensor_names_cover_the_model_exactly():
    for d in (RUPERAX_A, RUPERAX_B):
        arch, cfg, model = build(d)
        names = arch.hf_names(cfg)
        specs = model.weight_specs()
        assert set(specs) <= set(names.values())
        short = {v: k for k, v in names.items()}
        assert short["blk.0.mix.dq_norm.weight"] == "l0.mix.dq.norm" and short["blk.0.mlp.down.bias"] == "l0.mlp.down.b"
        # a reader layer has no key/value down-projection, a layer without feed-forward no second norm or gate
        i = next(k for k, l in enumerate(cfg.layers) if l.mixer.kv_from is not None)
        assert f"blk.{i}.mix.dkv.weight" not in specs and f"blk.{i}.mix.uk.weight" in specs
        j = next(k for k, l in enumerate(cfg.layers) if l.mlp is None)
        assert f"blk.{j}.norm2.weight" not in specs and f"blk.{j}.rg2.weight" not in specs and f"blk.{j}.rg1.bias" in specs


def test_cache_layout_groups_planes_states_and_reader_windows():
    from ferrum_b200.cache.storage import CacheLayout
    _, cfg, model = build(RUPERAX_A)
    lay = CacheLayout(model)
    # layer 1 reads layer 0's rows with a narrower window: the plane keeps the wider one; one part per page
    assert lay.group_keys == [(1, 28, 19, 1), (1, 41, 500, 1)] and lay.run_plane == [0, 0, 0] and lay.run_group == [0, 0, 1]
    assert lay.run_state == [0, 1, 2] and [tuple(n.shape) for n in lay.state_needs] == [(60,)] * 3
    _, cfg, model = build(RUPERAX_B)
    lay = CacheLayout(model)
    # layer 2 looks back further (40) than its source layer 1 (33): the plane keeps 40
    assert lay.group_keys == [(1, 96, 48, 1), (1, 144, 40, 1)] and lay.run_group == [0, 1, 1, 0]
    assert lay.bytes_per_token(torch.bfloat16) == 2 * (96 + 144)


def test_a_checkpoint_with_a_wrong_or_missing_tensor_is_refused(tmp_path):
    from ferrum_b200 import WeightsError
    from ferrum_b200.weights import SafetensorsFile, write_safetensors
    from ferrum_b200.weights.loader import check_weights
    folder = write_model(RUPERAX_A, str(tmp_path / "m"), 1)
    arch, cfg, model = build(RUPERAX_A)
    st = SafetensorsFile(os.path.join(folder, "model.safetensors"))
    have = {n: st.shape(n) for n in st.names()}
    specs = {n: s for n, (s, _, _) in model.weight_specs().items()}
    assert len(check_weights(specs, have, arch.hf_names(cfg))) == len(have)
    have["l1.mix.dkv"] = (28, 60)
    del have["l2.shift"]
    have["l0.mix.g"] = (4, 60)
    with pytest.raises(WeightsError) as e:
        check_weights(specs, have, arch.hf_names(cfg))
    assert "l1.mix.dkv" in str(e.value) and "l2.shift" in str(e.value) and "l0.mix.g" in str(e.value)


def test_random_weights_folder_is_read_by_the_plain_reader(tmp_path):
    folder = write_model(RUPERAX_A, str(tmp_path / "m"), 2)
    cfg, w = P.read_model(folder)
    assert cfg["layers"][1]["mixer"]["kv_from"] == 0
    assert w["l0.mix.uq"].shape == (3 * 16, 18) and w["l1.mix.uk"].shape == (24, 22) and "l1.mix.dkv" not in w
    assert w["pos"].shape == (192, 60) and w["l0.shift"].min() >= 0 and w["l0.shift"].max() <= 1
    logits = P.forward(cfg, w, [1, 2, 3, 4, 5])
    assert logits.shape == (5, 211) and np.isfinite(logits).all()


# ---------------------------------------------------------------- the plain implementation, by hand
def test_plain_group_norm_and_shift_by_hand():
    x = np.array([[3.0, 4.0, 0.0, 2.0]])
    n = P.group_norm(x, 2, 0.0)
    assert np.allclose(n, [[3 / np.sqrt(12.5), 4 / np.sqrt(12.5), 0.0, np.sqrt(2.0)]])
    a = np.array([[1.0, 2.0], [3.0, 6.0], [5.0, 10.0]])
    m = P.token_shift(a, np.array([0.0, 0.5]))
    assert np.allclose(m, [[1.0, 1.0], [3.0, 4.0], [5.0, 8.0]])
    assert np.allclose(P.token_shift(a[1:], np.array([1.0, 1.0]), before=a[0]), [[1.0, 2.0], [3.0, 6.0]])


def test_plain_rotation_by_hand():
    v = np.array([[[1.0, 0.0, 0.0, 1.0, 9.0]]])                      # dims 4 of 5: pairs (0, 2) and (1, 3)
    out = P.rotate_half(v, [2], 4, 100.0)
    a0, a1 = 2.0, 2.0 * 100.0 ** -0.5
    assert np.allclose(out[0, 0], [np.cos(a0), -np.sin(a1), np.sin(a0), np.cos(a1), 9.0])


def test_plain_window_is_exact_by_hand():
    """One head, identity-like maps: a query sees itself and the size - 1 keys before it."""
    E = 2
    w = {"p.dq": np.eye(E), "p.dq.norm": np.ones(E), "p.uq": np.eye(E), "p.uk": np.eye(E), "p.uv": np.eye(E),
         "p.g": np.zeros((1, E)), "p.o": np.eye(E)}
    mix = dict(heads=1, dim=2, rot_dim=0, vdim=2, kv_rank=2, scale=0.0, mask={"size": 3}, rot={"dims": 0, "base": 1.0})
    c = np.array([[1.0, 0.0], [0.0, 1.0], [2.0, 2.0], [4.0, 0.0], [0.0, 8.0]])
    m = np.ones((5, E))
    out = P.latent_attention(m, w, "p.", mix, 1e-6, np.arange(5), (c, np.zeros((5, 0))))
    want = np.array([c[0], c[:2].mean(0), c[:3].mean(0), c[1:4].mean(0), c[2:5].mean(0)]) * 0.5     # scale 0: plain means; gate 1/2
    assert np.allclose(out, want)


def test_command_line_writes_and_lists_a_random_model(tmp_path, capsys):
    from ferrum_b200 import cli
    cfg = tmp_path / "cfg.json"
    cfg.write_text(json.dumps(RUPERAX_B))
    out = tmp_path / "model"
    assert cli.main(["random-weights", "--config", str(cfg), "--out", str(out), "--seed", "3", "--dtype", "bfloat16"]) == 0
    capsys.readouterr()
    assert cli.main(["dump", str(out)]) == 0
    listing = capsys.readouterr().out
    assert "l2.mix.uk [128, 128] bfloat16" in listing and "l3.rg1.b [128] float32" in listing and "l3.norm2" not in listing
    c, w = P.read_model(str(out))
    assert c["architecture"] == "Ruperax" and w["head"].shape == (256, 128)
