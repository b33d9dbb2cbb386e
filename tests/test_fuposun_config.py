"""Fuposun without a GPU: the typed configuration and its rules, the layout as parts and tensor names, the
decay rank taken from a checkpoint's shapes, random model folders, and the plain implementation's mechanisms
against independent restatements."""
import copy
import json
import os

import numpy as np
import pytest
import torch

from plain import fuposun_plain as FP

RAW = dict(architecture="Fuposun", vocab=90, width=24, residual_mult=0.6, logit_softcap=12.0, norm={"eps": 1e-5}, layers=[
    {"type": "gla", "mixer": {"heads": 2, "dim": 4, "vdim": 6, "tau": 3.0, "decay_rank": 3}, "mlp": None},
    {"type": "latent_attention", "mixer": {"heads": 3, "dim": 4, "vdim": 2, "q_rank": 8, "kv_rank": 16, "scale": 0.5,
                                           "mask": {"size": 5}},
     "mlp": {"kind": "moe", "router": {"experts": 4, "top": 2}, "expert": {"ff": 10, "limit": 0.5},
             "shared": {"ff": 6, "limit": 0.7}}},
    {"type": "latent_attention", "mixer": {"heads": 1, "dim": 8, "vdim": 8, "q_rank": 4, "kv_rank": 8, "scale": 0.3},
     "mlp": {"kind": "dense", "ff": 20}}])


def test_the_registry_finds_the_design_and_the_config_round_trips():
    from quicknn_b200.config import FuposunConfig, find_architecture
    arch = find_architecture(RAW)
    assert arch.name == "Fuposun" and arch.config_cls is FuposunConfig
    cfg = FuposunConfig.from_dict(RAW)
    assert cfg.layers[0].type == "gla" and cfg.layers[0].mlp is None and cfg.layers[0].decay_rank == 3
    assert cfg.layers[1].window == 5 and cfg.layers[2].window is None
    assert cfg.layers[1].mlp.top == 2 and cfg.layers[1].mlp.shared_ff == 6 and cfg.layers[2].mlp.ff == 20
    again = FuposunConfig.from_dict(cfg.to_dict())
    assert again == cfg


def test_every_broken_rule_is_named():
    from quicknn_b200.config import ConfigError, FuposunConfig
    bad = copy.deepcopy(RAW)
    bad["layers"][1]["mlp"]["router"]["top"] = 9
    bad["layers"][1]["mixer"]["scale"] = 0.0
    bad["layers"][0]["mixer"]["tau"] = -1.0
    bad["norm"]["eps"] = 0.0
    with pytest.raises(ConfigError) as e:
        FuposunConfig.from_dict(bad)
    text = str(e.value)
    for piece in ("top 9 of 4", "scale must be > 0", "tau must be > 0", "norm.eps"):
        assert piece in text
    for key, value in (("type", "conv"), ("mlp", {"kind": "sparse"})):
        worse = copy.deepcopy(RAW)
        worse["layers"][0][key] = value
        with pytest.raises(ConfigError):
            FuposunConfig.from_dict(worse)
    no_rank = copy.deepcopy(RAW)
    del no_rank["layers"][0]["mixer"]["decay_rank"]
    with pytest.raises(ConfigError) as e:
        FuposunConfig.from_dict(no_rank)
    assert "decay_rank" in str(e.value)


def test_layout_and_tensor_names():
    from quicknn_b200.config import FuposunConfig, fuposun_spec
    from quicknn_b200.parts import expected_tensors
    spec = fuposun_spec(FuposunConfig.from_dict(RAW))
    names = expected_tensors(spec)
    assert names["embed"][0] == (90, 24) and names["head"][0] == (90, 24) and names["embed.norm"][0] == (24,)
    assert names["l0.mix.a1"][0] == (3, 24) and names["l0.mix.a2"][0] == (8, 3) and names["l0.mix.a2.b"][0] == (8,)
    assert names["l0.mix.norm"][0] == (6,) and names["l0.mix.g"][0] == (12, 24)
    assert "l0.norm2" not in names and spec.optional_tensors == ("l0.norm2",)      # no feed-forward, no norm before it
    assert names["l1.mix.uk"][0] == (12, 16) and names["l1.mix.uv"][0] == (6, 16) and names["l1.mix.g"][0] == (3, 24)
    assert names["l1.mix.dq.norm"][0] == (8,) and names["l1.mlp.e3.down"][0] == (24, 10)
    assert names["l1.mlp.router"][0] == (4, 24) and names["l1.mlp.shared.gate"][0] == (6, 24)
    assert names["l2.mlp.up"][0] == (20, 24) and "l2.mlp.router" not in names
    assert spec.layers[0].feed_forward is None and spec.layers[0].block.get("residual_mult") == 0.6
    assert spec.layers[1].mixer.get("window") == 5 and spec.layers[2].mixer.get("window") is None
    assert spec.head.softcap == 12.0 and not spec.head.tied


def test_a_random_folder_loads_and_the_decay_rank_comes_from_the_checkpoint(tmp_path):
    from quicknn_b200.config import FUPOSUN, FuposunConfig, load_config
    from quicknn_b200.weights import write_model_folder
    cfg = FuposunConfig.from_dict(RAW)
    d = write_model_folder(str(tmp_path / "m"), FUPOSUN, cfg, 5, torch.bfloat16, 0.2)
    arch, back = load_config(d)
    assert arch is FUPOSUN and back == cfg
    raw = json.load(open(os.path.join(d, "config.json")))
    del raw["layers"][0]["mixer"]["decay_rank"]
    json.dump(raw, open(os.path.join(d, "config.json"), "w"))
    assert load_config(d)[1].layers[0].decay_rank == 3
    plain = FP.PlainFuposun(d)
    w = plain.w
    assert abs(float(w["l1.norm1"].mean()) - 1.0) < 0.3 and abs(float(w["l0.mix.a2.b"].mean())) < 0.3
    logits = plain.logits([1, 2, 3, 4, 5, 6, 7])
    assert logits.shape == (7, 90) and np.isfinite(logits).all() and np.abs(logits).max() <= 12.0


def test_plain_mechanisms_against_other_ways_of_writing_them():
    rng = np.random.default_rng(0)
    # the recurrence, unrolled: o_t = sum_{s<=t} (prod_{s<u<=t} a_u * k_s) . q_t  v_s
    H, dim, vdim, n, W = 1, 3, 2, 6, 5
    w = {k: rng.normal(size=s) for k, s in (("q", (dim, W)), ("k", (dim, W)), ("v", (vdim, W)), ("g", (vdim, W)),
                                             ("o", (W, vdim)), ("a1", (2, W)), ("a2", (dim, 2)), ("a2.b", (dim,)))}
    w["norm"] = np.ones(vdim)
    x = rng.normal(size=(n, W))
    m = {"heads": H, "dim": dim, "vdim": vdim, "tau": 2.0}
    q, k, v = x @ w["q"].T * dim ** -0.5, x @ w["k"].T, x @ w["v"].T
    a = (1 / (1 + np.exp(-((x @ w["a1"].T) @ w["a2"].T + w["a2.b"])))) ** 0.5
    o = np.zeros((n, vdim))
    for t in range(n):
        for s in range(t + 1):
            decay = np.prod(a[s + 1:t + 1], axis=0)
            o[t] += ((decay * k[s]) @ q[t]) * v[s]
    o = o / np.sqrt((o * o).mean(-1, keepdims=True) + 1e-5)
    g = x @ w["g"].T
    want = (o * g / (1 + np.exp(-g))) @ w["o"].T
    assert np.abs(FP.gla(x, w, m, 1e-5) - want).max() < 1e-10
    # the window: row i sees exactly the last `size` positions up to itself
    vis = FP.window_mask(6, 3)
    assert vis[5].tolist() == [False, False, False, True, True, True] and vis[1].tolist() == [True, True] + [False] * 4
    assert FP.window_mask(4, None)[3].all()
    # routing: the score goes on the input, so a doubled score is not a doubled output
    mlp = {"router": {"experts": 2, "top": 1}, "expert": {"ff": 3, "limit": 10.0}}
    we = {"router": np.array([[5.0, 0, 0, 0, 0], [0, 0, 0, 0, 0]])}
    for e in range(2):
        we[f"e{e}.gate"], we[f"e{e}.up"], we[f"e{e}.down"] = rng.normal(size=(3, W)), rng.normal(size=(3, W)), rng.normal(size=(W, 3))
    xr = np.array([[1.0, .2, .3, .4, .5], [-1.0, .2, .3, .4, .5]])
    out = FP.routed_ff(xr, we, mlp)
    s0 = 1 / (1 + np.exp(-5.0))
    assert np.allclose(out[0], FP.clamped_expert(s0 * xr[:1], we["e0.gate"], we["e0.up"], we["e0.down"], 10.0)[0])
    assert np.allclose(out[1], FP.clamped_expert(0.5 * xr[1:], we["e1.gate"], we["e1.up"], we["e1.down"], 10.0)[0])
    gate = np.array([[3.0, -3.0]])
    assert np.allclose(FP.clamped_expert(np.eye(1), gate.T, np.array([[5.0], [-5.0]]), np.eye(2), 1.0),
                       [[1 / (1 + np.exp(-1.702)) * 2.0, 0.0]])


def test_the_command_line_writes_and_describes_a_random_model(tmp_path, capsys):
    from quicknn_b200.cli import main
    cfg = tmp_path / "config.json"
    cfg.write_text(json.dumps(RAW))
    out = tmp_path / "model"
    assert main(["random", "--config", str(cfg), "--seed", "3", "--out", str(out)]) == 0
    capsys.readouterr()
    assert main(["info", "--model", str(out)]) == 0
    info = json.loads(capsys.readouterr().out)
    assert info["architecture"] == "Fuposun" and info["layers"] == 3
    assert info["config"]["layers"][0]["mixer"]["decay_rank"] == 3 and info["config"]["layers"][0]["mlp"] is None
