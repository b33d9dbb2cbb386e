"""Tumudra without a GPU: the configuration (registry, round trip, every broken rule named), the layout and the
checkpoint's tensor names, a random folder, and the plain mechanisms against other ways of writing them."""
import copy
import json
import math
import os

import numpy as np
import pytest
import torch

from plain import tumudra_plain as TP
from quicknn_b200.config import TUMUDRA, ConfigError, TumudraConfig, find_architecture, load_config, tumudra_spec
from quicknn_b200.parts import MIXERS, PartSpec, expected_tensors
from quicknn_b200.parts.position import Rotary
from quicknn_b200.weights import random_tensors, write_safetensors


def _rot(base, dims, scaling=None):
    r = {"base": base, "dims": dims}
    if scaling:
        r["scaling"] = dict(zip(("factor", "low", "high", "original"), scaling))
    return r


RAW = dict(architecture="Tumudra", vocab=120, width=48, embedding={"scale": 2.0}, norm={"eps": 1e-5}, initializer_range=0.05,
           layers=[
               {"type": "attention", "mlp": {"kind": "dense", "ff": 64},
                "mixer": {"heads": 4, "kv_heads": 2, "dim": 8, "vdim": 12, "scale": 0.3, "rot": _rot(1e4, 8)}},
               {"type": "retention", "mlp": None,
                "mixer": {"heads": 2, "dim": 8, "vdim": 4, "decay": [0.9, 0.99], "rot": _rot(1e3, 4)}},
               {"type": "parallel", "mlp": {"kind": "dense", "ff": 32},
                "mixer": {"left": {"heads": 2, "kv_heads": 1, "dim": 12, "vdim": 8, "scale": 0.25, "mask": {"size": 5},
                                   "rot": _rot(500.0, 6, (4.0, 1.0, 2.0, 32))},
                          "right": {"heads": 3, "dim": 4, "vdim": 8, "gate_cap": 9.0}}},
               {"type": "attention", "mlp": None,
                "mixer": {"heads": 4, "kv_heads": 2, "dim": 8, "vdim": 12, "scale": 0.3, "rot": _rot(1e4, 8), "kv_from": 0}}])


def test_registry_round_trip_and_layout():
    assert find_architecture({"architecture": "Tumudra"}) is TUMUDRA
    cfg = TumudraConfig.from_dict(RAW)
    assert TumudraConfig.from_dict(cfg.to_dict()) == cfg
    assert TumudraConfig.from_dict(json.loads(json.dumps(cfg.to_dict()))) == cfg
    spec = tumudra_spec(cfg)
    assert [l.mixer.kind for l in spec.layers] == ["attention", "retention", "parallel", "attention"]
    assert [l.block.kind for l in spec.layers] == ["postnorm"] * 4 and spec.head.norm.kind == "layernorm"
    assert [(e.layer, e.cache, e.writes_cache) for e in spec.schedule] == [(0, 0, True), (1, 1, True), (2, 2, True), (3, 0, False)]
    assert spec.layers[1].feed_forward is None and spec.layers[0].feed_forward.params["activation"] == "relu2"
    assert spec.embedding.scale == 2.0 and not spec.head.tied and spec.head.softcap is None
    left = spec.layers[2].mixer.params["branches"]["left"]
    assert left.params["window"] == 5 and left.params["position"].params["layout"] == "interleaved"
    assert spec.layers[0].mixer.params["position"].params["layout"] == "half" and spec.layers[0].mixer.params["bias"]
    names = expected_tensors(spec)
    assert names["l0.mix.q"][0] == (32, 48) and names["l0.mix.v"][0] == (24, 48) and names["l0.mix.o"][0] == (48, 48)
    assert names["l0.mix.q.b"][0] == (32,) and names["l0.mix.o.b"][0] == (48,) and names["l0.mix.k.norm"][0] == (8,)
    assert names["l1.mix.g"][0] == (8, 48) and "l1.norm2" not in names and "l1.mlp.up" not in names
    assert names["l2.mix.left.q"][0] == (24, 48) and "l2.mix.left.q.b" not in names and names["l2.mix.left.out"][0] == (48,)
    assert names["l2.mix.right.i"][0] == (3, 48) and names["l2.mix.right.f.b"][0] == (3,) and names["l2.mix.right.norm"][0] == (24,)
    assert "l3.mix.k" not in names and "l3.mix.v.b" not in names and "l3.mix.k.norm" not in names and "l3.mix.q.norm" in names
    assert names["l3.mix.o.b"][0] == (48,) and names["head"][0] == (120, 48) and names["final.norm"][0] == (48,)
    assert set(n.split(".")[0] for n in names) == {"embed", "final", "head", "l0", "l1", "l2", "l3"}


def _broken(change):
    raw = copy.deepcopy(RAW)
    change(raw)
    return raw


@pytest.mark.parametrize("change,says", [
    (lambda r: r.pop("embedding"), "embedding"),
    (lambda r: r["layers"][0].update(type="conv"), "layer type"),
    (lambda r: r["layers"][0]["mixer"].update(kv_heads=3), "kv_heads do not divide"),
    (lambda r: r["layers"][0]["mixer"]["rot"].update(dims=10), "rot.dims"),
    (lambda r: r["layers"][0]["mixer"]["rot"].update(dims=3), "rot.dims"),
    (lambda r: r["layers"][1]["mixer"].update(decay=[0.9]), "one number per head"),
    (lambda r: r["layers"][1]["mixer"].update(decay=[0.9, 1.5]), "[0, 1]"),
    (lambda r: r["layers"][2]["mixer"]["right"].update(gate_cap=0.0), "gate_cap"),
    (lambda r: r["layers"][2]["mixer"]["left"]["mask"].update(size=0), "mask.size"),
    (lambda r: r["layers"][2]["mixer"]["left"]["rot"]["scaling"].update(high=0.5), "scaling"),
    (lambda r: r["layers"][3]["mixer"].update(kv_from=1), "kv_from"),
    (lambda r: r["layers"][3]["mixer"].update(kv_from=3), "kv_from"),
    (lambda r: r["layers"][3]["mixer"].update(dim=16), "differ"),
    (lambda r: r["layers"][2]["mixer"]["left"].update(kv_from=0), "kv_from"),
    (lambda r: r["layers"][0]["mlp"].update(kind="moe"), "mlp.kind"),
    (lambda r: r["layers"][0]["mlp"].update(ff=0), "mlp.ff"),
    (lambda r: r["norm"].update(eps=0.0), "norm.eps"),
    (lambda r: r["layers"][1]["mixer"].update(dim=512), "at most 256"),
])
def test_every_broken_rule_is_named(change, says):
    with pytest.raises((ConfigError, ValueError, TypeError)) as e:
        TumudraConfig.from_dict(_broken(change))
    assert says in str(e.value), str(e.value)


def test_a_random_folder_loads_by_its_config(tmp_path):
    cfg = TumudraConfig.from_dict(RAW)
    tensors = dict(random_tensors(TUMUDRA, cfg, 7, torch.bfloat16))
    assert set(tensors) == set(expected_tensors(tumudra_spec(cfg)))
    assert abs(float(tensors["l0.norm1"].float().mean()) - 1.0) < 0.2 and abs(float(tensors["l0.mix.q.b"].float().mean())) < 0.2
    with open(tmp_path / "config.json", "w") as fh:
        json.dump(cfg.to_dict(), fh)
    write_safetensors(str(tmp_path / "model.safetensors"), tensors)
    arch, again = load_config(str(tmp_path))
    assert arch is TUMUDRA and again == cfg
    plain = TP.PlainTumudra(str(tmp_path))
    z = plain.logits([5, 6, 7, 8, 9, 10, 11])
    assert z.shape == (7, 120) and np.isfinite(z).all()
    # every position depends on the tokens before it only
    assert np.abs(plain.logits([5, 6, 7, 8])[:4] - z[:4]).max() < 1e-9


def test_the_rotary_parts_frequencies_are_the_plain_ones():
    for dims, scaling in ((8, None), (56, (16.0, 1.0, 4.0, 512)), (6, (4.0, 1.0, 2.0, 32)), (64, (32.0, 0.5, 3.0, 16)), (0, None)):
        rot = _rot(30000.0, dims, scaling)
        params = {"head_dim": max(8, dims), "theta": 30000.0, "rotary_dim": dims, "layout": "interleaved"}
        if scaling:
            params["scaling"] = rot["scaling"]
        got = Rotary(PartSpec("rotary", params)).frequencies().numpy()
        assert got.shape == (dims // 2,) and np.allclose(got, TP.rotary_frequencies(rot), rtol=1e-12, atol=0)
    f = TP.rotary_frequencies(_rot(30000.0, 56, (16.0, 1.0, 4.0, 512)))
    plain = TP.rotary_frequencies(_rot(30000.0, 56))
    wave = 2 * math.pi / plain
    assert np.all(f[wave < 128] == plain[wave < 128]) and np.allclose(f[wave > 512], plain[wave > 512] / 16)
    mid = (wave >= 128) & (wave <= 512)
    assert mid.any() and np.all(f[mid] <= plain[mid]) and np.all(f[mid] >= plain[mid] / 16)


def test_the_two_rotation_layouts_are_one_rotation_under_a_permutation():
    rng = np.random.default_rng(0)
    x = rng.normal(size=(9, 2, 12))
    rot = _rot(300.0, 8)
    perm = np.array([0, 4, 1, 5, 2, 6, 3, 7, 8, 9, 10, 11])        # interleaved column c holds half-split column perm[c]
    a = TP.rotate(x[..., perm], rot, True)
    b = TP.rotate(x, rot, False)[..., perm]
    assert np.allclose(a, b) and np.allclose(a[..., 8:], x[..., 8:]) and np.allclose(a[0], x[0][..., perm])
    assert np.allclose(TP.rotate(x[3:], rot, False, first_position=3), TP.rotate(x, rot, False)[3:])


def test_retention_is_a_decayed_sum_over_earlier_tokens():
    rng = np.random.default_rng(1)
    W, m = 10, {"heads": 2, "dim": 4, "vdim": 6, "decay": [0.8, 0.97], "rot": _rot(50.0, 4)}
    w = {"q": rng.normal(size=(8, W)), "k": rng.normal(size=(8, W)), "v": rng.normal(size=(12, W)), "g": rng.normal(size=(12, W)),
         "o": rng.normal(size=(W, 12))}
    h = rng.normal(size=(7, W))
    q = TP.rotate((h @ w["q"].T).reshape(7, 2, 4), m["rot"], False)
    k = TP.rotate((h @ w["k"].T).reshape(7, 2, 4), m["rot"], False) * 0.5
    v = (h @ w["v"].T).reshape(7, 2, 6)
    o = np.zeros((7, 2, 6))
    for a in range(2):
        for t in range(7):
            for j in range(t + 1):
                o[t, a] += m["decay"][a] ** (t - j) * (q[t, a] @ k[j, a]) * v[j, a]
    g = h @ w["g"].T
    want = (TP.rms_unit(o, 1e-5).reshape(7, 12) * g * TP.sigmoid(g)) @ w["o"].T
    assert np.allclose(TP.retention(h, w, m, 1e-5), want)


def test_the_running_maximum_changes_nothing_but_the_range():
    """The matrix memory against the same recurrence without a maximum, in plain exponentials (float64 holds them here):
    C_t = F C_{t-1} + I k v^T, n likewise, o = C^T q / (max(|n . q|, 1) + 1e-6 e^m) with m only in the last term."""
    rng = np.random.default_rng(2)
    W, m = 9, {"heads": 2, "dim": 3, "vdim": 5, "gate_cap": 4.0}
    w = {"q": rng.normal(size=(6, W)), "k": rng.normal(size=(6, W)), "v": rng.normal(size=(10, W)), "g": rng.normal(size=(10, W)),
         "o": rng.normal(size=(W, 10)), "norm": rng.normal(size=10), "i": rng.normal(size=(2, W)), "i.b": rng.normal(size=2),
         "f": rng.normal(size=(2, W)), "f.b": rng.normal(size=2)}
    h = rng.normal(size=(12, W))
    q = (h @ w["q"].T).reshape(12, 2, 3) * 3 ** -0.5
    k, v = (h @ w["k"].T).reshape(12, 2, 3), (h @ w["v"].T).reshape(12, 2, 5)
    gi = 4.0 * np.tanh((h @ w["i"].T + w["i.b"]) / 4.0)
    gf = TP.log_sigmoid(4.0 * np.tanh((h @ w["f"].T + w["f.b"]) / 4.0))
    o = np.zeros((12, 2, 5))
    for a in range(2):
        C, n, mx = np.zeros((3, 5)), np.zeros(3), 0.0
        for t in range(12):
            C = math.exp(gf[t, a]) * C + math.exp(gi[t, a]) * np.outer(k[t, a], v[t, a])
            n = math.exp(gf[t, a]) * n + math.exp(gi[t, a]) * k[t, a]
            mx = max(gf[t, a] + mx, gi[t, a])
            o[t, a] = (C.T @ q[t, a]) / (max(abs(n @ q[t, a]), 1.0) + 1e-6 * math.exp(mx))
    want = (TP.rms_unit(o, 1e-5).reshape(12, 10) * w["norm"] * TP.sigmoid(h @ w["g"].T)) @ w["o"].T
    assert np.allclose(TP.matrix_memory(h, w, m, 1e-5), want)


def test_window_and_shared_keys_in_the_plain_attention():
    assert TP.visible(5, 2).astype(int).tolist() == [[1, 0, 0, 0, 0], [1, 1, 0, 0, 0], [0, 1, 1, 0, 0], [0, 0, 1, 1, 0], [0, 0, 0, 1, 1]]
    assert TP.visible(3, None).astype(int).tolist() == [[1, 0, 0], [1, 1, 0], [1, 1, 1]]
    rng = np.random.default_rng(3)
    W, m = 8, {"heads": 2, "kv_heads": 1, "dim": 4, "vdim": 6, "scale": 0.5, "rot": _rot(100.0, 4)}
    w = {"q": rng.normal(size=(8, W)), "k": rng.normal(size=(4, W)), "v": rng.normal(size=(6, W)), "o": rng.normal(size=(W, 12)),
         "q.norm": rng.normal(size=4), "k.norm": rng.normal(size=4), "q.b": rng.normal(size=8), "k.b": rng.normal(size=4),
         "v.b": rng.normal(size=6), "o.b": rng.normal(size=W)}
    h = rng.normal(size=(6, W))
    y, kv = TP.attention(h, w, m, 1e-5)
    y2, _ = TP.attention(h, {k: v for k, v in w.items() if k[0] not in "kv"}, m, 1e-5, kv=kv)
    assert np.allclose(y, y2) and kv[0].shape == (6, 1, 4) and kv[1].shape == (6, 1, 6)
    # the last position with a window of 1 sees itself alone: its output is its own value through W_o
    y1, kv = TP.attention(h, w, dict(m, mask={"size": 1}), 1e-5)
    assert np.allclose(y1[-1], np.tile(kv[1][-1, 0], 2) @ w["o"].T + w["o.b"])


def test_parts_declare_their_parameters_without_a_gpu():
    spec = tumudra_spec(TumudraConfig.from_dict(RAW))
    par = spec.layers[2].mixer
    shapes = MIXERS.get("parallel").param_shapes(par)
    assert shapes["left.q_proj"][0] == (24, 48) and shapes["right.gate"][0] == (24, 48) and shapes["right.out"][0] == (48,)
    m = MIXERS.get("parallel")(par)
    assert m.cache_need().window == 5 and m.cache_need().head_dim == 16 and m.state_need().shape == (3 * 4 * 9 + 3,)
    with pytest.raises(ValueError):
        MIXERS.get("parallel")(PartSpec("parallel", {"hidden_size": 48, "eps": 1e-5, "branches": {
            "a": par.params["branches"]["right"], "b": par.params["branches"]["right"]}}))
    shared = MIXERS.get("attention")(spec.layers[3].mixer)
    assert shared.heads.n_kv_heads == 0 and shared.cache_need().head_dim == 16
