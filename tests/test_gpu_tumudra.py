"""Tumudra on the GPU against the plain implementation (tests/plain/tumudra_plain.py): the small kernels; each mixer
alone over a cache of its own (prompts, single tokens, portions, a slot handed out again, long prompts in segments,
keys at window and page edges, a far key that one score singles out); then whole models through bin/trace_run under
every cutting, in portions down to two tokens, through the entry point's generation loop, and configurations drawn
at random.  The configurations are small and differ from one another in every size and constant."""
import json
import math
import os

import numpy as np
import pytest
import torch

from conftest import close
from plain import tumudra_plain as TP
from test_gpu_fuposun import part_step
from test_gpu_replay import Replay, run_all_cuttings

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.fixture(scope="module", autouse=True)
def _need_gpu():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")


def dev(a, dtype=torch.float32):
    return torch.from_numpy(np.asarray(a)).to(DEV).to(dtype).contiguous()


def host(t):
    return t.detach().float().cpu().numpy().astype(np.float64)


def rnd(shape, seed, scale=1.0):
    return (np.random.default_rng(seed).normal(size=shape) * scale).astype(np.float32)


def bf(a):
    return torch.from_numpy(np.asarray(a, dtype=np.float32)).to(torch.bfloat16).float().numpy()


def f64(w):
    return {k: np.asarray(v, dtype=np.float64) for k, v in w.items()}


def near(got, ref, dtype, float32=1e-4):
    """How whole models are compared.  A layer adds the NORMED output of its sublayers, so an error in a sublayer's output
    reaches the stream at full size whatever the output's own size was, and the norm per head after a memory keeps only
    the direction of a read-out: where a query stands almost at a right angle to what the memory holds (one row in a
    hundred or so, with the queries and keys scaled as they are here), float32 rounding of the read-out becomes 5e-5 of
    the logits, in the plain order of operations as in any other.  float32: by the largest difference, 1e-4 of the
    largest logit (3e-4 for the configurations drawn at random, whose gates span up to e^60); a wrong mask, key, window
    or state moves these models' logits by 1e-2 and more.  bfloat16: a row is compared by the root mean square of its
    difference against that of the logits, at most a tenth, and one row in thirty (or one) may lie beyond (at a sequence's
    first tokens the state has rank one and the norm keeps only a sign)."""
    got, ref = np.asarray(got, dtype=np.float64), np.asarray(ref, dtype=np.float64)
    if dtype == "float32":
        tol = float32 * max(1.0, float(np.abs(ref).max()))
        err = float(np.abs(got - ref).max()) if got.size else 0.0
        return err <= tol, err, tol
    if not got.size:
        return True, 0.0, 0.1
    d = got - ref
    d = d - d.mean(axis=-1, keepdims=True)
    r = ref - ref.mean(axis=-1, keepdims=True)
    e = np.sqrt((d * d).mean(axis=-1)) / np.sqrt((r * r).mean())
    over = int((e > 0.1).sum())
    return over <= max(1, len(e) // 30), float(np.sort(e)[-1 - min(over, max(1, len(e) // 30), len(e) - 1)]), 0.1


@pytest.fixture
def whole_model_tolerance(monkeypatch):
    import test_gpu_replay
    monkeypatch.setattr(test_gpu_replay, "close", near)


# ---- configurations -------------------------------------------------------------------------------------

def _rot(base, dims, scaling=None):
    r = {"base": base, "dims": dims}
    if scaling:
        r["scaling"] = dict(zip(("factor", "low", "high", "original"), scaling))
    return r


def _att(heads, kv, dim, vdim, scale, rot, window=None, kv_from=None):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale, "rot": rot}
    if window is not None:
        m["mask"] = {"size": window}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def _layer(kind, mixer, ff):
    return {"type": kind, "mixer": mixer, "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def _mem(heads, dim, vdim, cap):
    return {"heads": heads, "dim": dim, "vdim": vdim, "gate_cap": cap}


def _ret(heads, dim, vdim, decay, rot):
    return {"heads": heads, "dim": dim, "vdim": vdim, "decay": decay, "rot": rot}


# A: a recurrent layer first and without a feed-forward, as many kv heads as heads in the windowed branch, a shared
#    layer that also lacks a feed-forward, key sizes above and below the value sizes, a partly rotated retention
TUMU_A = dict(architecture="Tumudra", vocab=300, width=64, embedding={"scale": 3.0}, norm={"eps": 1e-6},
              initializer_range=0.08, layers=[
                  _layer("retention", _ret(2, 16, 24, [0.9, 0.995], _rot(500.0, 8)), None),
                  _layer("attention", _att(4, 2, 16, 24, 0.25, _rot(10000.0, 16)), 96),
                  _layer("parallel", {"left": _att(2, 2, 24, 8, 0.2, _rot(3000.0, 12, (4.0, 1.0, 3.0, 64)), window=9),
                                      "right": _mem(1, 8, 16, 8.0)}, 40),
                  _layer("attention", _att(4, 2, 16, 24, 0.25, _rot(10000.0, 16), kv_from=1), None)])
# B: head size 64 (the tensor-core attention kernels in bfloat16), a window beyond a page, two shared layers on one
#    owner with a layer between, several memory heads, a scale of exactly 1 on the embedding
TUMU_B = dict(architecture="Tumudra", vocab=512, width=128, embedding={"scale": 1.0}, norm={"eps": 1e-5},
              initializer_range=0.06, layers=[
                  _layer("parallel", {"left": _att(4, 1, 64, 64, 0.125, _rot(50000.0, 32, (8.0, 1.0, 4.0, 128)), window=70),
                                      "right": _mem(3, 32, 16, 15.0)}, 192),
                  _layer("attention", _att(2, 2, 64, 32, 0.11, _rot(1e6, 64)), 64),
                  _layer("attention", _att(2, 2, 64, 32, 0.11, _rot(1e6, 64), kv_from=1), 160),
                  _layer("retention", _ret(3, 64, 32, [0.96875, 0.99, 1.0], _rot(1e4, 64)), 96),
                  _layer("attention", _att(2, 2, 64, 32, 0.11, _rot(1e6, 64), kv_from=1), 64)])
# C: a width, head sizes and a vocabulary that are no multiple of 8, a window of one token, no rotation at all in
#    one layer, one head everywhere in another.  (Gate caps stay moderate here: with a cap of 30 the gates span e^60 and
#    float32 itself is no longer good to the 2e-5 that these models are held to; the random configurations have such caps.)
TUMU_C = dict(architecture="Tumudra", vocab=301, width=100, embedding={"scale": 7.5}, norm={"eps": 1e-4},
              initializer_range=0.07, layers=[
                  _layer("attention", _att(5, 5, 12, 20, 0.3, _rot(777.0, 0)), 70),
                  _layer("parallel", {"left": _att(3, 1, 20, 12, 0.22, _rot(2e4, 20), window=1),
                                      "right": _mem(2, 12, 20, 3.0)}, None),
                  _layer("retention", _ret(1, 20, 12, [0.75], _rot(100.0, 20)), 36),
                  _layer("parallel", {"left": _att(1, 1, 8, 8, 0.35, _rot(1e3, 4, (2.0, 0.5, 2.0, 16)), window=11),
                                      "right": _mem(1, 20, 4, 6.0)}, 36)])
CONFIGS = {"A": (TUMU_A, 3), "B": (TUMU_B, 4), "C": (TUMU_C, 5)}
LENGTHS = [70, 33, 129, 45, 100, 64]
LENGTHS_B = [170, 33, 257, 45, 100, 64]


def make_folder(base, name, storage, peaky):
    """Random weights; ``peaky`` scales what decides where attention and memory look (the head norms' weights, which
    set the size of queries and keys after their norm; the memories' query and key products) and spreads the gates'
    biases from forgetting fast to hardly at all."""
    from quicknn_b200.config import TUMUDRA, TumudraConfig
    from quicknn_b200.weights import random_tensors, write_safetensors
    raw, seed = CONFIGS[name]
    cfg = TumudraConfig.from_dict(raw)
    d = os.path.join(str(base), f"tumu{name}_{storage}{'_peaky' if peaky else ''}")
    os.makedirs(d, exist_ok=True)
    tensors = dict(random_tensors(TUMUDRA, cfg, seed, torch.float32, 0.2))
    if peaky:
        for k in list(tensors):
            if k.endswith(("q.norm", "k.norm")):
                tensors[k] = tensors[k] * 2.5
            elif k.endswith((".mix.q", ".mix.k", "right.q", "right.k")):
                tensors[k] = tensors[k] * 3.0
            elif k.endswith(("right.i", "right.f")):
                tensors[k] = tensors[k] * 3.0
            elif k.endswith("right.f.b"):
                tensors[k] = torch.linspace(-1.0, 6.0, tensors[k].numel())
            elif k.endswith("right.i.b"):
                tensors[k] = torch.linspace(-2.0, 2.0, tensors[k].numel())
    dt = torch.float32 if storage == "float32" else torch.bfloat16
    with open(os.path.join(d, "config.json"), "w") as fh:
        json.dump(cfg.to_dict(), fh)
    write_safetensors(os.path.join(d, "model.safetensors"), {k: v.to(dt) for k, v in tensors.items()})
    return d


@pytest.fixture(scope="module")
def tumu(tmp_path_factory):
    base = tmp_path_factory.mktemp("tumudra")
    made = {}

    def get(name, storage="float32", peaky=False):
        key = (name, storage, peaky)
        if key not in made:
            folder = make_folder(base, name, storage, peaky)
            made[key] = (folder, TP.PlainTumudra(folder))
        return made[key]
    return get


def prompts(name, lengths, seed=0):
    rng = np.random.default_rng(100 + seed)
    return [rng.integers(1, CONFIGS[name][0]["vocab"], n).tolist() for n in lengths]


# ---- the small kernels ------------------------------------------------------------------------------------

@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_layer_norm_alone_and_added_to_the_stream(dtype):
    from quicknn_b200.kernels import ops
    for rows, width in ((3, 100), (70, 64), (5, 2304), (2, 12288)):
        x, w = bf(rnd((rows, width), 1, 2.0) + 0.7), bf(rnd(width, 3, 0.2) + 1.0)
        ref = TP.layer_norm(x.astype(np.float64), w.astype(np.float64), 1e-5)
        tol = (2e-5 if dtype == torch.float32 else 0.02) * np.abs(ref).max()
        assert np.abs(host(ops.layernorm(dev(x, dtype), dev(w, dtype), 1e-5, dtype)) - ref).max() < tol
        resid, bias = rnd((rows, width), 4, 3.0), bf(rnd(width, 5, 0.5))
        r = dev(resid)
        copy = ops.add_layernorm(r, dev(x, dtype), dev(w, dtype), 1e-5, dev(bias, dtype), dtype)
        want = resid + TP.layer_norm(x.astype(np.float64) + bias, w.astype(np.float64), 1e-5)
        assert np.abs(host(r) - want).max() < 3e-5 * np.abs(want).max()          # the stream itself is float32
        assert (copy is r) if dtype == torch.float32 else (np.abs(host(copy) - want).max() < 0.01 * np.abs(want).max())
        r2 = dev(resid)
        assert ops.add_layernorm(r2, dev(x, dtype), dev(w, dtype), 1e-5) is None
        want = resid + ref
        assert np.abs(host(r2) - want).max() < 3e-5 * np.abs(want).max()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_mean_of_normed_branches_bias_and_squared_relu(dtype):
    from quicknn_b200.kernels import ops
    for rows, width, n in ((4, 100, 2), (33, 64, 3), (2, 4096, 2), (3, 24, 1)):
        ys = [bf(rnd((rows, width), 10 + b, 1.0 + b)) for b in range(n)]
        ws = [bf(rnd(width, 20 + b, 0.2) + 1.0) for b in range(n)]
        mean = sum(TP.rms_unit(y.astype(np.float64), 1e-6) * w for y, w in zip(ys, ws)) / n
        got = host(ops.mean_rmsnorm([dev(y, dtype) for y in ys], [dev(w, dtype) for w in ws], 1e-6, dtype))
        assert np.abs(got - mean).max() < (2e-5 if dtype == torch.float32 else 0.02) * np.abs(mean).max()
        resid, w = rnd((rows, width), 30, 2.0), bf(rnd(width, 31, 0.2) + 1.0)
        r = dev(resid)
        copy = ops.add_mean_layernorm(r, [dev(y, dtype) for y in ys], [dev(x, dtype) for x in ws], 1e-6, dev(w, dtype), 1e-5,
                                      dtype)
        want = resid + TP.layer_norm(mean, w.astype(np.float64), 1e-5)
        assert np.abs(host(r) - want).max() < 3e-5 * np.abs(want).max()
        assert np.abs(host(copy) - want).max() < (3e-5 if dtype == torch.float32 else 0.01) * np.abs(want).max()
    y, b = bf(rnd((5, 37), 40)), bf(rnd(37, 41))
    t = dev(y, dtype)
    ops.add_bias_(t, dev(b, dtype))
    assert np.abs(host(t) - (y + b)).max() < (1e-6 if dtype == torch.float32 else 0.02)
    z = bf(rnd((6, 50), 42, 2.0))
    got = host(ops.activation(dev(z, dtype), "relu2"))
    want = np.maximum(z, 0.0).astype(np.float64) ** 2
    assert np.abs(got - want).max() < (1e-6 if dtype == torch.float32 else 0.01) * want.max()


@pytest.mark.parametrize("interleaved", [False, True])
@pytest.mark.parametrize("hd,norm_dim,rot", [(16, 16, 16), (24, 20, 8), (8, 8, 0), (40, 36, 36), (96, 88, 40), (128, 128, 128),
                                             (256, 256, 64), (64, 64, 32)])
@pytest.mark.parametrize("c_in,c_out,spare", [(3, 1, 5), (8, 4, 16)])
def test_bias_head_norms_and_rotation_in_one_kernel(interleaved, hd, norm_dim, rot, c_in, c_out, spare):
    """Against the plain pieces: heads carried wider than they are normed, partly rotated, both pairings, float32 rows
    written beside bfloat16 ones; rows that start on 16 bytes (the kernel with 16-byte accesses) and rows that do not."""
    from quicknn_b200.kernels import ops
    nq, nk, T, eps = 3, 2, 7, 1e-5
    nv = nk * hd
    width = (nq + nk) * hd + nv
    x, bias = bf(rnd((T, width + spare), 1)), bf(rnd(width, 2, 0.3))
    wq, wk = bf(rnd(norm_dim, 3, 0.2) + 1), bf(rnd(norm_dim, 4, 0.2) + 1)
    pos = np.array([0, 1, 5, 63, 64, 300, 2000], dtype=np.int32)
    rot_cfg = {"base": 5000.0, "dims": rot, "scaling": {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 256}}
    inv = torch.tensor(TP.rotary_frequencies(rot_cfg) if rot else np.zeros(0), dtype=torch.float64).to(torch.float32).to(DEV)

    def plain_heads(cols, n, w):
        h = (x[:, c_in + cols:c_in + cols + n * hd] + bias[cols:cols + n * hd]).astype(np.float64).reshape(T, n, hd)
        h[..., :norm_dim] = TP.rms_unit(h[..., :norm_dim], eps) * w
        out = np.stack([TP.rotate(h[t:t + 1], rot_cfg, interleaved, int(pos[t]))[0] for t in range(T)]) if rot else h
        return out.reshape(T, n * hd)
    want = np.concatenate([plain_heads(0, nq, wq), plain_heads(nq * hd, nk, wk),
                           (x[:, c_in + (nq + nk) * hd:c_in + width] + bias[(nq + nk) * hd:]).astype(np.float64)], axis=1)
    for dtype in (torch.float32, torch.bfloat16):
        src = dev(x, dtype)
        out32 = torch.zeros((T, width + 2 * c_out), device=DEV)
        ops.head_prep(src, c_in, nq, nk, nv, hd, dst=out32, dst_col0=c_out, bias=dev(bias), q_norm=dev(wq, dtype),
                      k_norm=dev(wk, dtype), norm_dim=norm_dim, eps=eps, rot_dim=rot, inv_freq=inv, interleaved=interleaved,
                      tok_pos=dev(pos, torch.int32))
        got = host(out32)
        assert np.abs(got[:, c_out:c_out + width] - want).max() < 3e-5 * np.abs(want).max()      # float32 rows: nothing rounded
        assert not got[:, :c_out].any() and not got[:, c_out + width:].any()
        assert np.array_equal(host(src), x.astype(np.float64))                          # the source is left alone
        ops.head_prep(src, c_in, nq, nk, nv, hd, bias=dev(bias), q_norm=dev(wq, dtype), k_norm=dev(wk, dtype),
                      norm_dim=norm_dim, eps=eps, rot_dim=rot, inv_freq=inv, interleaved=interleaved,
                      tok_pos=dev(pos, torch.int32))                                     # in place
        got = host(src)
        assert np.abs(got[:, c_in:c_in + width] - want).max() < (3e-5 if dtype == torch.float32 else 0.02) * np.abs(want).max()
        assert np.array_equal(got[:, :c_in], x[:, :c_in].astype(np.float64))
        assert np.array_equal(got[:, c_in + width:], x[:, c_in + width:].astype(np.float64))


def test_gates_with_a_running_maximum_match_the_row_by_row_recurrence():
    """Sequences of 1, 31, 32, 33 and 100 rows (the scan takes 32 at a time), then more rows onto the kept maxima, a
    row of no sequence, gates driven into their caps."""
    from quicknn_b200.kernels import ops
    H, cap = 3, 5.0
    lens = [1, 31, 32, 33, 100]
    T = sum(lens)
    pre = rnd((T + len(lens), 2 * H), 1, 6.0)
    bias = rnd(2 * H, 2)
    state = torch.zeros((8, 10 + H), device=DEV)

    def plain(rows, m0):
        gi = cap * np.tanh((rows[:, :H].astype(np.float64) + bias[:H]) / cap)
        gf = TP.log_sigmoid(cap * np.tanh((rows[:, H:].astype(np.float64) + bias[H:]) / cap))
        out, m = np.zeros((len(rows), 3 * H)), m0.copy()
        for t in range(len(rows)):
            new = np.maximum(gf[t] + m, gi[t])
            out[t] = np.concatenate([np.exp(gf[t] + m - new), np.exp(gi[t] - new), np.exp(-new)])
            m = new
        return out, m
    first = np.cumsum([0] + lens[:-1])
    slots = [5, 0, 3, 1, 7]
    i32 = lambda a: torch.tensor(np.asarray(a), dtype=torch.int32, device=DEV)  # noqa: E731
    got = host(ops.mlstm_gates(dev(pre[:T]), dev(bias), cap, i32(first), i32(lens), i32(slots), state, 10, len(lens), H))
    ms = []
    for r0, n in zip(first, lens):
        want, m = plain(pre[r0:r0 + n], np.zeros(H))
        ms.append(m)
        assert (np.abs(got[r0:r0 + n] - want) / np.maximum(1.0, np.abs(want))).max() < 1e-5       # e^-m may be large
    st = host(state)
    assert all(np.abs(st[s, 10:] - m).max() < 1e-5 for s, m in zip(slots, ms)) and not st[:, :10].any()
    # one more row each, as a decode step brings it; the second row belongs to no sequence
    slots2 = [5, -1, 3, 1, 7]
    got = host(ops.mlstm_gates(dev(pre[T:]), dev(bias), cap, None, None, i32(slots2), state, 10, len(lens), H))
    for i, (s, m) in enumerate(zip(slots2, ms)):
        want, _ = plain(pre[T + i:T + i + 1], m)
        if s >= 0:
            assert (np.abs(got[i] - want[0]) / np.maximum(1.0, np.abs(want[0]))).max() < 1e-5
        else:
            assert np.array_equal(got[i], np.array([0.0] * (2 * H) + [1.0] * H))
    assert np.abs(host(state)[0, 10:] - ms[1]).max() < 1e-5                      # the skipped sequence's maxima stay


# ---- the memory mixers alone -----------------------------------------------------------------------------------

def _memory_mixer(kind, W, heads, dim, vdim, seed, extra, gate_scale=0.8):
    from quicknn_b200.parts import MIXERS, PartSpec
    spec = PartSpec(kind, dict({"hidden_size": W, "n_heads": heads, "dim": dim, "vdim": vdim, "eps": 1e-5}, **extra))
    mixer = MIXERS.get(kind)(spec)
    w = {"q": rnd((heads * dim, W), seed + 1, 0.3), "k": rnd((heads * dim, W), seed + 2, 0.3),
         "v": rnd((heads * vdim, W), seed + 3, 0.3), "g": rnd((heads * vdim, W), seed + 4, 0.3),
         "o": rnd((W, heads * vdim), seed + 5, 0.3)}
    names = {"q": "q", "k": "k", "v": "v", "g": "gate", "o": "o"}
    if kind == "mlstm":
        w.update({"norm": rnd(heads * vdim, seed + 6, 0.2) + 1, "i": rnd((heads, W), seed + 7, gate_scale),
                  "i.b": np.linspace(-2, 2, heads).astype(np.float32), "f": rnd((heads, W), seed + 8, gate_scale),
                  "f.b": np.linspace(0, 6, heads).astype(np.float32)})      # memories from a few tokens to hundreds
        names.update({"norm": "norm", "i": "i", "i.b": "i_bias", "f": "f", "f.b": "f_bias"})
    mixer.load({names[k]: dev(v) for k, v in w.items()}, torch.float32, DEV)
    return mixer, f64(w)


def _walk_a_memory_mixer(mixer, plain, W, lens, more, tol):
    """Prompts of unequal length (one of a single token), single tokens, a portion, a slot handed out again."""
    from quicknn_b200.cache import KVCache
    cache = KVCache([None], [mixer.state_need()], 4096, 3, 2048, torch.float32, DEV)
    xs = [rnd((n + more, W), 20 + i) for i, n in enumerate(lens)]
    ref = [plain(x.astype(np.float64)) for x in xs]
    slots = [cache.allocate() for _ in lens][::-1]

    def check(y, want):
        assert np.abs(host(y) - want).max() < tol * max(1.0, np.abs(want).max())
    step = part_step(lens, [0] * len(lens), slots, "prefill", torch.float32, cache, mixer)
    check(mixer.forward(dev(np.concatenate([x[:n] for x, n in zip(xs, lens)])), step, cache.line(0)),
          np.concatenate([r[:n] for r, n in zip(ref, lens)]))
    for t in range(2):
        step = part_step([1] * len(lens), [n + t for n in lens], slots, "decode", torch.float32, cache, mixer)
        check(mixer.forward(dev(np.stack([x[n + t] for x, n in zip(xs, lens)])), step, cache.line(0)),
              np.stack([r[n + t] for r, n in zip(ref, lens)]))
    a, b = lens[0] + 2, lens[2] + 2
    step = part_step([more - 3, 2], [a, b], [slots[0], slots[2]], "extend", torch.float32, cache, mixer)
    check(mixer.forward(dev(np.concatenate([xs[0][a:a + more - 3], xs[2][b:b + 2]])), step, cache.line(0)),
          np.concatenate([ref[0][a:a + more - 3], ref[2][b:b + 2]]))
    cache.free(slots[0])
    again = cache.allocate()
    assert again == slots[0]
    step = part_step([lens[2]], [0], [again], "prefill", torch.float32, cache, mixer)
    check(mixer.forward(dev(xs[2][:lens[2]]), step, cache.line(0)), ref[2][:lens[2]])


@pytest.mark.parametrize("heads,dim,vdim,rot", [(2, 16, 24, 8), (1, 12, 40, 12), (3, 64, 32, 64), (1, 200, 8, 0),
                                                (2, 32, 72, 32), (1, 8, 63, 4)])
def test_retention_alone(heads, dim, vdim, rot):
    from quicknn_b200.parts import PartSpec
    W = 48
    decay = [1.0 - 2.0 ** -(3 + 2 * h) for h in range(heads)]
    pos = PartSpec("rotary", {"head_dim": dim, "theta": 300.0, "rotary_dim": rot, "layout": "half"})
    mixer, w = _memory_mixer("retention", W, heads, dim, vdim, 0, {"decay": decay, "position": pos})
    assert mixer.cache_need() is None and mixer.state_need().shape == (heads * dim * vdim,)
    m = {"heads": heads, "dim": dim, "vdim": vdim, "decay": decay, "rot": {"base": 300.0, "dims": rot}}
    _walk_a_memory_mixer(mixer, lambda x: TP.retention(x, w, m, 1e-5), W, [150, 1, 37], 8, 3e-5)


@pytest.mark.parametrize("heads,dim,vdim,cap", [(2, 16, 24, 8.0), (1, 12, 40, 3.0), (3, 64, 32, 15.0), (1, 200, 8, 30.0),
                                                (5, 32, 64, 9.0), (1, 8, 63, 1.0)])
def test_matrix_memory_with_gates_alone(heads, dim, vdim, cap):
    """vdim 64 and 63: the normaliser's column opens a block of its own, or fills the last one."""
    W = 48
    mixer, w = _memory_mixer("mlstm", W, heads, dim, vdim, 50, {"gate_cap": cap})
    assert mixer.cache_need() is None and mixer.state_need().shape == (heads * dim * (vdim + 1) + heads,)
    m = {"heads": heads, "dim": dim, "vdim": vdim, "gate_cap": cap}
    _walk_a_memory_mixer(mixer, lambda x: TP.matrix_memory(x, w, m, 1e-5), W, [150, 1, 37], 8, 3e-5)


@pytest.mark.parametrize("kind", ["retention", "mlstm"])
def test_long_prompts_of_the_memories_walk_their_segments_side_by_side(kind):
    """From 512 rows on: beside a long prompt a short one and one that ends inside a segment; then a long portion
    onto a state that is not empty, then single tokens."""
    from quicknn_b200.cache import KVCache
    from quicknn_b200.kernels import ops
    from quicknn_b200.parts import PartSpec
    W, heads, dim, vdim = 32, 2, 24, 40
    if kind == "retention":
        decay = [0.98, 0.9995]
        pos = PartSpec("rotary", {"head_dim": dim, "theta": 1e4, "rotary_dim": 16, "layout": "half"})
        mixer, w = _memory_mixer(kind, W, heads, dim, vdim, 70, {"decay": decay, "position": pos})
        m = {"heads": heads, "dim": dim, "vdim": vdim, "decay": decay, "rot": {"base": 1e4, "dims": 16}}
        plain = lambda x: TP.retention(x, w, m, 1e-5)  # noqa: E731
    else:
        mixer, w = _memory_mixer(kind, W, heads, dim, vdim, 80, {"gate_cap": 10.0}, gate_scale=0.15)
        m = {"heads": heads, "dim": dim, "vdim": vdim, "gate_cap": 10.0}
        plain = lambda x: TP.matrix_memory(x, w, m, 1e-5)  # noqa: E731
    cache = KVCache([None], [mixer.state_need()], 4096, 3, 2048, torch.float32, DEV)
    lens = [700, 5, 300]
    assert max(lens) >= ops.GLA_SEGMENTS_FROM
    xs = [rnd((n + 650, W), 40 + i) for i, n in enumerate(lens)]
    ref = [plain(x.astype(np.float64)) for x in xs]
    slots = [cache.allocate() for _ in lens]

    def check(y, want):
        assert np.abs(host(y) - want).max() < 5e-5 * max(1.0, np.abs(want).max())
    step = part_step(lens, [0, 0, 0], slots, "prefill", torch.float32, cache, mixer)
    check(mixer.forward(dev(np.concatenate([x[:n] for x, n in zip(xs, lens)])), step, cache.line(0)),
          np.concatenate([r[:n] for r, n in zip(ref, lens)]))
    step = part_step([600, 1], [700, 300], [slots[0], slots[2]], "extend", torch.float32, cache, mixer)
    check(mixer.forward(dev(np.concatenate([xs[0][700:1300], xs[2][300:301]])), step, cache.line(0)),
          np.concatenate([ref[0][700:1300], ref[2][300:301]]))
    step = part_step([1, 1], [1300, 301], [slots[0], slots[2]], "decode", torch.float32, cache, mixer)
    check(mixer.forward(dev(np.stack([xs[0][1300], xs[2][301]])), step, cache.line(0)), np.stack([ref[0][1300], ref[2][301]]))


def test_a_memory_still_holds_a_token_from_hundreds_of_rows_back():
    """A decay of nearly 1 and a first row whose key and value stand out: the read-out hundreds of rows later is that
    row's value, and with a fast decay it is not.  A state that lost its early rows would fail the first half."""
    from quicknn_b200.cache import KVCache
    from quicknn_b200.parts import PartSpec
    W, heads, dim, vdim, n = 16, 2, 8, 8, 400
    decay = [0.9999, 0.5]
    pos = PartSpec("rotary", {"head_dim": dim, "theta": 1e4, "rotary_dim": 0, "layout": "half"})
    mixer, w = _memory_mixer("retention", W, heads, dim, vdim, 90, {"decay": decay, "position": pos})
    x = rnd((n, W), 91, 0.05)
    x[0] = 30.0 * rnd(W, 92)                    # one loud row at the start, the query's row the same direction
    x[-1] = x[0] / 30.0
    m = {"heads": heads, "dim": dim, "vdim": vdim, "decay": decay, "rot": {"base": 1e4, "dims": 0}}
    ref = TP.retention(x.astype(np.float64), w, m, 1e-5)
    quiet = x.copy()
    quiet[0] = 0.0
    assert np.abs(ref[-1] - TP.retention(quiet.astype(np.float64), w, m, 1e-5)[-1]).max() > 0.1 * np.abs(ref[-1]).max()
    cache = KVCache([None], [mixer.state_need()], 1024, 2, 1024, torch.float32, DEV)
    s = cache.allocate()
    step = part_step([n - 1], [0], [s], "prefill", torch.float32, cache, mixer)
    mixer.forward(dev(x[:n - 1]), step, cache.line(0))
    step = part_step([1], [n - 1], [s], "decode", torch.float32, cache, mixer)
    y = host(mixer.forward(dev(x[n - 1:]), step, cache.line(0)))
    assert np.abs(y[0] - ref[-1]).max() < 3e-5 * max(1.0, np.abs(ref).max())


# ---- the attention mixer's options alone ---------------------------------------------------------------------------

def _attention_mixer(W, m, biased, layout, dtype, seed, shared=False, tie_qk=False):
    from quicknn_b200.parts import MIXERS, PartSpec
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos = {"head_dim": d, "theta": m["rot"]["base"], "rotary_dim": m["rot"]["dims"], "layout": layout}
    if m["rot"].get("scaling"):
        pos["scaling"] = m["rot"]["scaling"]
    size = (m.get("mask") or {}).get("size")
    spec = PartSpec("attention", {"hidden_size": W, "n_heads": H, "n_kv_heads": G, "head_dim": d, "v_head_dim": dv,
                                  "scale": m["scale"], "softcap": None, "window": size, "bias": biased,
                                  "qk_norm": {"eps": 1e-5}, "shared_kv": shared, "position": PartSpec("rotary", pos)})
    mixer = MIXERS.get("attention")(spec)
    w = {"q": rnd((H * d, W), seed + 1, 0.3), "k": rnd((G * d, W), seed + 2, 0.3), "v": rnd((G * dv, W), seed + 3, 0.3),
         "o": rnd((W, H * dv), seed + 4, 0.3), "q.norm": rnd(d, seed + 5, 0.2) + 1, "k.norm": rnd(d, seed + 6, 0.2) + 1}
    if biased:
        w.update({"q.b": rnd(H * d, seed + 7, 0.5), "k.b": rnd(G * d, seed + 8, 0.5), "v.b": rnd(G * dv, seed + 9, 0.5),
                  "o.b": rnd(W, seed + 10, 0.5)})
    if tie_qk:                        # a key matches the query of the same row's direction in the first head(s)
        w["k"] = w["q"][:G * d].copy()
        w["q.norm"] = w["k.norm"] = np.ones(d, dtype=np.float32)
    w = {k: bf(v) for k, v in w.items()}
    names = {"q": "q_proj", "k": "k_proj", "v": "v_proj", "o": "o_proj", "q.norm": "q_norm", "k.norm": "k_norm",
             "q.b": "q_bias", "k.b": "k_bias", "v.b": "v_bias", "o.b": "o_bias"}
    want = set(type(mixer).param_shapes(spec))
    mixer.load({names[k]: dev(v, dtype) for k, v in w.items() if names[k] in want}, dtype, DEV)
    return mixer, f64(w)


@pytest.mark.parametrize("dtype,d,dv,G,window,rot,layout,biased", [
    (torch.float32, 16, 24, 2, None, 16, "half", True), (torch.float32, 24, 8, 1, 9, 12, "interleaved", False),
    (torch.float32, 12, 20, 4, 64, 0, "half", True), (torch.float32, 20, 12, 2, 65, 20, "interleaved", True),
    (torch.float32, 64, 64, 1, 1, 32, "interleaved", False), (torch.float32, 32, 32, 2, 63, 32, "half", False),
    (torch.bfloat16, 64, 40, 1, None, 64, "half", True), (torch.bfloat16, 64, 64, 2, 70, 32, "interleaved", False),
    (torch.bfloat16, 96, 80, 1, 44, 32, "interleaved", False), (torch.bfloat16, 128, 64, 4, 130, 64, "half", True),
    (torch.bfloat16, 24, 40, 2, 7, 24, "half", True)])
def test_attention_with_its_options_alone_and_a_window_one_token_off_would_show(dtype, d, dv, G, window, rot, layout, biased):
    """A prompt longer than the window and two pages, then 70 tokens one by one across a page edge and the ring, then
    a portion; in float32 the scores are scaled until attention is nearly one-hot, so that a window one token off, a
    key at the wrong page or a pairing of the wrong columns moves the output."""
    from quicknn_b200.cache import KVCache
    W, H = 64, 4
    sharp = dtype == torch.float32
    m = _att(H, G, d, dv, 2.0 if sharp else 0.3, _rot(700.0, rot, (4.0, 1.0, 4.0, 32) if layout == "interleaved" else None),
             window=window)
    mixer, w = _attention_mixer(W, m, biased, layout, dtype, 100)
    need = mixer.cache_need()
    D = d if d == dv and d % 8 == 0 else (max(d, dv) + 7) // 8 * 8
    assert (need.n_kv_heads, need.head_dim, need.window) == (G, D, window)
    n, single, portion = 150, 70, 6
    x = bf(rnd((n + single + portion, W), 7))
    ref, _ = TP.attention(x.astype(np.float64), w, m, 1e-5, interleaved=layout == "interleaved")
    if window is not None and window > 1 and sharp:
        wrong = dict(m, mask={"size": window - 1})
        off, _ = TP.attention(x.astype(np.float64), w, wrong, 1e-5, interleaved=layout == "interleaved")
        assert np.abs(off - ref).max() > 0.05 * np.abs(ref).max()
    cache = KVCache([need], [None], 1024, 2, 512, dtype, DEV)
    s = cache.allocate()
    tol = (3e-5 if sharp else 0.03) * max(1.0, np.abs(ref).max())
    step = part_step([n], [0], [s], "prefill", dtype, cache, mixer)
    assert np.abs(host(mixer.forward(dev(x[:n], dtype), step, cache.line(0))) - ref[:n]).max() < tol
    for t in range(n, n + single):
        step = part_step([1], [t], [s], "decode", dtype, cache, mixer)
        y = host(mixer.forward(dev(x[t:t + 1], dtype), step, cache.line(0)))
        assert np.abs(y - ref[t:t + 1]).max() < tol, f"position {t}"
    t = n + single
    step = part_step([portion], [t], [s], "extend", dtype, cache, mixer)
    step.whole = None
    assert np.abs(host(mixer.forward(dev(x[t:], dtype), step, cache.line(0))) - ref[t:]).max() < tol


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_a_far_key_that_one_score_singles_out(dtype):
    """Among 600 keys the third one is made to match the last query (the key matrix is the first head's query matrix,
    and the head norms make a row's size irrelevant to its direction), while its value is five times the last row's own:
    without a window the output is dominated by that far value, with a window of 500 it is not, and the kernels give
    the plain result in both cases."""
    from quicknn_b200.cache import KVCache
    W, H, G, d, dv, n = 32, 2, 1, 32, 16, 600
    outs = {}
    for window in (None, 500):
        m = _att(H, G, d, dv, 1.0, _rot(1e4, 0), window=window)
        mixer, w = _attention_mixer(W, m, False, "half", dtype, 200, tie_qk=True)
        x = bf(rnd((n, W), 8, 0.3))
        x[2] = bf(5.0 * rnd(W, 9))
        x[-1] = bf(x[2] / 5.0)
        ref, _ = TP.attention(x.astype(np.float64), w, m, 1e-5)
        outs[window] = ref[-1]
        cache = KVCache([mixer.cache_need()], [None], 1024, 1, 1024, dtype, DEV)
        s = cache.allocate()
        step = part_step([n - 1], [0], [s], "prefill", dtype, cache, mixer)
        mixer.forward(dev(x[:n - 1], dtype), step, cache.line(0))
        step = part_step([1], [n - 1], [s], "decode", dtype, cache, mixer)
        y = host(mixer.forward(dev(x[n - 1:], dtype), step, cache.line(0)))
        assert np.abs(y - ref[-1:]).max() < (3e-5 if dtype == torch.float32 else 0.03) * max(1.0, np.abs(ref).max())
    assert np.abs(outs[None] - outs[500]).max() > 0.3 * np.abs(outs[None]).max()       # the far key does carry weight


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_a_layer_that_reads_another_layers_keys_and_values(dtype):
    """Two mixers over one cache line: the second has queries only.  Prompts of unequal lengths, single tokens, a portion."""
    from quicknn_b200.cache import KVCache
    W = 48
    m = _att(4, 2, 16, 24, 0.4, _rot(900.0, 8))
    owner, w1 = _attention_mixer(W, m, True, "half", dtype, 300)
    reader, w2 = _attention_mixer(W, m, True, "half", dtype, 400, shared=True)
    assert "k_proj" not in type(reader).param_shapes(reader.spec) and "k_norm" not in type(reader).param_shapes(reader.spec)
    lens, more = [70, 5, 129], 6
    xs = [bf(rnd((n + more, W), 30 + i)) for i, n in enumerate(lens)]
    ys = [bf(rnd((n + more, W), 40 + i)) for i, n in enumerate(lens)]          # the reader's input differs from the owner's
    refs = []
    for x, y in zip(xs, ys):
        _, kv = TP.attention(x.astype(np.float64), w1, m, 1e-5)
        refs.append(TP.attention(y.astype(np.float64), w2, m, 1e-5, kv=kv)[0])
    cache = KVCache([owner.cache_need()], [None], 1024, 3, 512, dtype, DEV)
    slots = [cache.allocate() for _ in lens]
    tol = (3e-5 if dtype == torch.float32 else 0.03) * max(1.0, max(np.abs(r).max() for r in refs))

    def both(mode, counts, starts, who):
        step = part_step(counts, starts, [slots[i] for i in who], mode, dtype, cache, owner)
        step.whole = None
        owner.forward(dev(np.concatenate([xs[i][s:s + c] for i, s, c in zip(who, starts, counts)]), dtype), step,
                      cache.line(0, writes=True))
        got = host(reader.forward(dev(np.concatenate([ys[i][s:s + c] for i, s, c in zip(who, starts, counts)]), dtype), step,
                                  cache.line(0, writes=False)))
        want = np.concatenate([refs[i][s:s + c] for i, s, c in zip(who, starts, counts)])
        assert np.abs(got - want).max() < tol, mode
    both("prefill", lens, [0, 0, 0], [0, 1, 2])
    both("decode", [1, 1, 1], lens, [0, 1, 2])
    both("extend", [more - 1, 2], [lens[0] + 1, lens[2] + 1], [0, 2])


def test_branches_side_by_side_share_one_cache_line():
    """The parallel mixer hands each branch what it asked for: keys and values to the one, a state to the other."""
    from quicknn_b200.cache import KVCache
    from quicknn_b200.parts import MIXERS, PartSpec
    W = 40
    left = PartSpec("attention", {"hidden_size": W, "n_heads": 2, "n_kv_heads": 1, "head_dim": 8, "v_head_dim": 16,
                                  "scale": 0.3, "softcap": None, "window": 5, "bias": False, "qk_norm": {"eps": 1e-5},
                                  "position": PartSpec("rotary", {"head_dim": 8, "theta": 100.0, "rotary_dim": 4,
                                                                  "layout": "interleaved"})})
    right = PartSpec("mlstm", {"hidden_size": W, "n_heads": 2, "dim": 8, "vdim": 4, "gate_cap": 6.0, "eps": 1e-5})
    spec = PartSpec("parallel", {"hidden_size": W, "eps": 1e-5, "branches": {"left": left, "right": right}})
    mixer = MIXERS.get("parallel")(spec)
    shapes = type(mixer).param_shapes(spec)
    assert shapes["left.out"] == ((W,), "scale") and "right.i_bias" in shapes and "left.k_norm" in shapes
    w = {k: (rnd(s, 500 + i, 0.3) + (1.0 if role == "scale" else 0.0)) for i, (k, (s, role)) in enumerate(shapes.items())}
    mixer.load({k: dev(v) for k, v in w.items()}, torch.float32, DEV)
    assert mixer.cache_need().window == 5 and mixer.state_need().shape == (2 * 8 * 5 + 2,)
    ck = {"left.q": "left.q_proj", "left.k": "left.k_proj", "left.v": "left.v_proj", "left.o": "left.o_proj",
          "left.q.norm": "left.q_norm", "left.k.norm": "left.k_norm", "left.out": "left.out", "right.out": "right.out",
          "right.g": "right.gate", "right.i.b": "right.i_bias", "right.f.b": "right.f_bias"}
    for n in ("q", "k", "v", "o", "norm", "i", "f"):
        ck[f"right.{n}"] = f"right.{n}"
    wp = f64({c: w[l] for c, l in ck.items()})
    m = {"left": _att(2, 1, 8, 16, 0.3, _rot(100.0, 4), window=5), "right": _mem(2, 8, 4, 6.0)}
    x = rnd((30, W), 9)
    ref = TP.parallel(x.astype(np.float64), wp, m, 1e-5)
    cache = KVCache([mixer.cache_need()], [mixer.state_need()], 256, 2, 128, torch.float32, DEV)
    s = cache.allocate()
    step = part_step([20], [0], [s], "prefill", torch.float32, cache, mixer)
    assert np.abs(host(mixer.forward(dev(x[:20]), step, cache.line(0))) - ref[:20]).max() < 3e-5 * np.abs(ref).max()
    for t in range(20, 30):
        step = part_step([1], [t], [s], "decode", torch.float32, cache, mixer)
        assert np.abs(host(mixer.forward(dev(x[t:t + 1]), step, cache.line(0))) - ref[t:t + 1]).max() < 3e-5 * np.abs(ref).max()


# ---- whole models -----------------------------------------------------------------------------------------------

@pytest.mark.parametrize("name,dtype,peaky", [("A", "float32", True), ("A", "bfloat16", False), ("B", "float32", True),
                                              ("B", "bfloat16", False), ("C", "float32", True), ("C", "bfloat16", False),
                                              ("A", "float32", False)])
def test_every_cutting_gives_the_plain_logits(tumu, tmp_path, whole_model_tolerance, name, dtype, peaky):
    folder, plain = tumu(name, dtype, peaky)
    requests = prompts(name, LENGTHS_B if name == "B" else LENGTHS)
    ref = [plain.logits(t) for t in requests]
    replay = Replay(folder, dtype, tmp_path, max_tokens=576 if name == "B" else 384)
    try:
        worst = run_all_cuttings(replay, requests, ref, dtype)
    finally:
        replay.close()
    print(f"tumudra {name} {dtype} peaky={peaky}: largest error {worst:.3g}")


def test_the_stream_after_every_layer(tumu):
    """float32, layer by layer: what each block leaves in the stream is the plain implementation's."""
    from quicknn_b200.engine import Engine, Model
    for name in ("A", "B", "C"):
        folder, plain = tumu(name, "float32", True)
        toks = prompts(name, [90], seed=11)[0]
        want = plain.residual_stream(toks)[1:]
        model = Model.from_folder(folder, "float32", DEV)
        seen = []
        for blk in model.blocks:
            def wrapped(resid, step, line, normed=None, next_norm=None, _inner=blk.forward):
                out = _inner(resid, step, line, normed=normed, next_norm=next_norm)
                seen.append(host(out[0] if isinstance(out, tuple) else out))
                return out
            blk.forward = wrapped
        eng = Engine(model, max_tokens=256)
        eng.step([(eng.new_sequence(), toks)], "last")
        assert len(seen) == len(want)
        for i, (g, r) in enumerate(zip(seen, want)):
            assert np.abs(g - r).max() < 3e-5 * max(1.0, np.abs(r).max()), f"model {name}, layer {i}"


@pytest.mark.parametrize("name,dtype,peaky", [("A", "float32", True), ("B", "float32", True), ("B", "bfloat16", False),
                                              ("A", "bfloat16", False), ("C", "float32", True)])
def test_prompts_in_portions_down_to_two_tokens(tumu, tmp_path, name, dtype, peaky):
    """Steps that continue sequences by several tokens, beside requests that join or sit out."""
    folder, plain = tumu(name, dtype, peaky)
    big = name == "B"
    requests = prompts(name, [257, 170, 45] if big else [129, 70, 45], seed=7)
    ref = [plain.logits(t) for t in requests]
    replay = Replay(folder, dtype, tmp_path, max_tokens=576 if big else 384)
    pos = [0, 0, 0]

    def step(*parts, end=()):
        entries = [(f"r{i}", requests[i][pos[i]:pos[i] + n], range(n)) for i, n in parts]
        got = replay.step(entries, end=[f"r{i}" for i in end])
        r = 0
        for i, n in parts:
            ok, err, tol = near(got[r:r + n], ref[i][pos[i]:pos[i] + n], dtype)
            assert ok, f"request {i} positions {pos[i]}..{pos[i] + n - 1}: error {err:.3g} > {tol:.3g}"
            pos[i] += n
            r += n
    try:
        a, b = len(requests[0]), len(requests[1])
        step((0, 2), (1, 62))
        step((0, 62))                            # request 1 sits out; request 0 reaches the page edge
        step((0, 2), (1, 2), (2, 40))            # portions of two across the edge; request 2 joins
        step((0, 1), (1, 1), (2, 1))
        step((0, a - 67 - 3), (2, 4), end=[2])   # a portion longer than the windows
        step((0, 3), (1, b - 65), end=[0, 1])
        assert pos == [a, b, 45]
        got = replay.step([("again", requests[0], [a - 1])], end=["again"])      # what they held is free again
        ok, err, tol = near(got, ref[0][a - 1:a], dtype)
        assert ok, (err, tol)
    finally:
        replay.close()


@pytest.mark.parametrize("name", ["A", "C"])
def test_greedy_generation_through_the_entry_point(tumu, name):
    """More requests than slots, so that slots, pages and states are handed out again; decode steps run from CUDA
    graphs, one step ahead of the host; the tokens are the plain implementation's."""
    from quicknn_b200.engine import LLM
    from quicknn_b200.sampling import GenerationOptions
    folder, plain = tumu(name, "float32", True)
    reqs = prompts(name, [5, 70, 1, 33, 12], seed=3)
    llm = LLM(folder, max_context=256, max_batch=2, dtype="float32")
    res = llm.generate(reqs, GenerationOptions.greedy(12), stop_ids=[])
    for r, p in zip(res, reqs):
        seq = list(p)
        for t in r.tokens:                      # the best token at its place (a tie within rounding may go either way)
            row = plain.logits(seq)[-1]
            assert row[t] >= row.max() - 1e-4 * max(1.0, np.abs(row).max()), f"request {r.index}"
            seq.append(t)
    llm16 = LLM(folder, max_context=256, max_batch=4, dtype="bfloat16")
    for r, p in zip(llm16.generate(reqs, GenerationOptions.greedy(6), stop_ids=[]), reqs):
        seq = list(p)
        for t in r.tokens:                      # bfloat16: every token is at least a near-best one of the plain logits
            row = plain.logits(seq)[-1]
            assert row[t] >= row.max() - 0.1 * max(1.0, np.abs(row).max())
            seq.append(t)


def test_long_decoding_keeps_state_window_and_shared_keys(tumu):
    """150 tokens generated one by one after a short prompt: the window of 9 and the ring of a page pass over decoded
    tokens, the states are carried all the way, the shared layer reads what its owner appended."""
    from quicknn_b200.engine import LLM
    from quicknn_b200.sampling import GenerationOptions
    folder, plain = tumu("A", "float32", True)
    p = prompts("A", [3], seed=9)[0]
    llm = LLM(folder, max_context=256, max_batch=1, dtype="float32")
    got = llm.generate([p], GenerationOptions.greedy(150), stop_ids=[])[0].tokens
    seq = p + got
    ref = plain.logits(seq[:-1])
    for i, t in enumerate(got):
        row = ref[len(p) - 1 + i]
        assert row[t] >= row.max() - 1e-4 * max(1.0, np.abs(row).max()), f"token {i}"


def test_the_command_line_serves_the_design(tumu, tmp_path):
    import subprocess
    import sys
    from conftest import ROOT

    def run(*argv):
        return subprocess.run([sys.executable, "-m", "quicknn_b200", *argv], cwd=ROOT, capture_output=True, text=True)
    folder, plain = tumu("A", "float32", True)
    r = run("info", "--model", folder)
    assert r.returncode == 0, r.stderr
    info = json.loads(r.stdout)
    assert info["architecture"] == "Tumudra" and info["layers"] == len(TUMU_A["layers"])
    p = prompts("A", [9, 4], seed=5)
    r = run("generate", "--model", folder, "--prompt-ids", ";".join(",".join(map(str, q)) for q in p), "--max-new-tokens", "8",
            "--temperature", "0", "--dtype", "float32", "--max-context", "64", "--stop-ids", "")
    assert r.returncode == 0, r.stderr
    got = [json.loads(l) for l in r.stdout.splitlines() if l.strip()]
    assert [g["tokens"] for g in got] == [plain.greedy(q, 8) for q in p]
    # a model folder with random weights from a configuration file, and its replay
    cfg = tmp_path / "cfg.json"
    cfg.write_text(json.dumps(TUMU_C))
    out = tmp_path / "random_c"
    r = run("random", "--config", str(cfg), "--seed", "3", "--out", str(out), "--dtype", "bfloat16")
    assert r.returncode == 0, r.stderr
    ref = TP.PlainTumudra(str(out))
    toks = prompts("C", [21], seed=6)[0]
    replay = Replay(str(out), "float32", tmp_path / "logits", max_tokens=64)       # bfloat16 weights, widened exactly
    try:
        got = replay.step([("x", toks, range(len(toks)))], end=["x"])
    finally:
        replay.close()
    ok, err, tol = close(got, ref.logits(toks), "float32")
    assert ok, (err, tol)


def test_layer_sizes_that_take_the_tensor_core_kernels(tmp_path):
    """Head size 128 (the tcgen05 prompt attention and the tensor-core decode attention, also for the layer on shared keys
    and values and for values carried wider than they are), products of several hundred rows (the tcgen05 GEMMs with the
    squared relu in their epilogue), prompts long enough for the memories' segments and for a window to pass inside a
    prompt; then single tokens."""
    from quicknn_b200.engine import Engine, Model
    att = _att(4, 1, 128, 64, 0.09, _rot(1e5, 128))
    raw = dict(architecture="Tumudra", vocab=1000, width=512, embedding={"scale": 2.0}, norm={"eps": 1e-5}, initializer_range=0.04,
               layers=[_layer("parallel", {"left": _att(4, 2, 128, 128, 0.1, _rot(2e4, 64, (8.0, 1.0, 4.0, 256)), window=300),
                                           "right": _mem(2, 64, 128, 10.0)}, 768),
                       _layer("attention", att, 1024),
                       _layer("retention", _ret(2, 128, 64, [0.97, 0.999], _rot(1e4, 128)), None),
                       _layer("attention", dict(att, kv_from=1), 768)])
    CONFIGS["L"] = (raw, 21)
    lens, extra = [600, 130], 3
    reqs = prompts("L", [n + extra for n in lens], seed=4)
    for dtype in ("float32", "bfloat16"):
        folder = make_folder(tmp_path, "L", dtype, False)
        plain = TP.PlainTumudra(folder)
        ref = [plain.logits(t) for t in reqs]
        eng = Engine(Model.from_folder(folder, dtype, DEV), max_tokens=2048)
        slots = [eng.new_sequence() for _ in reqs]
        got = eng.step([(s, t[:n]) for s, t, n in zip(slots, reqs, lens)], "all").cpu().numpy()
        at = 0
        for r, n in zip(ref, lens):
            ok, err, tol = near(got[at:at + n], r[:n], dtype)
            assert ok, f"{dtype}: prompt of {n}: error {err:.3g} > {tol:.3g}"
            at += n
        for t in range(extra):
            got = eng.step([(s, [q[n + t]]) for s, q, n in zip(slots, reqs, lens)], "last").cpu().numpy()
            for i, (r, n) in enumerate(zip(ref, lens)):
                ok, err, tol = near(got[i:i + 1], r[n + t:n + t + 1], dtype)
                assert ok, f"{dtype}: request {i} decoded token {t}: error {err:.3g} > {tol:.3g}"


# ---- configurations drawn at random ---------------------------------------------------------------------------------

def random_config(seed):
    """Every size, the order of the layers and every constant drawn from a seed."""
    rng = np.random.default_rng(2000 + seed)
    pick = lambda xs: xs[int(rng.integers(len(xs)))]  # noqa: E731

    def softmax(window_from):
        G = pick([1, 2, 3])
        d = pick([8, 12, 16, 24, 32, 64])
        scaling = pick([None, (pick([2.0, 8.0, 32.0]), pick([0.5, 1.0]), pick([2.0, 4.0]), pick([16, 64, 1024]))])
        return _att(G * pick([1, 2, 4]), G, d, pick([8, 16, 20, 32, 64]), float(rng.uniform(0.1, 0.4)),
                    _rot(pick([100.0, 1e4, 1e6]), pick([0, d // 2 // 2 * 2, d]), scaling), window=pick(window_from))
    width = pick([48, 64, 96, 100, 160])
    layers, owners = [], []
    for i in range(int(rng.integers(1, 7))):
        ff = pick([None, 32, 72, 128])
        kind = pick(["attention", "attention", "parallel", "retention"])
        if kind == "attention":
            if owners and rng.random() < 0.4:
                j = pick(owners)
                layers.append(_layer(kind, dict(layers[j]["mixer"], kv_from=j), ff))
            else:
                owners.append(i)
                layers.append(_layer(kind, softmax([None]), ff))
        elif kind == "parallel":
            layers.append(_layer(kind, {"left": softmax([1, 3, 17, 63, 64, 65, 80, None]),
                                        "right": _mem(int(rng.integers(1, 5)), pick([4, 8, 16, 32, 64]), pick([8, 16, 63, 64]),
                                                      pick([1.0, 12.0, 30.0]))}, ff))
        else:
            H, d = int(rng.integers(1, 5)), pick([8, 16, 32, 64, 128])
            layers.append(_layer(kind, _ret(H, d, pick([8, 16, 32, 64]), [float(1 - 2.0 ** -rng.uniform(1, 12)) for _ in range(H)],
                                            _rot(pick([1e3, 1e6]), pick([0, d // 2, d]))), ff))
    return dict(architecture="Tumudra", vocab=int(rng.integers(100, 700)), width=width,
                embedding={"scale": float(pick([1.0, 4.0, 11.5]))}, norm={"eps": pick([1e-5, 1e-6])},
                initializer_range=0.07, layers=layers)


@pytest.mark.parametrize("seed", range(24))
def test_configurations_drawn_at_random(tmp_path, seed):
    """Prompts of unequal lengths in one step, then tokens one by one, against the plain logits: float32 sharply for
    every configuration, bfloat16 for every other one."""
    from quicknn_b200.engine import Engine, Model
    raw = random_config(seed)
    name = f"R{seed}"
    CONFIGS[name] = (raw, 50 + seed)
    lens, extra = [130, 7, 1, 70], 5
    reqs = prompts(name, [n + extra for n in lens], seed=seed)
    for dtype in (("float32", "bfloat16") if seed % 2 == 0 else ("float32",)):
        folder = make_folder(tmp_path, name, dtype, dtype == "float32")
        plain = TP.PlainTumudra(folder)
        ref = [plain.logits(t) for t in reqs]
        eng = Engine(Model.from_folder(folder, dtype, DEV), max_tokens=1024)
        slots = [eng.new_sequence() for _ in reqs]
        got = eng.step([(s, t[:n]) for s, t, n in zip(slots, reqs, lens)], "all").cpu().numpy()
        at = 0
        for r, n in zip(ref, lens):
            ok, err, tol = near(got[at:at + n], r[:n], dtype, 3e-4)
            assert ok, f"seed {seed} {dtype}: prompt of {n}: error {err:.3g} > {tol:.3g}  ({raw['layers']})"
            at += n
        for t in range(extra):
            got = eng.step([(s, [q[n + t]]) for s, q, n in zip(slots, reqs, lens)], "last").cpu().numpy()
            for i, (r, n) in enumerate(zip(ref, lens)):
                ok, err, tol = near(got[i:i + 1], r[n + t:n + t + 1], dtype, 3e-4)
                assert ok, f"seed {seed} {dtype}: request {i} decoded token {t}: error {err:.3g} > {tol:.3g}"
        for s in slots:
            eng.release(s)
        eng.cache.audit()
