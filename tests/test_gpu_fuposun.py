"""Fuposun on the GPU against the plain implementation (tests/plain/fuposun_plain.py): each mechanism alone
(gated linear attention with its state, latent attention with its window and cache line, routed experts, the
small kernels around them), then whole models through bin/trace_run under every cutting, in portions, and
through the entry point's generation loop.  The configurations are small and differ from one another in every
size; queries, keys, routers and decays are scaled so that a wrong key, a lost state or a window that is one
token off moves the logits far beyond the tolerance."""
import json
import os

import numpy as np
import pytest
import torch

from conftest import close
from plain import fuposun_plain as FP
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


# ---- configurations -------------------------------------------------------------------------------------

def _latent(heads, dim, vdim, q_rank, kv_rank, scale, window, mlp):
    m = {"heads": heads, "dim": dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank, "scale": scale}
    if window is not None:
        m["mask"] = {"size": window}
    return {"type": "latent_attention", "mixer": m, "mlp": mlp}


def _gla(heads, dim, vdim, tau, rank, mlp):
    return {"type": "gla", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau, "decay_rank": rank}, "mlp": mlp}


def _moe(experts, top, ff, limit, shared=None):
    m = {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff, "limit": limit}}
    if shared:
        m["shared"] = {"ff": shared[0], "limit": shared[1]}
    return m


# A: a recurrent layer first, two experts per token beside a shared one, a layer without a feed-forward and
#    without a window, one head, head sizes 64 (tensor-core kernels in bfloat16) and 32
FUPO_A = dict(architecture="Fuposun", vocab=300, width=64, residual_mult=0.5, logit_softcap=20.0, norm={"eps": 1e-6},
              initializer_range=0.08, layers=[
                  _gla(2, 16, 24, 8.0, 8, {"kind": "dense", "ff": 96}),
                  _latent(3, 16, 8, 24, 64, 0.2, 9, _moe(5, 2, 40, 0.3, (24, 1.2))),
                  _latent(2, 8, 16, 16, 32, 0.3, None, None),
                  _gla(1, 8, 8, 4.0, 4, _moe(3, 1, 16, 1.0))])
# B: latent sizes 128 and 256, windows beyond a page and beyond two, a multiplier of exactly 1, no softcap
FUPO_B = dict(architecture="Fuposun", vocab=512, width=128, residual_mult=1.0, logit_softcap=None, norm={"eps": 1e-5},
              initializer_range=0.06, layers=[
                  _latent(4, 32, 16, 64, 128, 0.17, 70, _moe(8, 2, 48, 0.5)),
                  _gla(2, 64, 32, 16.0, 16, {"kind": "dense", "ff": 192}),
                  _latent(1, 16, 32, 32, 256, 0.25, 130, {"kind": "dense", "ff": 64})])
# C: a width, ranks and head sizes that are no multiple of 8 or of 32
FUPO_C = dict(architecture="Fuposun", vocab=301, width=100, residual_mult=0.6, logit_softcap=15.0, norm={"eps": 1e-4},
              initializer_range=0.07, layers=[
                  _latent(5, 12, 20, 20, 48, 0.3, 11, {"kind": "dense", "ff": 70}),
                  _gla(3, 12, 20, 6.0, 5, _moe(4, 3, 28, 0.4, (36, 0.6)))])
CONFIGS = {"A": (FUPO_A, 3), "B": (FUPO_B, 4), "C": (FUPO_C, 5)}
LENGTHS = [70, 33, 129, 45, 100, 64]
LENGTHS_B = [170, 33, 257, 45, 100, 64]


def make_folder(base, name, storage, peaky, keep_rank=True):
    """Random weights; ``peaky`` scales what decides where attention and state look: the query and key sides of
    both mixers, and decay biases from fast to nearly none."""
    from quicknn_b200.config import FUPOSUN, FuposunConfig
    from quicknn_b200.weights import random_tensors, write_safetensors
    raw, seed = CONFIGS[name]
    cfg = FuposunConfig.from_dict(raw)
    d = os.path.join(str(base), f"fupo{name}_{storage}{'_peaky' if peaky else ''}{'' if keep_rank else '_norank'}")
    os.makedirs(d, exist_ok=True)
    tensors = dict(random_tensors(FUPOSUN, cfg, seed, torch.float32, 0.2))
    if peaky:
        for k in list(tensors):
            if k.endswith((".mix.uq", ".mix.uk")):
                tensors[k] = tensors[k] * 4.0
            elif k.endswith((".mix.q", ".mix.k")):
                tensors[k] = tensors[k] * 3.0
            elif k.endswith(".mix.a2.b"):
                tensors[k] = torch.linspace(-2.0, 9.0, tensors[k].numel())
    # Routing is made decisive, as a choice between experts must not hang on the rounding of an activation: the first
    # columns of the stream carry a ranking of the experts that the token's embedding sets (well separated values
    # in a random order) and every router reads its experts' columns only.
    most = max([l.mlp.experts for l in cfg.layers if l.mlp is not None and l.mlp.kind == "moe"] or [0])
    if most:
        g = torch.Generator().manual_seed(seed)
        ranks = torch.stack([torch.randperm(most, generator=g) for _ in range(cfg.vocab)]).float()
        tensors["embed"] = tensors["embed"] / raw["initializer_range"]          # entries of size 1 beside the ranking
        tensors["embed"][:, :most] = (ranks - (most - 1) / 2) * (12.0 / max(1, most - 1))
        for i, l in enumerate(cfg.layers):
            if l.mlp is not None and l.mlp.kind == "moe":
                r = torch.zeros_like(tensors[f"l{i}.mlp.router"])
                r[:, :l.mlp.experts] = 8.0 * torch.eye(l.mlp.experts)
                tensors[f"l{i}.mlp.router"] = r
                tensors[f"l{i}.norm2"][:most] = 1.0            # equal weights keep the ranking's spacing
        tensors["embed.norm"][:most] = 1.0
        for k in list(tensors):                            # and no layer writes into the ranking's columns
            if k.endswith((".mix.o", ".down")):
                tensors[k][:most] = 0.0
    dt = torch.float32 if storage == "float32" else torch.bfloat16
    out = cfg.to_dict()
    if not keep_rank:                      # as a file from elsewhere: the decay's rank is the tensor's extent
        for layer in out["layers"]:
            layer["mixer"].pop("decay_rank", None)
    with open(os.path.join(d, "config.json"), "w") as fh:
        json.dump(out, fh)
    write_safetensors(os.path.join(d, "model.safetensors"), {k: v.to(dt) for k, v in tensors.items()})
    return d


@pytest.fixture(scope="module")
def fupo(tmp_path_factory):
    base = tmp_path_factory.mktemp("fuposun")
    made = {}

    def get(name, storage="float32", peaky=False, keep_rank=True):
        key = (name, storage, peaky, keep_rank)
        if key not in made:
            folder = make_folder(base, name, storage, peaky, keep_rank)
            made[key] = (folder, FP.PlainFuposun(folder))
        return made[key]
    return get


def prompts(name, lengths, seed=0):
    rng = np.random.default_rng(100 + seed)
    return [rng.integers(1, CONFIGS[name][0]["vocab"], n).tolist() for n in lengths]


# ---- the small kernels ------------------------------------------------------------------------------------

@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_scaled_add_with_the_next_norm(dtype):
    from quicknn_b200.kernels import ops
    for rows, width in ((3, 100), (70, 64), (5, 2304)):
        resid, y, w = rnd((rows, width), 1, 2.0), bf(rnd((rows, width), 2)), bf(rnd(width, 3) + 1.0)
        r = dev(resid)
        out = ops.add_scaled_rmsnorm(r, dev(y, dtype), 0.7, dev(w, dtype), 1e-5, False, dtype)
        want = resid.astype(np.float64) + 0.7 * y
        assert np.abs(host(r) - want).max() < 1e-5
        ref = FP.rms_norm(want, w.astype(np.float64), 1e-5)
        assert np.abs(host(out) - ref).max() < (1e-5 if dtype == torch.float32 else 0.02) * np.abs(ref).max()
        r2 = dev(resid)
        assert ops.add_scaled_rmsnorm(r2, dev(y, dtype), 1.0) is None       # the add alone, a multiplier of 1
        assert np.abs(host(r2) - (resid.astype(np.float64) + y)).max() < 1e-5


def test_norms_over_pieces_of_rows_head_gates_and_float32_products():
    from quicknn_b200.kernels import ops
    x, w = rnd((9, 50), 1), rnd(20, 2) + 1.0
    out = torch.zeros((9, 70), device=DEV)
    ops.rmsnorm_cols(dev(x), 13, 20, dev(w), 1e-5, out, 5, 45)
    ref = FP.rms_norm(x[:, 13:33].astype(np.float64), w.astype(np.float64), 1e-5)
    got = host(out)
    assert np.abs(got[:, 5:25] - ref).max() < 1e-5 and np.abs(got[:, 45:65] - ref).max() < 1e-5
    assert not got[:, :5].any() and not got[:, 25:45].any() and not got[:, 65:].any()
    src, dst = rnd((4, 12), 3), torch.zeros((4, 30), device=DEV)
    ops.copy_cols(dev(src), dst, 7)
    assert np.array_equal(host(dst)[:, 7:19], src.astype(np.float64)) and not host(dst)[:, 19:].any()
    o, g = rnd((6, 3 * 10), 4), rnd((6, 3), 5, 2.0)
    t = dev(o)
    ops.scale_heads(t, dev(g), 3)
    ref = (o.reshape(6, 3, 10) * FP.sigmoid(g.astype(np.float64))[:, :, None]).reshape(6, 30)
    assert np.abs(host(t) - ref).max() < 1e-6
    for width in (20, 100, 2304):                               # the gate's logits formed in the same kernel
        xg, wg = bf(rnd((6, width), 9)), bf(rnd((3, width), 10, 0.2))
        for dt in (torch.float32, torch.bfloat16):
            t = dev(o)
            ops.gate_heads(t, dev(xg, dt), dev(wg, dt), 3)
            ref = (o.reshape(6, 3, 10) * FP.sigmoid(xg.astype(np.float64) @ wg.T.astype(np.float64))[:, :, None]).reshape(6, 30)
            assert np.abs(host(t) - ref).max() < 1e-5
    for K in (5, 16, 100, 321):                                 # a thread per output, a warp per row
        a, b = bf(rnd((11, K), 6)), bf(rnd((7, K), 7))
        for dt in (torch.float32, torch.bfloat16):
            got = host(ops.small_linear_f32(dev(a, dt), dev(b, dt)))
            assert np.abs(got - a.astype(np.float64) @ b.T).max() < 1e-4
    gu = rnd((5, 2 * 33), 8, 2.0)
    got = host(ops.gated_act_clamped(dev(gu), 0.9, 1.702))
    g_, u_ = np.minimum(gu[:, :33].astype(np.float64), 0.9), np.clip(gu[:, 33:].astype(np.float64), -0.9, 0.9)
    assert np.abs(got - g_ * FP.sigmoid(1.702 * g_) * (u_ + 1)).max() < 1e-6


# ---- the mixers alone ----------------------------------------------------------------------------------------

def part_step(lens, starts, slots, mode, dtype, cache, part):
    """A step as the engine would build it, for one part over a cache of its own."""
    from quicknn_b200.engine.batch import StepBatch
    i32 = lambda a: torch.tensor(np.asarray(a), dtype=torch.int32, device=DEV)  # noqa: E731
    T = sum(lens)
    pos = np.concatenate([np.arange(s, s + n) for s, n in zip(starts, lens)])
    slot = np.concatenate([np.full(n, s) for s, n in zip(slots, lens)])
    first = np.cumsum([0] + lens[:-1])
    row0 = np.concatenate([np.full(n, r) for r, n in zip(first, lens)])
    cache.extend([(s, st + n) for s, st, n in zip(slots, starts, lens)])
    cache.sync()
    step = StepBatch(mode, T, len(lens), i32(np.zeros(T)), i32(pos), i32(slot), i32(row0), i32(slots), i32([T - 1]),
                     dtype, max(lens), seq_row0=i32(first), seq_len=i32(lens), max_seq=cache.max_seq,
                     tuning={"decode_splits": 2})
    need = part.scratch_need(step)
    step.scratch = torch.empty(need, dtype=torch.uint8, device=DEV) if need else None
    return step


@pytest.mark.parametrize("heads,dim,vdim", [(2, 16, 24), (1, 12, 40), (3, 64, 32), (1, 200, 8)])
def test_gated_linear_attention_alone_prompts_then_single_tokens_then_a_reused_slot(heads, dim, vdim):
    from quicknn_b200.cache import KVCache
    from quicknn_b200.parts import MIXERS, PartSpec
    W, rank, tau = 48, 6, 5.0
    spec = PartSpec("gla", {"hidden_size": W, "n_heads": heads, "dim": dim, "vdim": vdim, "tau": tau, "decay_rank": rank,
                            "eps": 1e-5})
    mixer = MIXERS.get("gla")(spec)
    assert mixer.cache_need() is None and mixer.state_need().shape == (heads, dim, vdim)
    w = {"q": rnd((heads * dim, W), 1, 0.3), "k": rnd((heads * dim, W), 2, 0.3), "v": rnd((heads * vdim, W), 3, 0.3),
         "g": rnd((heads * vdim, W), 4, 0.3), "o": rnd((W, heads * vdim), 5, 0.3), "norm": rnd(vdim, 6, 0.2) + 1,
         "a1": rnd((rank, W), 7, 0.3), "a2": rnd((heads * dim, rank), 8, 0.5),
         "a2.b": np.linspace(-3, 10, heads * dim).astype(np.float32)}        # memories from a few tokens to thousands
    names = {"q": "q", "k": "k", "v": "v", "g": "gate", "o": "o", "norm": "norm", "a1": "a1", "a2": "a2", "a2.b": "a2_bias"}
    mixer.load({names[k]: dev(v) for k, v in w.items()}, torch.float32, DEV)
    cache = KVCache([None], [mixer.state_need()], 1024, 3, 512, torch.float32, DEV)
    m = {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau}
    w64 = {k: v.astype(np.float64) for k, v in w.items()}
    lens = [150, 1, 37]                       # a sequence that starts with one token among longer ones
    xs = [rnd((n + 5, W), 20 + i) for i, n in enumerate(lens)]
    ref = [FP.gla(x.astype(np.float64), w64, m, 1e-5) for x in xs]
    slots = [cache.allocate() for _ in lens][::-1]
    step = part_step(lens, [0, 0, 0], slots, "prefill", torch.float32, cache, mixer)
    y = host(mixer.forward(dev(np.concatenate([x[:n] for x, n in zip(xs, lens)])), step, cache.line(0)))
    want = np.concatenate([r[:n] for r, n in zip(ref, lens)])
    assert np.abs(y - want).max() < 2e-5 * max(1.0, np.abs(want).max())
    for t in range(2):                        # one token each
        step = part_step([1, 1, 1], [n + t for n in lens], slots, "decode", torch.float32, cache, mixer)
        y = host(mixer.forward(dev(np.stack([x[n + t] for x, n in zip(xs, lens)])), step, cache.line(0)))
        want = np.stack([r[n + t] for r, n in zip(ref, lens)])
        assert np.abs(y - want).max() < 2e-5 * max(1.0, np.abs(want).max())
    step = part_step([3, 2], [lens[0] + 2, lens[2] + 2], [slots[0], slots[2]], "extend", torch.float32, cache, mixer)
    y = host(mixer.forward(dev(np.concatenate([xs[0][152:155], xs[2][39:41]])), step, cache.line(0)))
    want = np.concatenate([ref[0][152:155], ref[2][39:41]])
    assert np.abs(y - want).max() < 2e-5 * max(1.0, np.abs(want).max())
    # a slot that is given back and handed out again starts from an empty state
    cache.free(slots[0])
    again = cache.allocate()
    assert again == slots[0]
    step = part_step([37], [0], [again], "prefill", torch.float32, cache, mixer)
    y = host(mixer.forward(dev(xs[2][:37]), step, cache.line(0)))
    assert np.abs(y - ref[2][:37]).max() < 2e-5 * max(1.0, np.abs(ref[2]).max())


def test_long_prompts_walk_their_segments_side_by_side():
    """From 512 rows on a step's sequences are cut into segments of 256 rows: beside a long prompt a short one
    (segments of no rows) and one that ends inside a segment; then a long portion onto a state that is not empty."""
    from quicknn_b200.cache import KVCache
    from quicknn_b200.kernels import ops
    from quicknn_b200.parts import MIXERS, PartSpec
    W, heads, dim, vdim, rank, tau = 32, 2, 24, 40, 4, 7.0
    spec = PartSpec("gla", {"hidden_size": W, "n_heads": heads, "dim": dim, "vdim": vdim, "tau": tau, "decay_rank": rank,
                            "eps": 1e-5})
    mixer = MIXERS.get("gla")(spec)
    w = {"q": rnd((heads * dim, W), 1, 0.3), "k": rnd((heads * dim, W), 2, 0.3), "v": rnd((heads * vdim, W), 3, 0.3),
         "g": rnd((heads * vdim, W), 4, 0.3), "o": rnd((W, heads * vdim), 5, 0.3), "norm": rnd(vdim, 6, 0.2) + 1,
         "a1": rnd((rank, W), 7, 0.3), "a2": rnd((heads * dim, rank), 8, 0.5),
         "a2.b": np.linspace(0, 11, heads * dim).astype(np.float32)}
    names = {"q": "q", "k": "k", "v": "v", "g": "gate", "o": "o", "norm": "norm", "a1": "a1", "a2": "a2", "a2.b": "a2_bias"}
    mixer.load({names[k]: dev(v) for k, v in w.items()}, torch.float32, DEV)
    cache = KVCache([None], [mixer.state_need()], 4096, 3, 2048, torch.float32, DEV)
    m = {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau}
    w64 = {k: v.astype(np.float64) for k, v in w.items()}
    lens = [700, 5, 300]
    assert max(lens) >= ops.GLA_SEGMENTS_FROM
    xs = [rnd((n + 650, W), 40 + i) for i, n in enumerate(lens)]
    ref = [FP.gla(x.astype(np.float64), w64, m, 1e-5) for x in xs]
    slots = [cache.allocate() for _ in lens]
    step = part_step(lens, [0, 0, 0], slots, "prefill", torch.float32, cache, mixer)
    y = host(mixer.forward(dev(np.concatenate([x[:n] for x, n in zip(xs, lens)])), step, cache.line(0)))
    want = np.concatenate([r[:n] for r, n in zip(ref, lens)])
    assert np.abs(y - want).max() < 3e-5 * max(1.0, np.abs(want).max())
    step = part_step([600, 1], [700, 300], [slots[0], slots[2]], "extend", torch.float32, cache, mixer)
    y = host(mixer.forward(dev(np.concatenate([xs[0][700:1300], xs[2][300:301]])), step, cache.line(0)))
    want = np.concatenate([ref[0][700:1300], ref[2][300:301]])
    assert np.abs(y - want).max() < 3e-5 * max(1.0, np.abs(want).max())
    step = part_step([1, 1], [1300, 301], [slots[0], slots[2]], "decode", torch.float32, cache, mixer)
    y = host(mixer.forward(dev(np.stack([xs[0][1300], xs[2][301]])), step, cache.line(0)))
    want = np.stack([ref[0][1300], ref[2][301]])
    assert np.abs(y - want).max() < 3e-5 * max(1.0, np.abs(want).max())


@pytest.mark.parametrize("dtype,kv_rank,window,H", [
    (torch.float32, 48, 7, 3), (torch.float32, 64, 64, 3), (torch.float32, 32, 65, 3), (torch.float32, 24, None, 3),
    (torch.bfloat16, 64, 9, 3), (torch.bfloat16, 128, 64, 3), (torch.bfloat16, 256, 65, 3),
    (torch.float32, 128, 80, 8), (torch.bfloat16, 128, 80, 8), (torch.bfloat16, 64, 1, 16),      # many heads on the one latent
    (torch.float32, 20, 6, 2), (torch.bfloat16, 20, 6, 2), (torch.bfloat16, 100, 40, 5)])      # ranks that are no multiple of 8
def test_latent_attention_alone_and_a_window_one_token_off_would_show(dtype, kv_rank, window, H):
    from quicknn_b200.cache import KVCache
    from quicknn_b200.parts import MIXERS, PartSpec
    # float32 is the sharp check: its scores are scaled until attention is nearly one-hot.  In bfloat16 that scaling
    # turns the rounding of the latent alone into errors of a tenth of the output (measured with every window and
    # both kinds of kernel alike), so the bfloat16 cases keep a milder scale and check kernels and cache addressing.
    W, dim, vdim, rq, scale = 64, 8, 24, 40, (1.5 if dtype == torch.float32 else 0.3)
    spec = PartSpec("latent_attention", {"hidden_size": W, "n_heads": H, "dim": dim, "vdim": vdim, "q_rank": rq,
                                         "kv_rank": kv_rank, "scale": scale, "window": window, "eps": 1e-5})
    mixer = MIXERS.get("latent_attention")(spec)
    need = mixer.cache_need()
    assert (need.n_kv_heads, need.head_dim, need.window, need.values) == (1, (kv_rank + 7) // 8 * 8, window, False)
    w = {"dq": rnd((rq, W), 1, 0.3), "dq.norm": rnd(rq, 2, 0.2) + 1, "uq": rnd((H * dim, rq), 3, 0.6),
         "dkv": rnd((kv_rank, W), 4, 0.3), "dkv.norm": rnd(kv_rank, 5, 0.2) + 1, "uk": rnd((H * dim, kv_rank), 6, 0.6),
         "uv": rnd((H * vdim, kv_rank), 7, 0.2), "g": rnd((H, W), 8, 0.3), "o": rnd((W, H * vdim), 9, 0.2)}
    w = {k: bf(v) for k, v in w.items()}
    names = {"dq": "dq", "dq.norm": "dq_norm", "uq": "uq", "dkv": "dkv", "dkv.norm": "dkv_norm", "uk": "uk", "uv": "uv",
             "g": "gate", "o": "o"}
    mixer.load({names[k]: dev(v, dtype) for k, v in w.items()}, dtype, DEV)
    cache = KVCache([need], [None], 1024, 3, 512, dtype, DEV)
    assert cache.line(0).v is cache.line(0).k or cache.line(0).v.data_ptr() == cache.line(0).k.data_ptr()
    m = {"heads": H, "dim": dim, "vdim": vdim, "scale": scale, "mask": None if window is None else {"size": window}}
    w64 = {k: v.astype(np.float64) for k, v in w.items()}
    lens = [200, 1, 67]
    extra = 70                                 # decoded one by one: the window passes over decoded tokens and a page edge
    xs = [bf(rnd((n + extra, W), 30 + i)) for i, n in enumerate(lens)]
    ref = [FP.latent_attention(x.astype(np.float64), w64, m, 1e-5) for x in xs]
    tol = (3e-5 if dtype == torch.float32 else 8e-2) * max(np.abs(r).max() for r in ref)
    if window is not None and dtype == torch.float32:      # the test can see an edge that is off by one
        for off in ((-1, 1) if window > 1 else (1,)):
            other = FP.latent_attention(xs[0].astype(np.float64), w64, dict(m, mask={"size": window + off}), 1e-5)
            assert np.abs(other - ref[0]).max() > 5 * tol
    slots = [cache.allocate() for _ in lens]
    step = part_step(lens, [0, 0, 0], slots, "prefill", dtype, cache, mixer)
    y = host(mixer.forward(dev(np.concatenate([x[:n] for x, n in zip(xs, lens)]), dtype), step, cache.line(0)))
    assert np.abs(y - np.concatenate([r[:n] for r, n in zip(ref, lens)])).max() < tol
    for t in range(extra - 4):
        step = part_step([1, 1, 1], [n + t for n in lens], slots, "decode", dtype, cache, mixer)
        y = host(mixer.forward(dev(np.stack([x[n + t] for x, n in zip(xs, lens)]), dtype), step, cache.line(0)))
        err = np.abs(y - np.stack([r[n + t] for r, n in zip(ref, lens)])).max()
        assert err < tol, f"decoded token {t}: {err} > {tol}"
    t = extra - 4                              # the last four as portions of 3 and 1 rows, one sequence sits out
    step = part_step([3, 1], [lens[0] + t, lens[2] + t], [slots[0], slots[2]], "extend", dtype, cache, mixer)
    y = host(mixer.forward(dev(np.concatenate([xs[0][lens[0] + t:lens[0] + t + 3], xs[2][lens[2] + t:lens[2] + t + 1]]), dtype),
                           step, cache.line(0)))
    want = np.concatenate([ref[0][lens[0] + t:lens[0] + t + 3], ref[2][lens[2] + t:lens[2] + t + 1]])
    assert np.abs(y - want).max() < tol
    cache.audit()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("experts,top,shared", [(5, 1, None), (6, 2, (24, 1.1)), (3, 3, None), (40, 4, (8, 0.4))])
@pytest.mark.parametrize("W,ff", [(72, 40), (128, 64), (352, 160)])
def test_routed_experts_alone(dtype, experts, top, shared, W, ff):
    """Widths in whole blocks of 32 take the tensor-core tiles in bfloat16 (16 rows, and 64 where the experts get many
    rows each), other widths and float32 the plain tiles; (352, 160): more than one block of inner elements."""
    from quicknn_b200.parts import FEED_FORWARDS, PartSpec
    limit = 0.35
    sh = None if shared is None else PartSpec("clamped_mlp", {"hidden_size": W, "intermediate_size": shared[0],
                                                              "limit": shared[1]})
    spec = PartSpec("routed_experts", {"hidden_size": W, "experts": experts, "top": top, "intermediate_size": ff,
                                       "limit": limit, "shared": sh})
    part = FEED_FORWARDS.get("routed_experts")(spec)
    w = {"router": bf(rnd((experts, W), 1, 0.5))}
    for e in range(experts):
        w[f"e{e}.gate"], w[f"e{e}.up"] = bf(rnd((ff, W), 10 + e, 0.3)), bf(rnd((ff, W), 60 + e, 0.3))
        w[f"e{e}.down"] = bf(rnd((W, ff), 110 + e, 0.3))
    if shared:
        w["shared.gate"], w["shared.up"] = bf(rnd((shared[0], W), 2, 0.3)), bf(rnd((shared[0], W), 3, 0.3))
        w["shared.down"] = bf(rnd((W, shared[0]), 4, 0.3))
    local = {"router": dev(w["router"], dtype)}
    for k, v in w.items():
        if k.startswith("e"):
            e, n = k[1:].split(".")
            local[f"experts.{e}.{n}_proj"] = dev(v, dtype)
        elif k.startswith("shared."):
            local[f"shared.{k[7:]}_proj"] = dev(v, dtype)
    part.load(local, dtype, DEV)
    mlp = {"router": {"experts": experts, "top": top}, "expert": {"ff": ff, "limit": limit},
           "shared": None if shared is None else {"ff": shared[0], "limit": shared[1]}}
    w64 = {k: v.astype(np.float64) for k, v in w.items()}
    for rows in (1, 3, 150, 700):              # fewer rows than experts, tiles that are not full, many tiles, large tiles
        x = bf(rnd((rows, W), 200 + rows))
        got = host(part.forward(dev(x, dtype), None))
        ref = FP.routed_ff(x.astype(np.float64), w64, mlp)
        assert np.abs(got - ref).max() < (2e-5 if dtype == torch.float32 else 3e-2) * max(1.0, np.abs(ref).max())
    if dtype == torch.bfloat16:
        # the three kinds of tile give the same sums: grouped tcgen05 tiles of 128 rows against mma.sync tiles of
        # 64 and 16 rows (or the plain tiles where the widths are no whole blocks of 32)
        from quicknn_b200.kernels import ops
        xb = dev(bf(rnd((700, W), 900)), dtype)
        sel_e, sel_w = ops.moe_route(xb, part.w_router, top)
        outs = [host(ops.moe_experts(xb, sel_e, sel_w, top, part.w_gate_up, part.w_down, ops.GATED_CLAMPED, limit, 1.702,
                                     True, None, grouped=g)) for g in (True, False)]
        few = host(ops.moe_experts(xb[:40].contiguous(), sel_e[:40 * top].contiguous(), sel_w[:40 * top].contiguous(), top,
                                   part.w_gate_up, part.w_down, ops.GATED_CLAMPED, limit, 1.702, True, None, grouped=False))
        scale = max(1.0, np.abs(outs[1]).max())
        assert np.abs(outs[0] - outs[1]).max() < 2e-2 * scale and np.abs(few - outs[1][:40]).max() < 2e-2 * scale
    # a row's result does not depend on the rows beside it
    x = bf(rnd((150, W), 350))
    alone = host(part.forward(dev(x[77:78], dtype), None))
    among = host(part.forward(dev(x, dtype), None))[77:78]
    assert np.abs(alone - among).max() < (1e-5 if dtype == torch.float32 else 2e-2) * max(1.0, np.abs(among).max())


# ---- whole models ---------------------------------------------------------------------------------------------

@pytest.mark.parametrize("name,dtype,peaky", [("A", "float32", True), ("A", "bfloat16", False), ("A", "bfloat16", True),
                                              ("B", "bfloat16", False), ("B", "float32", True),
                                              ("C", "float32", True), ("C", "bfloat16", False)])
def test_every_cutting_gives_the_plain_logits(fupo, tmp_path, name, dtype, peaky):
    """Each request whole; its last 32 tokens one by one; batches of unequal lengths that shrink, one batch after
    another, so that slots, pages and states are used again."""
    folder, plain = fupo(name, dtype, peaky, keep_rank=(name != "A"))
    requests = prompts(name, LENGTHS_B if name == "B" else LENGTHS)
    ref = [plain.logits(t) for t in requests]
    replay = Replay(folder, dtype, tmp_path, max_tokens=576 if name == "B" else 384)
    try:
        worst = run_all_cuttings(replay, requests, ref, dtype)
    finally:
        replay.close()
    print(f"fuposun {name} {dtype} peaky={peaky}: largest error {worst:.3g}")


@pytest.mark.parametrize("name,dtype,peaky", [("A", "float32", True), ("B", "float32", True), ("B", "bfloat16", False),
                                              ("A", "bfloat16", False), ("C", "float32", True)])
def test_prompts_in_portions_down_to_two_tokens(fupo, tmp_path, name, dtype, peaky):
    """Steps that continue sequences by several tokens, beside requests that join or sit out.  (With the scaled
    queries and keys the bfloat16 rounding of the activations alone moves model B's logits by a quarter of their
    size, in whole prompts as in portions; the sharp checks are the float32 ones.)"""
    folder, plain = fupo(name, dtype, peaky)
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
            ok, err, tol = close(got[r:r + n], ref[i][pos[i]:pos[i] + n], dtype)
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
        ok, err, tol = close(got, ref[0][a - 1:a], dtype)
        assert ok, (err, tol)
    finally:
        replay.close()


@pytest.mark.parametrize("name", ["A", "C"])
def test_greedy_generation_through_the_entry_point(fupo, name):
    """More requests than slots, so that slots and recurrent states are handed out again; decode steps run from
    CUDA graphs, one step ahead of the host; the tokens are the plain implementation's."""
    from quicknn_b200.engine import LLM
    from quicknn_b200.sampling import GenerationOptions
    folder, plain = fupo(name, "float32", True)
    reqs = prompts(name, [5, 70, 1, 33, 12], seed=3)
    llm = LLM(folder, max_context=256, max_batch=2, dtype="float32")
    res = llm.generate(reqs, GenerationOptions.greedy(12), stop_ids=[])
    for r, p in zip(res, reqs):
        assert r.tokens == plain.greedy(p, 12), f"request {r.index}"
    llm16 = LLM(folder, max_context=256, max_batch=4, dtype="bfloat16")
    for r, p in zip(llm16.generate(reqs, GenerationOptions.greedy(6), stop_ids=[]), reqs):
        seq = list(p)
        for t in r.tokens:                      # bfloat16: every token is at least a near-best one of the plain logits
            row = plain.logits(seq)[-1]
            assert row[t] >= row.max() - 0.1 * max(1.0, np.abs(row).max())
            seq.append(t)


def test_long_decoding_keeps_state_and_window(fupo):
    """150 tokens generated one by one after a short prompt: the windows (9 tokens; none) and the ring of a page
    pass over decoded tokens, the recurrent state is carried all the way."""
    from quicknn_b200.engine import LLM
    from quicknn_b200.sampling import GenerationOptions
    folder, plain = fupo("A", "float32", True)
    p = prompts("A", [3], seed=9)[0]
    llm = LLM(folder, max_context=256, max_batch=1, dtype="float32")
    got = llm.generate([p], GenerationOptions.greedy(150), stop_ids=[])[0].tokens
    seq = p + got
    ref = plain.logits(seq[:-1])
    for i, t in enumerate(got):                 # every generated token is the best one at its place
        row = ref[len(p) - 1 + i]
        assert row[t] >= row.max() - 1e-4 * max(1.0, np.abs(row).max()), f"token {i}"


# ---- configurations drawn at random ---------------------------------------------------------------------------------

def random_config(seed):
    """Every size, the order of the layers and every constant drawn from a seed."""
    rng = np.random.default_rng(1000 + seed)
    pick = lambda xs: xs[int(rng.integers(len(xs)))]  # noqa: E731
    width = pick([48, 64, 96, 100, 160, 352])
    layers = []
    for _ in range(int(rng.integers(1, 6))):
        kind = pick(["none", "dense", "moe", "moe"])
        if kind == "none":
            mlp = None
        elif kind == "dense":
            mlp = {"kind": "dense", "ff": pick([32, 72, 128, 256])}
        else:
            experts = int(rng.integers(2, 17))
            mlp = _moe(experts, int(rng.integers(1, min(4, experts) + 1)), pick([16, 40, 64, 96]), pick([0.3, 1.0, 7.0]),
                       pick([None, (pick([24, 32, 96]), pick([0.5, 1.5]))]))
        if rng.random() < 0.6:
            layers.append(_latent(int(rng.integers(1, 9)), pick([8, 16, 24, 32, 64]), pick([8, 16, 32, 48]),
                                  pick([16, 24, 64, 128]), pick([16, 32, 40, 64, 96, 128, 256]),
                                  float(rng.uniform(0.1, 0.5)), pick([None, 1, 3, 17, 63, 64, 65, 80, 100]), mlp))
        else:
            layers.append(_gla(int(rng.integers(1, 7)), pick([4, 8, 16, 32, 64, 128]), pick([8, 16, 32, 64]),
                               float(rng.uniform(2.0, 32.0)), pick([4, 8, 16, 32]), mlp))
    return dict(architecture="Fuposun", vocab=int(rng.integers(100, 700)), width=width,
                residual_mult=float(pick([1.0, 0.7, 0.35])), logit_softcap=pick([None, 12.0, 30.0]),
                norm={"eps": pick([1e-5, 1e-6])}, initializer_range=0.07, layers=layers)


@pytest.mark.parametrize("seed", range(30))
def test_configurations_drawn_at_random(tmp_path, seed):
    """Prompts of unequal lengths in one step, then tokens one by one, against the plain logits: float32 sharply for
    every configuration, bfloat16 for every other one.  (A wider sweep of 100 seeds passed but for two bfloat16 cases,
    both at the first token of a sequence in a linear-attention layer: there the state has rank one, o = v (k . q),
    and the norm that follows keeps only the sign of k . q, which rounding can turn when the product is near zero;
    float32 agrees there too.)"""
    from quicknn_b200.engine import Engine, Model
    raw = random_config(seed)
    name = f"R{seed}"
    CONFIGS[name] = (raw, 50 + seed)
    lens, extra = [130, 7, 1, 70], 5
    reqs = prompts(name, [n + extra for n in lens], seed=seed)
    for dtype in (("float32", "bfloat16") if seed % 2 == 0 else ("float32",)):
        folder = make_folder(tmp_path, name, dtype, dtype == "float32", keep_rank=bool(seed % 3))
        plain = FP.PlainFuposun(folder)
        ref = [plain.logits(t) for t in reqs]
        eng = Engine(Model.from_folder(folder, dtype, DEV), max_tokens=1024)
        slots = [eng.new_sequence() for _ in reqs]
        got = eng.step([(s, t[:n]) for s, t, n in zip(slots, reqs, lens)], "all").cpu().numpy()
        at = 0
        for r, n in zip(ref, lens):
            ok, err, tol = close(got[at:at + n], r[:n], dtype)
            assert ok, f"seed {seed} {dtype}: prompt of {n}: error {err:.3g} > {tol:.3g}  ({raw['layers']})"
            at += n
        for t in range(extra):
            got = eng.step([(s, [q[n + t]]) for s, q, n in zip(slots, reqs, lens)], "last").cpu().numpy()
            for i, (r, n) in enumerate(zip(ref, lens)):
                ok, err, tol = close(got[i:i + 1], r[n + t:n + t + 1], dtype)
                assert ok, f"seed {seed} {dtype}: request {i} decoded token {t}: error {err:.3g} > {tol:.3g}"
        for s in slots:
            eng.release(s)
        eng.cache.audit()
