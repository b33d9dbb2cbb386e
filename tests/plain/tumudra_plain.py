"""Plain, slow Tumudra: whole sequences, no cache, one function per mechanism, NumPy only.

A decoder whose ``config.json`` lists its layers.  A layer adds the *normed output* of its
sublayers to the stream, and the sublayers read the stream itself:

    x <- x + LN1(mixer(x));   x <- x + LN2(ff(x))          LN: layer norm with a weight, no bias

Three kinds of mixer:

* ``attention``: grouped-query softmax attention with biases on all four products, an RMS norm per
  head on queries and keys before a half-split rotation of the first ``rot.dims`` columns, a key
  size that may differ from the value size, and optionally the keys and values of an earlier layer
  (``kv_from``) instead of its own;
* ``parallel``: two branches on the same input whose outputs are each RMS-normed over the width and
  averaged.  Left: sliding-window attention without biases, interleaved rotation with the
  frequencies rescaled by wavelength.  Right: a matrix memory with exponential input gate,
  sigmoid forget gate (both soft-capped), a running maximum that keeps the exponentials bounded and
  a normaliser vector, read out as S^T q / (max(|n.q|, e^-m) + 1e-6);
* ``retention``: a matrix memory with a fixed decay per head and no denominator.

The feed-forward is W_down relu(W_up h)^2.  It shares no code with the library: its own
safetensors reader, its own reading of ``config.json``, one whole sequence at a time, float64.
"""
from __future__ import annotations

import json
import math
import os
import struct
from typing import Dict, List, Optional, Sequence

import numpy as np

F = np.float64


# ---- files ---------------------------------------------------------------------

def read_safetensors(path: str) -> Dict[str, np.ndarray]:
    with open(path, "rb") as fh:
        (n,) = struct.unpack("<Q", fh.read(8))
        header = json.loads(fh.read(n).decode("utf-8"))
        data = fh.read()
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        b, e = info["data_offsets"]
        raw = data[b:e]
        if info["dtype"] == "BF16":
            arr = (np.frombuffer(raw, dtype="<u2").astype(np.uint32) << 16).view(np.float32)
        elif info["dtype"] == "F32":
            arr = np.frombuffer(raw, dtype="<f4")
        else:
            raise ValueError(f"plain reader: dtype {info['dtype']} of {name}")
        out[name] = arr.reshape(info["shape"]).astype(F)
    return out


# ---- small pieces ------------------------------------------------------------------

def rms_unit(x: np.ndarray, eps: float) -> np.ndarray:
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / np.sqrt((x * x).mean(axis=-1, keepdims=True) + eps)


def layer_norm(x: np.ndarray, w: np.ndarray, eps: float) -> np.ndarray:
    d = x - x.mean(axis=-1, keepdims=True)
    return d / np.sqrt((d * d).mean(axis=-1, keepdims=True) + eps) * w


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def log_sigmoid(z):
    return -np.logaddexp(0.0, -z)


def rotary_frequencies(rot: dict) -> np.ndarray:
    """f_i = base^(-2i/dims), i < dims/2; with ``scaling`` the long wavelengths are slowed down:
    wavelength below original/high: kept; above original/low: divided by factor; between: blended."""
    dims = int(rot["dims"])
    f = float(rot["base"]) ** (-2.0 * np.arange(dims // 2, dtype=F) / dims)
    sc = rot.get("scaling")
    if sc:
        factor, lo, hi, orig = float(sc["factor"]), float(sc["low"]), float(sc["high"]), float(sc["original"])
        out = f.copy()
        for i, fi in enumerate(f):
            wave = 2.0 * math.pi / fi
            if wave < orig / hi:
                continue
            if wave > orig / lo:
                out[i] = fi / factor
            else:
                s = (orig / wave - lo) / (hi - lo)
                out[i] = (1.0 - s) * fi / factor + s * fi
        f = out
    return f


def rotate(x: np.ndarray, rot: dict, interleaved: bool, first_position: int = 0) -> np.ndarray:
    """x: [n, heads, dim]; rotates the first rot.dims columns of every head by position * f_i.
    Half-split: column i pairs with i + dims/2.  Interleaved: column 2i pairs with 2i + 1."""
    dims = int(rot["dims"])
    if dims == 0:
        return x
    n = x.shape[0]
    # the design forms positions and angles in 32-bit: frequency and product are rounded to float32
    pos = (np.arange(n) + first_position).astype(np.float32)
    ang = (pos[:, None] * rotary_frequencies(rot).astype(np.float32)[None, :]).astype(F)          # [n, dims/2]
    c, s = np.cos(ang)[:, None, :], np.sin(ang)[:, None, :]
    out = x.copy()
    if interleaved:
        u, v = x[..., 0:dims:2], x[..., 1:dims:2]
        out[..., 0:dims:2] = u * c - v * s
        out[..., 1:dims:2] = v * c + u * s
    else:
        u, v = x[..., :dims // 2], x[..., dims // 2:dims]
        out[..., :dims // 2] = u * c - v * s
        out[..., dims // 2:dims] = v * c + u * s
    return out


def visible(n: int, size: Optional[int]) -> np.ndarray:
    d = np.arange(n)[:, None] - np.arange(n)[None, :]
    return (d >= 0) if size is None else ((d >= 0) & (d < size))


def softmax_attention(q, k, v, scale: float, size: Optional[int]) -> np.ndarray:
    """q: [n, H, d]; k: [n, G, d]; v: [n, G, dv]; query head a reads kv head a // (H/G)."""
    n, H, _ = q.shape
    G = k.shape[1]
    vis = visible(n, size)
    out = np.zeros((n, H, v.shape[2]), dtype=F)
    for a in range(H):
        g = a // (H // G)
        s = np.where(vis, (q[:, a] @ k[:, g].T) * scale, -np.inf)
        e = np.exp(s - s.max(axis=-1, keepdims=True))
        out[:, a] = (e / e.sum(axis=-1, keepdims=True)) @ v[:, g]
    return out


# ---- mixers --------------------------------------------------------------------------

def attention_keys_values(h, w, m, eps, interleaved):
    n = h.shape[0]
    G, d, dv = int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    k = h @ w["k"].T + (w["k.b"] if "k.b" in w else 0.0)
    v = h @ w["v"].T + (w["v.b"] if "v.b" in w else 0.0)
    k = rms_unit(k.reshape(n, G, d), eps) * w["k.norm"]
    return rotate(k, m["rot"], interleaved), v.reshape(n, G, dv)


def attention(h, w, m, eps, interleaved=False, kv=None):
    """``kv``: (keys, values) of another layer, used as they are; None: this layer's own.
    Returns (output, (keys, values))."""
    n = h.shape[0]
    H, d = int(m["heads"]), int(m["dim"])
    q = h @ w["q"].T + (w["q.b"] if "q.b" in w else 0.0)
    q = rotate(rms_unit(q.reshape(n, H, d), eps) * w["q.norm"], m["rot"], interleaved)
    if kv is None:
        kv = attention_keys_values(h, w, m, eps, interleaved)
    size = (m.get("mask") or {}).get("size")
    o = softmax_attention(q, kv[0], kv[1], float(m["scale"]), None if size is None else int(size))
    y = o.reshape(n, -1) @ w["o"].T + (w["o.b"] if "o.b" in w else 0.0)
    return y, kv


def matrix_memory(h, w, m, eps):
    """The right branch of a parallel mixer."""
    n = h.shape[0]
    H, d, dv, cap = int(m["heads"]), int(m["dim"]), int(m["vdim"]), float(m["gate_cap"])
    q = (h @ w["q"].T).reshape(n, H, d) * d ** -0.5
    k = (h @ w["k"].T).reshape(n, H, d)
    v = (h @ w["v"].T).reshape(n, H, dv)
    gi = cap * np.tanh((h @ w["i"].T + w["i.b"]) / cap)                         # log input gate   [n, H]
    gf = log_sigmoid(cap * np.tanh((h @ w["f"].T + w["f.b"]) / cap))            # log forget gate
    out = np.zeros((n, H, dv), dtype=F)
    for a in range(H):
        S, nv, mx = np.zeros((d, dv), dtype=F), np.zeros(d, dtype=F), 0.0
        for t in range(n):
            new = max(gf[t, a] + mx, gi[t, a])
            keep, take = math.exp(gf[t, a] + mx - new), math.exp(gi[t, a] - new)
            S = keep * S + take * np.outer(k[t, a], v[t, a])
            nv = keep * nv + take * k[t, a]
            mx = new
            out[t, a] = (S.T @ q[t, a]) / (max(abs(float(nv @ q[t, a])), math.exp(-mx)) + 1e-6)
    out = rms_unit(out, eps).reshape(n, H * dv) * w["norm"]
    return (out * sigmoid(h @ w["g"].T)) @ w["o"].T


def parallel(h, w, m, eps):
    left = {k[5:]: v for k, v in w.items() if k.startswith("left.") and k != "left.out"}
    right = {k[6:]: v for k, v in w.items() if k.startswith("right.") and k != "right.out"}
    a, _ = attention(h, left, m["left"], eps, interleaved=True)
    b = matrix_memory(h, right, m["right"], eps)
    return 0.5 * (rms_unit(a, eps) * w["left.out"] + rms_unit(b, eps) * w["right.out"])


def retention(h, w, m, eps):
    n = h.shape[0]
    H, d, dv = int(m["heads"]), int(m["dim"]), int(m["vdim"])
    q = rotate((h @ w["q"].T).reshape(n, H, d), m["rot"], False)
    k = rotate((h @ w["k"].T).reshape(n, H, d), m["rot"], False) * d ** -0.5
    v = (h @ w["v"].T).reshape(n, H, dv)
    out = np.zeros((n, H, dv), dtype=F)
    for a in range(H):
        S = np.zeros((d, dv), dtype=F)
        for t in range(n):
            S = float(m["decay"][a]) * S + np.outer(k[t, a], v[t, a])
            out[t, a] = S.T @ q[t, a]
    g = h @ w["g"].T
    return (rms_unit(out, eps).reshape(n, H * dv) * (g * sigmoid(g))) @ w["o"].T


def feed_forward(h, w):
    return (np.maximum(h @ w["up"].T, 0.0) ** 2) @ w["down"].T


# ---- the model ---------------------------------------------------------------------

class PlainTumudra:
    def __init__(self, model_dir: str):
        with open(os.path.join(model_dir, "config.json"), "r", encoding="utf-8") as fh:
            self.cfg = json.load(fh)
        self.w = read_safetensors(os.path.join(model_dir, "model.safetensors"))
        self.eps = float(self.cfg["norm"]["eps"])

    def sub(self, prefix: str) -> Dict[str, np.ndarray]:
        return {k[len(prefix):]: v for k, v in self.w.items() if k.startswith(prefix)}

    def residual_stream(self, ids: Sequence[int]) -> List[np.ndarray]:
        """The stream after the embedding and after every layer."""
        cfg, w, eps = self.cfg, self.w, self.eps
        x = w["embed"][np.asarray(ids, dtype=np.int64)] * float(cfg["embedding"]["scale"])
        streams, kept = [x], {}
        for i, layer in enumerate(cfg["layers"]):
            mix, m = self.sub(f"l{i}.mix."), layer["mixer"]
            if layer["type"] == "attention":
                src = m.get("kv_from")
                y, kept[i] = attention(x, mix, m, eps, kv=None if src is None else kept[int(src)])
            elif layer["type"] == "parallel":
                y = parallel(x, mix, m, eps)
            elif layer["type"] == "retention":
                y = retention(x, mix, m, eps)
            else:
                raise ValueError(f"plain: mixer {layer['type']!r}")
            x = x + layer_norm(y, w[f"l{i}.norm1"], eps)
            if layer.get("mlp"):
                x = x + layer_norm(feed_forward(x, self.sub(f"l{i}.mlp.")), w[f"l{i}.norm2"], eps)
            streams.append(x)
        return streams

    def logits(self, ids: Sequence[int]) -> np.ndarray:
        x = self.residual_stream(ids)[-1]
        return layer_norm(x, self.w["final.norm"], self.eps) @ self.w["head"].T

    def greedy(self, prompt: Sequence[int], n: int) -> List[int]:
        seq, out = list(prompt), []
        for _ in range(n):
            t = int(np.argmax(self.logits(seq)[-1]))
            out.append(t)
            seq.append(t)
        return out
