"""Plain, slow Fuposun: whole sequences, no cache, one function per mechanism, NumPy only.

A decoder that mixes two kinds of token mixer, layer by layer, around a pre-norm residual
stream whose sublayer outputs are multiplied by a constant before they are added:

* latent attention: queries and keys/values pass through low-rank latents with an RMS norm
  each; keys and values of every head are products of the one latent row per token; no
  positions; a sliding window; softmax; a sigmoid gate per head; an output product;
* gated linear attention: a matrix state per head that decays per key channel,
  S_t = diag(a_t) S_{t-1} + k_t v_t^T, read with the scaled query; RMS norm per head,
  a SiLU gate, an output product;

and two kinds of feed-forward: a dense SiLU-gated one, and routed experts (sigmoid scores,
the best ``top`` experts, the score multiplies the expert's *input*) beside a shared expert,
with a clamped activation g * sigmoid(1.702 g) * (u + 1).

It shares no code with the library: its own safetensors reader, its own reading of
``config.json``, one whole sequence at a time, float64 arithmetic.
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


# ---- mechanisms ------------------------------------------------------------------

def rms_norm(x: np.ndarray, w: Optional[np.ndarray], eps: float) -> np.ndarray:
    """x / sqrt(mean(x^2) + eps) over the last axis, times w (a plain weight) when given."""
    y = x / np.sqrt((x * x).mean(axis=-1, keepdims=True) + eps)
    return y if w is None else y * w


def sigmoid(z: np.ndarray) -> np.ndarray:
    return 1.0 / (1.0 + np.exp(-z))


def silu(z: np.ndarray) -> np.ndarray:
    return z * sigmoid(z)


def softmax_rows(s: np.ndarray, visible: np.ndarray) -> np.ndarray:
    s = np.where(visible, s, -np.inf)
    s = s - s.max(axis=-1, keepdims=True)
    e = np.where(visible, np.exp(s), 0.0)
    return e / e.sum(axis=-1, keepdims=True)


def window_mask(n: int, size: Optional[int]) -> np.ndarray:
    """visible[i, j]: 0 <= i - j < size (every earlier position when size is None)."""
    i = np.arange(n)[:, None]
    j = np.arange(n)[None, :]
    d = i - j
    return (d >= 0) if size is None else ((d >= 0) & (d < size))


def latent_attention(h: np.ndarray, w: Dict[str, np.ndarray], m: dict, eps: float) -> np.ndarray:
    """h: [n, width].  ``w`` holds the mixer's tensors by their short names."""
    H, dim, vdim = int(m["heads"]), int(m["dim"]), int(m["vdim"])
    n = h.shape[0]
    cq = rms_norm(h @ w["dq"].T, w["dq.norm"], eps)
    q = (cq @ w["uq"].T).reshape(n, H, dim)
    c = rms_norm(h @ w["dkv"].T, w["dkv.norm"], eps)
    k = (c @ w["uk"].T).reshape(n, H, dim)
    v = (c @ w["uv"].T).reshape(n, H, vdim)
    gate = sigmoid(h @ w["g"].T)                                   # [n, H]
    size = (m.get("mask") or {}).get("size")
    vis = window_mask(n, None if size is None else int(size))
    out = np.zeros((n, H, vdim), dtype=F)
    for a in range(H):
        s = (q[:, a] @ k[:, a].T) * float(m["scale"])
        out[:, a] = softmax_rows(s, vis) @ v[:, a]
        out[:, a] *= gate[:, a:a + 1]
    return out.reshape(n, H * vdim) @ w["o"].T


def gla(h: np.ndarray, w: Dict[str, np.ndarray], m: dict, eps: float) -> np.ndarray:
    H, dim, vdim, tau = int(m["heads"]), int(m["dim"]), int(m["vdim"]), float(m["tau"])
    n = h.shape[0]
    q = (h @ w["q"].T).reshape(n, H, dim) * dim ** -0.5
    k = (h @ w["k"].T).reshape(n, H, dim)
    v = (h @ w["v"].T).reshape(n, H, vdim)
    z = (h @ w["a1"].T) @ w["a2"].T + w["a2.b"]
    alpha = (sigmoid(z) ** (1.0 / tau)).reshape(n, H, dim)
    out = np.zeros((n, H, vdim), dtype=F)
    for a in range(H):
        S = np.zeros((dim, vdim), dtype=F)
        for t in range(n):
            S = alpha[t, a][:, None] * S + np.outer(k[t, a], v[t, a])
            out[t, a] = S.T @ q[t, a]
    out = rms_norm(out, w["norm"], eps).reshape(n, H * vdim)
    return (out * silu(h @ w["g"].T)) @ w["o"].T


def dense_ff(h: np.ndarray, w: Dict[str, np.ndarray]) -> np.ndarray:
    return (silu(h @ w["gate"].T) * (h @ w["up"].T)) @ w["down"].T


def clamped_expert(h: np.ndarray, gate: np.ndarray, up: np.ndarray, down: np.ndarray, limit: float) -> np.ndarray:
    g = np.minimum(h @ gate.T, limit)
    u = np.clip(h @ up.T, -limit, limit)
    return (g * sigmoid(1.702 * g) * (u + 1.0)) @ down.T


def routed_ff(h: np.ndarray, w: Dict[str, np.ndarray], mlp: dict) -> np.ndarray:
    E, top = int(mlp["router"]["experts"]), int(mlp["router"]["top"])
    limit = float(mlp["expert"]["limit"])
    s = sigmoid(h @ w["router"].T)                                  # [n, E]
    out = np.zeros((h.shape[0], w["e0.down"].shape[0]), dtype=F)
    for t in range(h.shape[0]):
        order = sorted(range(E), key=lambda e: (-s[t, e], e))[:top]
        for e in order:
            out[t] += clamped_expert(s[t, e] * h[t:t + 1], w[f"e{e}.gate"], w[f"e{e}.up"], w[f"e{e}.down"], limit)[0]
    if mlp.get("shared"):
        out += clamped_expert(h, w["shared.gate"], w["shared.up"], w["shared.down"], float(mlp["shared"]["limit"]))
    return out


def softcap(x: np.ndarray, cap: Optional[float]) -> np.ndarray:
    return x if not cap else cap * np.tanh(x / cap)


# ---- the model ---------------------------------------------------------------------

class PlainFuposun:
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
        m = float(cfg["residual_mult"])
        x = rms_norm(w["embed"][np.asarray(ids, dtype=np.int64)], w["embed.norm"], eps)
        streams = [x]
        for i, layer in enumerate(cfg["layers"]):
            h = rms_norm(x, w[f"l{i}.norm1"], eps)
            mix = self.sub(f"l{i}.mix.")
            if layer["type"] == "latent_attention":
                y = latent_attention(h, mix, layer["mixer"], eps)
            elif layer["type"] == "gla":
                y = gla(h, mix, layer["mixer"], eps)
            else:
                raise ValueError(f"plain: mixer {layer['type']!r}")
            x = x + m * y
            mlp = layer.get("mlp")
            if mlp:
                h = rms_norm(x, w[f"l{i}.norm2"], eps)
                ff = self.sub(f"l{i}.mlp.")
                y = dense_ff(h, ff) if mlp["kind"] == "dense" else routed_ff(h, ff, mlp)
                x = x + m * y
            streams.append(x)
        return streams

    def logits(self, ids: Sequence[int]) -> np.ndarray:
        x = self.residual_stream(ids)[-1]
        z = rms_norm(x, self.w["final.norm"], self.eps) @ self.w["head"].T
        return softcap(z, self.cfg.get("logit_softcap"))

    def greedy(self, prompt: Sequence[int], n: int) -> List[int]:
        seq, out = list(prompt), []
        for _ in range(n):
            t = int(np.argmax(self.logits(seq)[-1]))
            out.append(t)
            seq.append(t)
        return out
