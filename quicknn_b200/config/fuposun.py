"""Fuposun: typed configuration and its layout as parts.

A decoder whose layers are listed one by one in ``config.json``: each entry names its token mixer
(``latent_attention`` or ``gla``) with the mixer's sizes, and its feed-forward (dense, routed experts, or none).

    {"architecture": "Fuposun", "vocab": V, "width": W, "residual_mult": m, "logit_softcap": c, "norm": {"eps": e},
     "layers": [{"type": "latent_attention",
                 "mixer": {"heads", "dim", "vdim", "q_rank", "kv_rank", "scale", "mask": {"size"}},
                 "mlp": {"kind": "dense", "ff"}},
                {"type": "gla", "mixer": {"heads", "dim", "vdim", "tau"},
                 "mlp": {"kind": "moe", "router": {"experts", "top"}, "expert": {"ff", "limit"},
                         "shared": {"ff", "limit"}}}, ...]}

The stream is the normed embedding; every layer is pre-norm with its sublayers' outputs multiplied by
``residual_mult`` before they are added; the head is a matrix of its own behind a final norm, with a softcap.
All norms are RMS norms with a plain weight and the one ``norm.eps``.  The rank of the gla decay's low-rank
projection is not a key of the file: it is the first extent of the layer's ``mix.a1`` tensor
(``sizes_from_shapes``); a config written by this library carries it as ``decay_rank``.

Checkpoint names: ``embed``, ``embed.norm``, ``final.norm``, ``head``; layer i: ``l<i>.norm1``, ``l<i>.norm2``,
``l<i>.mix.<name>`` and ``l<i>.mlp.<name>`` (experts ``e<j>.gate|up|down``, ``router``, ``shared.gate|up|down``).
"""
from __future__ import annotations

import dataclasses
import math
from typing import Any, Dict, List, Mapping, Optional, Tuple

from ..parts.spec import EmbeddingSpec, HeadSpec, LayerSpec, ModelSpec, PartSpec, default_schedule
from .base import Architecture, ModelConfig, as_float, as_int, as_opt_float, register_architecture

MIXER_KINDS = ("latent_attention", "gla")
MLP_KINDS = ("dense", "moe")
MAX_POSITIONS = 1 << 20          # the design has no positions; this only bounds a cache's longest sequence


def _obj(v: Any, what: str) -> Dict[str, Any]:
    if not isinstance(v, dict):
        raise TypeError(f"{what} must be an object, got {v!r}")
    return v


@dataclasses.dataclass(frozen=True)
class MlpConfig:
    kind: str
    ff: int = 0                      # dense: inner width
    experts: int = 0                 # moe
    top: int = 0
    expert_ff: int = 0
    expert_limit: float = 0.0
    shared_ff: Optional[int] = None  # None: no shared expert
    shared_limit: float = 0.0

    @classmethod
    def parse(cls, v: Any) -> Optional["MlpConfig"]:
        if v is None:
            return None
        v = _obj(v, "mlp")
        kind = v.get("kind")
        if kind == "dense":
            return cls(kind="dense", ff=as_int(v.get("ff")))
        if kind == "moe":
            router, expert = _obj(v.get("router"), "mlp.router"), _obj(v.get("expert"), "mlp.expert")
            shared = v.get("shared")
            return cls(kind="moe", experts=as_int(router.get("experts")), top=as_int(router.get("top")),
                       expert_ff=as_int(expert.get("ff")), expert_limit=as_float(expert.get("limit")),
                       shared_ff=None if shared is None else as_int(_obj(shared, "mlp.shared").get("ff")),
                       shared_limit=0.0 if shared is None else as_float(shared.get("limit")))
        raise ValueError(f"mlp.kind must be one of {MLP_KINDS} (got {kind!r})")

    def to_dict(self) -> Dict[str, Any]:
        if self.kind == "dense":
            return {"kind": "dense", "ff": self.ff}
        out: Dict[str, Any] = {"kind": "moe", "router": {"experts": self.experts, "top": self.top},
                               "expert": {"ff": self.expert_ff, "limit": self.expert_limit}}
        if self.shared_ff is not None:
            out["shared"] = {"ff": self.shared_ff, "limit": self.shared_limit}
        return out

    def problems(self, where: str) -> List[str]:
        p: List[str] = []
        if self.kind == "dense":
            if self.ff < 1:
                p.append(f"{where}.ff must be >= 1 (got {self.ff})")
            return p
        if self.experts < 1 or not (1 <= self.top <= self.experts):
            p.append(f"{where}.router: top {self.top} of {self.experts} experts")
        if self.expert_ff < 1 or (self.shared_ff is not None and self.shared_ff < 1):
            p.append(f"{where}: expert widths must be >= 1")
        if not self.expert_limit > 0 or (self.shared_ff is not None and not self.shared_limit > 0):
            p.append(f"{where}: limits must be > 0")
        return p


@dataclasses.dataclass(frozen=True)
class LayerConfig:
    type: str
    heads: int
    dim: int
    vdim: int
    mlp: Optional[MlpConfig]
    q_rank: int = 0                  # latent_attention
    kv_rank: int = 0
    scale: float = 0.0
    window: Optional[int] = None     # mask.size; None: every earlier position
    tau: float = 0.0                 # gla
    decay_rank: int = 0

    @classmethod
    def parse(cls, v: Any) -> "LayerConfig":
        v = _obj(v, "a layer")
        kind = v.get("type")
        if kind not in MIXER_KINDS:
            raise ValueError(f"layer type must be one of {MIXER_KINDS} (got {kind!r})")
        m = _obj(v.get("mixer"), "mixer")
        common = dict(type=kind, heads=as_int(m.get("heads")), dim=as_int(m.get("dim")), vdim=as_int(m.get("vdim")),
                      mlp=MlpConfig.parse(v.get("mlp")))
        if kind == "latent_attention":
            mask = m.get("mask")
            size = None if mask is None else _obj(mask, "mixer.mask").get("size")
            return cls(q_rank=as_int(m.get("q_rank")), kv_rank=as_int(m.get("kv_rank")), scale=as_float(m.get("scale")),
                       window=None if size is None else as_int(size), **common)
        if m.get("decay_rank") is None:
            raise ValueError("a gla mixer's decay_rank is neither in the config nor given by a checkpoint's 'mix.a1'")
        return cls(tau=as_float(m.get("tau")), decay_rank=as_int(m.get("decay_rank")), **common)

    def to_dict(self) -> Dict[str, Any]:
        m: Dict[str, Any] = {"heads": self.heads, "dim": self.dim, "vdim": self.vdim}
        if self.type == "latent_attention":
            m.update(q_rank=self.q_rank, kv_rank=self.kv_rank, scale=self.scale)
            if self.window is not None:
                m["mask"] = {"size": self.window}
        else:
            m.update(tau=self.tau, decay_rank=self.decay_rank)
        return {"type": self.type, "mixer": m, "mlp": None if self.mlp is None else self.mlp.to_dict()}

    def problems(self, where: str) -> List[str]:
        p: List[str] = []
        for name in ("heads", "dim", "vdim"):
            if getattr(self, name) < 1:
                p.append(f"{where}.mixer.{name} must be >= 1 (got {getattr(self, name)})")
        if self.type == "latent_attention":
            if self.q_rank < 1 or self.kv_rank < 1:
                p.append(f"{where}.mixer: q_rank and kv_rank must be >= 1")
            if not (self.scale > 0 and math.isfinite(self.scale)):
                p.append(f"{where}.mixer.scale must be > 0 (got {self.scale})")
            if self.window is not None and self.window < 1:
                p.append(f"{where}.mixer.mask.size must be >= 1 (got {self.window})")
        else:
            if not self.tau > 0:
                p.append(f"{where}.mixer.tau must be > 0 (got {self.tau})")
            if self.decay_rank < 1:
                p.append(f"{where}.mixer.decay_rank must be >= 1 (got {self.decay_rank})")
            if self.dim > 256:
                p.append(f"{where}.mixer.dim must be at most 256 (got {self.dim})")
        if self.mlp is not None:
            p.extend(self.mlp.problems(where + ".mlp"))
        return p


def _layers(v: Any) -> Tuple[LayerConfig, ...]:
    if not isinstance(v, (list, tuple)) or not v:
        raise TypeError("layers must be a list with at least one entry")
    return tuple(LayerConfig.parse(x) for x in v)


def _eps(v: Any) -> float:
    return as_float(_obj(v, "norm").get("eps"))


def _req(conv, key=None):
    md = {"convert": conv, "required": True}
    if key:
        md["key"] = key
    return dataclasses.field(default=None, metadata=md)


@dataclasses.dataclass(frozen=True)
class FuposunConfig(ModelConfig):
    vocab: int = _req(as_int)
    width: int = _req(as_int)
    layers: Tuple[LayerConfig, ...] = _req(_layers)
    norm_eps: float = _req(_eps, key="norm")
    residual_mult: float = dataclasses.field(default=1.0, metadata={"convert": as_float})
    logit_softcap: Optional[float] = dataclasses.field(default=None, metadata={"convert": as_opt_float})
    architecture: str = dataclasses.field(default="Fuposun", metadata={"convert": str})
    initializer_range: float = dataclasses.field(default=0.02, metadata={"convert": as_float})

    @classmethod
    def architecture_names(cls) -> Tuple[str, ...]:
        return ("Fuposun",)

    def to_dict(self) -> Dict[str, Any]:
        return {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
                "residual_mult": self.residual_mult, "logit_softcap": self.logit_softcap,
                "norm": {"eps": self.norm_eps}, "layers": [l.to_dict() for l in self.layers],
                "initializer_range": self.initializer_range}

    def problems(self) -> List[str]:
        p: List[str] = []
        if self.vocab < 1 or self.width < 1:
            p.append(f"vocab and width must be >= 1 (got {self.vocab}, {self.width})")
        if not self.norm_eps > 0:
            p.append(f"norm.eps must be > 0 (got {self.norm_eps})")
        if not math.isfinite(self.residual_mult):
            p.append(f"residual_mult must be finite (got {self.residual_mult})")
        if self.logit_softcap is not None and not (self.logit_softcap > 0 and math.isfinite(self.logit_softcap)):
            p.append(f"logit_softcap must be > 0 or null (got {self.logit_softcap})")
        if not (1 <= len(self.layers) <= 1024):
            p.append(f"between 1 and 1024 layers (got {len(self.layers)})")
        for i, layer in enumerate(self.layers):
            p.extend(layer.problems(f"layers[{i}]"))
        if not self.initializer_range > 0:
            p.append(f"initializer_range must be > 0 (got {self.initializer_range})")
        return p


def fuposun_sizes_from_shapes(raw: Dict[str, Any], shapes: Mapping[str, Tuple[int, ...]]) -> Dict[str, Any]:
    """Fill in what the file leaves to the tensors: a gla layer's ``decay_rank`` is the first extent of its
    ``mix.a1``.  The raw config is copied, not changed."""
    layers = raw.get("layers")
    if not isinstance(layers, list):
        return raw
    out = dict(raw)
    out["layers"] = []
    for i, layer in enumerate(layers):
        if isinstance(layer, dict) and layer.get("type") == "gla" and isinstance(layer.get("mixer"), dict) \
                and layer["mixer"].get("decay_rank") is None and f"l{i}.mix.a1" in shapes:
            layer = dict(layer)
            layer["mixer"] = dict(layer["mixer"], decay_rank=int(shapes[f"l{i}.mix.a1"][0]))
        out["layers"].append(layer)
    return out


def _mlp_spec(cfg: FuposunConfig, mlp: MlpConfig, pre: str) -> Tuple[PartSpec, Dict[str, str]]:
    W = cfg.width
    if mlp.kind == "dense":
        names = {f"ff.{n}_proj": f"{pre}mlp.{n}" for n in ("gate", "up", "down")}
        return PartSpec("gated_mlp", {"hidden_size": W, "intermediate_size": mlp.ff, "activation": "silu"}), names
    shared = None
    names = {"ff.router": f"{pre}mlp.router"}
    for e in range(mlp.experts):
        for n in ("gate", "up", "down"):
            names[f"ff.experts.{e}.{n}_proj"] = f"{pre}mlp.e{e}.{n}"
    if mlp.shared_ff is not None:
        shared = PartSpec("clamped_mlp", {"hidden_size": W, "intermediate_size": mlp.shared_ff, "limit": mlp.shared_limit})
        for n in ("gate", "up", "down"):
            names[f"ff.shared.{n}_proj"] = f"{pre}mlp.shared.{n}"
    spec = PartSpec("routed_experts", {
        "hidden_size": W, "experts": mlp.experts, "top": mlp.top, "intermediate_size": mlp.expert_ff,
        "limit": mlp.expert_limit, "score": "sigmoid", "renormalize": False, "weight_on": "input", "shared": shared})
    return spec, names


def fuposun_spec(cfg: FuposunConfig) -> ModelSpec:
    W = cfg.width
    norm = PartSpec("rmsnorm", {"size": W, "eps": cfg.norm_eps, "unit_offset": False})
    layers, optional = [], []
    for i, lc in enumerate(cfg.layers):
        pre = f"l{i}."
        tensors = {"norms.pre_mixer.weight": pre + "norm1"}
        if lc.type == "latent_attention":
            mixer = PartSpec("latent_attention", {
                "hidden_size": W, "n_heads": lc.heads, "dim": lc.dim, "vdim": lc.vdim, "q_rank": lc.q_rank,
                "kv_rank": lc.kv_rank, "scale": lc.scale, "window": lc.window, "eps": cfg.norm_eps})
            for local, name in (("dq", "dq"), ("dq_norm", "dq.norm"), ("uq", "uq"), ("dkv", "dkv"),
                                ("dkv_norm", "dkv.norm"), ("uk", "uk"), ("uv", "uv"), ("gate", "g"), ("o", "o")):
                tensors["mixer." + local] = f"{pre}mix.{name}"
        else:
            mixer = PartSpec("gla", {"hidden_size": W, "n_heads": lc.heads, "dim": lc.dim, "vdim": lc.vdim,
                                     "tau": lc.tau, "decay_rank": lc.decay_rank, "eps": cfg.norm_eps})
            for local, name in (("q", "q"), ("k", "k"), ("v", "v"), ("gate", "g"), ("o", "o"), ("norm", "norm"),
                                ("a1", "a1"), ("a2", "a2"), ("a2_bias", "a2.b")):
                tensors["mixer." + local] = f"{pre}mix.{name}"
        ff = None
        norms = {"pre_mixer": norm}
        if lc.mlp is not None:
            ff, names = _mlp_spec(cfg, lc.mlp, pre)
            tensors.update(names)
            tensors["norms.pre_ff.weight"] = pre + "norm2"
            norms["pre_ff"] = norm
        else:
            optional.append(pre + "norm2")          # a layer without a feed-forward may still carry its norm
        layers.append(LayerSpec(block=PartSpec("prenorm", {"residual_mult": cfg.residual_mult}), mixer=mixer,
                                feed_forward=ff, norms=norms, tensors=tensors))
    return ModelSpec(
        name="Fuposun", hidden_size=W,
        embedding=EmbeddingSpec(cfg.vocab, W, 1.0, "embed", norm=norm, norm_tensor="embed.norm"),
        layers=tuple(layers), schedule=default_schedule(len(layers)),
        head=HeadSpec(cfg.vocab, W, tied=False, tensor="head", softcap=cfg.logit_softcap, norm=norm,
                      norm_tensor="final.norm"),
        max_positions=MAX_POSITIONS, stop_ids=(), init_std=cfg.initializer_range, init_norm_std=0.1,
        optional_tensors=tuple(optional))


FUPOSUN = register_architecture(Architecture(
    name="Fuposun", config_cls=FuposunConfig, build_spec=fuposun_spec, aliases=("fuposun",),
    sizes_from_shapes=fuposun_sizes_from_shapes))
