"""Tumudra: typed configuration and its layout as parts.

A decoder whose layers are listed one by one in ``config.json``; a layer adds the normed output of its sublayers to
the stream (layer norms with a weight and no bias), and the sublayers read the stream itself.

    {"architecture": "Tumudra", "vocab": V, "width": W, "embedding": {"scale": s}, "norm": {"eps": e},
     "layers": [
       {"type": "attention",
        "mixer": {"heads", "kv_heads", "dim", "vdim", "scale", "rot": {"base", "dims"}, "kv_from": j (optional)},
        "mlp": {"kind": "dense", "ff"}},
       {"type": "parallel",
        "mixer": {"left": {"heads", "kv_heads", "dim", "vdim", "scale", "mask": {"size"},
                           "rot": {"base", "dims", "scaling": {"factor", "low", "high", "original"}}},
                  "right": {"heads", "dim", "vdim", "gate_cap"}},
        "mlp": ...},
       {"type": "retention", "mixer": {"heads", "dim", "vdim", "decay": [per head], "rot": {"base", "dims"}},
        "mlp": null}]}

``attention``: biases on all four products, an RMS norm per head on queries and keys, a half-split rotation, every
earlier position visible; with ``kv_from`` the layer has no keys and values and reads those of layer j.
``parallel``: sliding-window attention without biases and with an interleaved rotation (left) beside an mLSTM matrix
memory (right); the two outputs are RMS-normed over the width and averaged.  ``retention``: a matrix memory with a
fixed decay per head.  The feed-forward is down(relu(up(x))^2).  The head is a matrix of its own behind a final layer
norm.  ``mask``, ``scaling`` and ``kv_from`` are read wherever a softmax attention stands, so a file may give any of
them to either kind.

Checkpoint names: ``embed``, ``final.norm``, ``head``; layer i: ``l<i>.norm1``, ``l<i>.norm2``, ``l<i>.mix.<name>``
(``q k v o`` with ``.b`` for biases and ``q.norm k.norm``; ``g``; ``i f`` with ``.b``; ``norm``; under ``left.`` /
``right.`` in a parallel mixer, whose branch weights are ``left.out`` / ``right.out``), ``l<i>.mlp.up|down``.
"""
from __future__ import annotations

import dataclasses
import math
from typing import Any, Dict, List, Optional, Tuple

from ..parts.spec import EmbeddingSpec, HeadSpec, LayerSpec, ModelSpec, PartSpec, ScheduleEntry
from .base import Architecture, ModelConfig, as_float, as_int, register_architecture

LAYER_TYPES = ("attention", "parallel", "retention")
MAX_POSITIONS = 1 << 20          # rotations have no table; this only bounds a cache's longest sequence


def _obj(v: Any, what: str) -> Dict[str, Any]:
    if not isinstance(v, dict):
        raise TypeError(f"{what} must be an object, got {v!r}")
    return v


@dataclasses.dataclass(frozen=True)
class RotaryConfig:
    base: float
    dims: int
    scaling: Optional[Tuple[float, float, float, float]] = None      # factor, low, high, original

    @classmethod
    def parse(cls, v: Any, where: str) -> "RotaryConfig":
        v = _obj(v, where)
        sc = v.get("scaling")
        scaling = None
        if sc is not None:
            sc = _obj(sc, where + ".scaling")
            scaling = tuple(as_float(sc.get(k)) for k in ("factor", "low", "high", "original"))
        return cls(base=as_float(v.get("base")), dims=as_int(v.get("dims")), scaling=scaling)

    def to_dict(self) -> Dict[str, Any]:
        out: Dict[str, Any] = {"base": self.base, "dims": self.dims}
        if self.scaling is not None:
            out["scaling"] = dict(zip(("factor", "low", "high", "original"), self.scaling))
        return out

    def problems(self, where: str, dim: int) -> List[str]:
        p: List[str] = []
        if self.dims < 0 or self.dims % 2 or self.dims > dim:
            p.append(f"{where}.dims must be even and between 0 and dim {dim} (got {self.dims})")
        if not (self.base > 0 and math.isfinite(self.base)):
            p.append(f"{where}.base must be > 0 (got {self.base})")
        if self.scaling is not None:
            factor, low, high, original = self.scaling
            if not (factor > 0 and original > 0 and high > low >= 0):
                p.append(f"{where}.scaling: factor and original > 0, high > low >= 0 (got {self.scaling})")
        return p

    def part(self, head_dim: int, layout: str) -> PartSpec:
        params: Dict[str, Any] = {"head_dim": head_dim, "theta": self.base, "rotary_dim": self.dims, "layout": layout}
        if self.scaling is not None:
            params["scaling"] = dict(zip(("factor", "low", "high", "original"), self.scaling))
        return PartSpec("rotary", params)


@dataclasses.dataclass(frozen=True)
class SoftmaxConfig:
    """A softmax attention: the ``attention`` mixer, or the left branch of ``parallel``."""

    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    rot: RotaryConfig
    window: Optional[int] = None
    kv_from: Optional[int] = None

    @classmethod
    def parse(cls, m: Dict[str, Any], where: str) -> "SoftmaxConfig":
        mask = m.get("mask")
        size = None if mask is None else _obj(mask, where + ".mask").get("size")
        src = m.get("kv_from")
        return cls(heads=as_int(m.get("heads")), kv_heads=as_int(m.get("kv_heads")), dim=as_int(m.get("dim")),
                   vdim=as_int(m.get("vdim")), scale=as_float(m.get("scale")),
                   rot=RotaryConfig.parse(m.get("rot"), where + ".rot"),
                   window=None if size is None else as_int(size), kv_from=None if src is None else as_int(src))

    def to_dict(self) -> Dict[str, Any]:
        out: Dict[str, Any] = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim,
                               "scale": self.scale, "rot": self.rot.to_dict()}
        if self.window is not None:
            out["mask"] = {"size": self.window}
        if self.kv_from is not None:
            out["kv_from"] = self.kv_from
        return out

    def problems(self, where: str) -> List[str]:
        p: List[str] = []
        for name in ("heads", "kv_heads", "dim", "vdim"):
            if getattr(self, name) < 1:
                p.append(f"{where}.{name} must be >= 1 (got {getattr(self, name)})")
        if self.kv_heads >= 1 and self.heads % self.kv_heads:
            p.append(f"{where}: {self.kv_heads} kv_heads do not divide {self.heads} heads")
        if not (self.scale > 0 and math.isfinite(self.scale)):
            p.append(f"{where}.scale must be > 0 (got {self.scale})")
        if self.window is not None and self.window < 1:
            p.append(f"{where}.mask.size must be >= 1 (got {self.window})")
        p.extend(self.rot.problems(where + ".rot", self.dim))
        return p


@dataclasses.dataclass(frozen=True)
class MemoryConfig:
    """A matrix memory: the ``retention`` mixer (``decay``, ``rot``) or the right branch of ``parallel`` (``gate_cap``)."""

    heads: int
    dim: int
    vdim: int
    gate_cap: float = 0.0
    decay: Tuple[float, ...] = ()
    rot: Optional[RotaryConfig] = None

    def to_dict(self) -> Dict[str, Any]:
        out: Dict[str, Any] = {"heads": self.heads, "dim": self.dim, "vdim": self.vdim}
        if self.rot is not None:
            out.update(decay=list(self.decay), rot=self.rot.to_dict())
        else:
            out["gate_cap"] = self.gate_cap
        return out

    def problems(self, where: str) -> List[str]:
        p: List[str] = []
        for name in ("heads", "dim", "vdim"):
            if getattr(self, name) < 1:
                p.append(f"{where}.{name} must be >= 1 (got {getattr(self, name)})")
        if self.dim > 256:
            p.append(f"{where}.dim must be at most 256 (got {self.dim})")
        if self.rot is not None:
            if len(self.decay) != self.heads:
                p.append(f"{where}.decay needs one number per head ({len(self.decay)} for {self.heads})")
            if any(not (0.0 <= d <= 1.0) for d in self.decay):
                p.append(f"{where}.decay: every decay lies in [0, 1]")
            p.extend(self.rot.problems(where + ".rot", self.dim))
        elif not (self.gate_cap > 0 and math.isfinite(self.gate_cap)):
            p.append(f"{where}.gate_cap must be > 0 (got {self.gate_cap})")
        return p


@dataclasses.dataclass(frozen=True)
class LayerConfig:
    type: str
    ff: Optional[int]                        # inner width of the dense feed-forward; None: no feed-forward
    attention: Optional[SoftmaxConfig] = None
    memory: Optional[MemoryConfig] = None

    @classmethod
    def parse(cls, v: Any) -> "LayerConfig":
        v = _obj(v, "a layer")
        kind = v.get("type")
        if kind not in LAYER_TYPES:
            raise ValueError(f"layer type must be one of {LAYER_TYPES} (got {kind!r})")
        m = _obj(v.get("mixer"), "mixer")
        mlp = v.get("mlp")
        ff = None
        if mlp is not None:
            mlp = _obj(mlp, "mlp")
            if mlp.get("kind") != "dense":
                raise ValueError(f"mlp.kind must be 'dense' (got {mlp.get('kind')!r})")
            ff = as_int(mlp.get("ff"))
        if kind == "attention":
            return cls(kind, ff, attention=SoftmaxConfig.parse(m, "mixer"))
        if kind == "retention":
            decay = m.get("decay")
            if not isinstance(decay, (list, tuple)):
                raise TypeError(f"mixer.decay must be a list, got {decay!r}")
            return cls(kind, ff, memory=MemoryConfig(
                heads=as_int(m.get("heads")), dim=as_int(m.get("dim")), vdim=as_int(m.get("vdim")),
                decay=tuple(as_float(d) for d in decay), rot=RotaryConfig.parse(m.get("rot"), "mixer.rot")))
        right = _obj(m.get("right"), "mixer.right")
        return cls(kind, ff, attention=SoftmaxConfig.parse(_obj(m.get("left"), "mixer.left"), "mixer.left"),
                   memory=MemoryConfig(heads=as_int(right.get("heads")), dim=as_int(right.get("dim")),
                                       vdim=as_int(right.get("vdim")), gate_cap=as_float(right.get("gate_cap"))))

    def to_dict(self) -> Dict[str, Any]:
        if self.type == "attention":
            mixer = self.attention.to_dict()
        elif self.type == "retention":
            mixer = self.memory.to_dict()
        else:
            mixer = {"left": self.attention.to_dict(), "right": self.memory.to_dict()}
        return {"type": self.type, "mixer": mixer, "mlp": None if self.ff is None else {"kind": "dense", "ff": self.ff}}

    def problems(self, where: str) -> List[str]:
        p: List[str] = []
        if self.attention is not None:
            p.extend(self.attention.problems(where + (".mixer.left" if self.type == "parallel" else ".mixer")))
        if self.memory is not None:
            p.extend(self.memory.problems(where + (".mixer.right" if self.type == "parallel" else ".mixer")))
        if self.ff is not None and self.ff < 1:
            p.append(f"{where}.mlp.ff must be >= 1 (got {self.ff})")
        return p


def _layers(v: Any) -> Tuple[LayerConfig, ...]:
    if not isinstance(v, (list, tuple)) or not v:
        raise TypeError("layers must be a list with at least one entry")
    return tuple(LayerConfig.parse(x) for x in v)


def _eps(v: Any) -> float:
    return as_float(_obj(v, "norm").get("eps"))


def _embedding_scale(v: Any) -> float:
    return as_float(_obj(v, "embedding").get("scale"))


def _req(conv, key=None):
    md = {"convert": conv, "required": True}
    if key:
        md["key"] = key
    return dataclasses.field(default=None, metadata=md)


@dataclasses.dataclass(frozen=True)
class TumudraConfig(ModelConfig):
    vocab: int = _req(as_int)
    width: int = _req(as_int)
    layers: Tuple[LayerConfig, ...] = _req(_layers)
    norm_eps: float = _req(_eps, key="norm")
    embedding_scale: float = _req(_embedding_scale, key="embedding")
    architecture: str = dataclasses.field(default="Tumudra", metadata={"convert": str})
    initializer_range: float = dataclasses.field(default=0.02, metadata={"convert": as_float})

    @classmethod
    def architecture_names(cls) -> Tuple[str, ...]:
        return ("Tumudra",)

    def to_dict(self) -> Dict[str, Any]:
        return {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
                "embedding": {"scale": self.embedding_scale}, "norm": {"eps": self.norm_eps},
                "layers": [l.to_dict() for l in self.layers], "initializer_range": self.initializer_range}

    def problems(self) -> List[str]:
        p: List[str] = []
        if self.vocab < 1 or self.width < 1:
            p.append(f"vocab and width must be >= 1 (got {self.vocab}, {self.width})")
        if not self.norm_eps > 0:
            p.append(f"norm.eps must be > 0 (got {self.norm_eps})")
        if not math.isfinite(self.embedding_scale):
            p.append(f"embedding.scale must be finite (got {self.embedding_scale})")
        if not (1 <= len(self.layers) <= 1024):
            p.append(f"between 1 and 1024 layers (got {len(self.layers)})")
        for i, layer in enumerate(self.layers):
            where = f"layers[{i}]"
            p.extend(layer.problems(where))
            a = layer.attention
            if a is not None and a.kv_from is not None:
                j = a.kv_from
                src = self.layers[j].attention if 0 <= j < i else None
                if layer.type != "attention":
                    p.append(f"{where}.mixer: kv_from belongs to layers of type 'attention'")
                elif src is None or self.layers[j].type != layer.type or src.kv_from is not None:
                    p.append(f"{where}.mixer.kv_from must name an earlier layer of the same type with keys and values "
                             f"of its own (got {j})")
                elif (src.kv_heads, src.dim, src.vdim, src.rot) != (a.kv_heads, a.dim, a.vdim, a.rot):
                    p.append(f"{where}.mixer.kv_from: layer {j}'s kv_heads, dim, vdim and rot differ from this layer's")
        if not self.initializer_range > 0:
            p.append(f"initializer_range must be > 0 (got {self.initializer_range})")
        return p


def _softmax_part(cfg: TumudraConfig, a: SoftmaxConfig, pre: str, local: str, biased: bool, layout: str):
    """The attention mixer's spec and the map of its parameters to checkpoint names (``pre``: the checkpoint's
    prefix, ``local``: the prefix of the local parameter names)."""
    shared = a.kv_from is not None
    spec = PartSpec("attention", {
        "hidden_size": cfg.width, "n_heads": a.heads, "n_kv_heads": a.kv_heads, "head_dim": a.dim, "v_head_dim": a.vdim,
        "scale": a.scale, "softcap": None, "window": a.window, "bias": biased, "qk_norm": {"eps": cfg.norm_eps},
        "shared_kv": shared, "position": a.rot.part(a.dim, layout)})
    names = {}
    for n in ("q", "o") + (() if shared else ("k", "v")):
        names[f"{local}{n}_proj"] = f"{pre}{n}"
        if biased:
            names[f"{local}{n}_bias"] = f"{pre}{n}.b"
    names[f"{local}q_norm"] = f"{pre}q.norm"
    if not shared:
        names[f"{local}k_norm"] = f"{pre}k.norm"
    return spec, names


def _memory_names(pre: str, local: str, extra=()) -> Dict[str, str]:
    names = {f"{local}{n}": f"{pre}{n}" for n in ("q", "k", "v", "o")}
    names[f"{local}gate"] = f"{pre}g"
    for loc, ck in extra:
        names[f"{local}{loc}"] = f"{pre}{ck}"
    return names


def tumudra_spec(cfg: TumudraConfig) -> ModelSpec:
    W, eps = cfg.width, cfg.norm_eps
    norm = PartSpec("layernorm", {"size": W, "eps": eps})
    layers, schedule = [], []
    for i, lc in enumerate(cfg.layers):
        pre = f"l{i}."
        tensors = {"norms.post_mixer.weight": pre + "norm1"}
        line, writes = i, True
        if lc.type == "attention":
            mixer, names = _softmax_part(cfg, lc.attention, pre + "mix.", "mixer.", biased=True, layout="half")
            tensors.update(names)
        elif lc.type == "retention":
            m = lc.memory
            mixer = PartSpec("retention", {"hidden_size": W, "n_heads": m.heads, "dim": m.dim, "vdim": m.vdim,
                                           "decay": m.decay, "eps": eps, "position": m.rot.part(m.dim, "half")})
            tensors.update(_memory_names(pre + "mix.", "mixer."))
        else:
            left, names = _softmax_part(cfg, lc.attention, pre + "mix.left.", "mixer.left.", biased=False,
                                        layout="interleaved")
            tensors.update(names)
            m = lc.memory
            right = PartSpec("mlstm", {"hidden_size": W, "n_heads": m.heads, "dim": m.dim, "vdim": m.vdim,
                                       "gate_cap": m.gate_cap, "eps": eps})
            tensors.update(_memory_names(pre + "mix.right.", "mixer.right.",
                                         (("norm", "norm"), ("i", "i"), ("i_bias", "i.b"), ("f", "f"), ("f_bias", "f.b"))))
            tensors["mixer.left.out"] = pre + "mix.left.out"
            tensors["mixer.right.out"] = pre + "mix.right.out"
            mixer = PartSpec("parallel", {"hidden_size": W, "eps": eps, "branches": {"left": left, "right": right}})
        if lc.attention is not None and lc.attention.kv_from is not None:
            line, writes = lc.attention.kv_from, False        # the cache line of the layer whose keys and values it reads
        ff = None
        norms = {"post_mixer": norm}
        if lc.ff is not None:
            ff = PartSpec("mlp", {"hidden_size": W, "intermediate_size": lc.ff, "activation": "relu2"})
            tensors.update({"ff.up_proj": pre + "mlp.up", "ff.down_proj": pre + "mlp.down",
                            "norms.post_ff.weight": pre + "norm2"})
            norms["post_ff"] = norm
        layers.append(LayerSpec(block=PartSpec("postnorm", {}), mixer=mixer, feed_forward=ff, norms=norms,
                                tensors=tensors))
        schedule.append(ScheduleEntry(layer=i, cache=line, writes_cache=writes))
    return ModelSpec(
        name="Tumudra", hidden_size=W,
        embedding=EmbeddingSpec(cfg.vocab, W, cfg.embedding_scale, "embed"),
        layers=tuple(layers), schedule=tuple(schedule),
        head=HeadSpec(cfg.vocab, W, tied=False, tensor="head", softcap=None, norm=norm, norm_tensor="final.norm"),
        max_positions=MAX_POSITIONS, stop_ids=(), init_std=cfg.initializer_range, init_norm_std=0.1)


TUMUDRA = register_architecture(Architecture(
    name="Tumudra", config_cls=TumudraConfig, build_spec=tumudra_spec, aliases=("tumudra",)))
