"""Mixers side by side: several mixers read the same input, each output is RMS-normed over the model width with a
plain weight of its own, and the mixer's output is their mean.

    y = (1/n) sum_b  rmsnorm(branch_b(x)) * w_b

``branches`` maps a name to the branch's ``PartSpec`` (any registered mixer); the branch's parameters are this mixer's
``<name>.<parameter>`` and its weight ``<name>.out``.  The branches share one cache line: at most one of them may keep
keys and values and at most one a fixed-size state, and each sees what it asked for.  The mean is not formed here when
the block that holds the mixer can form it inside its own kernel (``forward_branches``).
"""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch

from ..kernels import ops
from .base import MIXERS, CacheNeed, Mixer, StateNeed
from .spec import PartSpec


@MIXERS.register("parallel")
class ParallelMixer(Mixer):
    def __init__(self, spec: PartSpec):
        super().__init__(spec)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.eps = float(p["eps"])
        self.names: List[str] = list(p["branches"])
        if not (1 <= len(self.names) <= 4):
            raise ValueError(f"parallel: one to four branches (got {len(self.names)})")
        self.branches: List[Mixer] = [MIXERS.get(p["branches"][n].kind)(p["branches"][n]) for n in self.names]
        if sum(b.cache_need() is not None for b in self.branches) > 1:
            raise ValueError("parallel: at most one branch may keep keys and values")
        if sum(b.state_need() is not None for b in self.branches) > 1:
            raise ValueError("parallel: at most one branch may keep a state")
        self.out_weights: List[torch.Tensor] = []

    @classmethod
    def param_shapes(cls, spec: PartSpec) -> Dict[str, Tuple[Tuple[int, ...], str]]:
        p = spec.params
        out: Dict[str, Tuple[Tuple[int, ...], str]] = {}
        for name, sub in p["branches"].items():
            for k, v in MIXERS.get(sub.kind).param_shapes(sub).items():
                out[f"{name}.{k}"] = v
            out[f"{name}.out"] = ((int(p["hidden_size"]),), cls.PARAM_ROLE_SCALE)
        return out

    def load(self, tensors, compute_dtype, device) -> None:
        self.out_weights = []
        for name, b in zip(self.names, self.branches):
            pre = name + "."
            b.load({k[len(pre):]: v for k, v in tensors.items() if k.startswith(pre) and k != pre + "out"},
                   compute_dtype, device)
            self.out_weights.append(tensors[pre + "out"].contiguous())

    def weight_bytes(self) -> int:
        return sum(b.weight_bytes() for b in self.branches) + sum(w.numel() * w.element_size() for w in self.out_weights)

    def cache_need(self) -> Optional[CacheNeed]:
        for b in self.branches:
            if b.cache_need() is not None:
                return b.cache_need()
        return None

    def state_need(self) -> Optional[StateNeed]:
        for b in self.branches:
            if b.state_need() is not None:
                return b.state_need()
        return None

    def scratch_need(self, step) -> int:
        return max(b.scratch_need(step) for b in self.branches)

    def schedule(self, step) -> tuple:
        return tuple(b.schedule(step) for b in self.branches)

    def forward_branches(self, x: torch.Tensor, step, line) -> List[torch.Tensor]:
        """The branches' outputs, not yet normed."""
        return [b.forward(x, step, line) for b in self.branches]

    def forward(self, x: torch.Tensor, step, line) -> torch.Tensor:
        return ops.mean_rmsnorm(self.forward_branches(x, step, line), self.out_weights, self.eps, x.dtype)
