"""Two mixers side by side: both read the same input, and the result is a weighted sum of theirs.

The mixers are parts of the "mixer" family named by the spec; what a run keeps per sequence is what both keep (keys and
values of the one beside the state of the other, say), so `cache_need()` gives both needs and the cache hands a view
with the fields of both.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from .. import kernels as K
from ..plan import PartPlan
from ..registry import part_class, register_part
from .base import Part


@dataclass(frozen=True)
class ParallelMixersSpec:
    left: PartPlan                # family "mixer"
    right: PartPlan
    left_scale: float = 1.0
    right_scale: float = 1.0


@dataclass
class WeightedPair:
    """scale_a * a + scale_b * b, not summed yet: a block whose next kernel can take the sum (`sums_pairs`) gets this."""
    a: torch.Tensor
    scale_a: float
    b: torch.Tensor
    scale_b: float


@register_part("mixer", "parallel_mixers")
class ParallelMixers(Part):
    family = "mixer"
    roles = ()
    gives_pairs = True            # forward(..., as_pair=True) leaves the weighted sum to the caller's next kernel

    def __init__(self, spec, tensors, runtime):
        super().__init__(spec, tensors, runtime)
        self.left = part_class("mixer", spec.left.kind)(spec.left.spec, spec.left.tensors, runtime)
        self.right = part_class("mixer", spec.right.kind)(spec.right.spec, spec.right.tensors, runtime)
        self.graph_safe = bool(getattr(self.left, "graph_safe", False) and getattr(self.right, "graph_safe", False))
        self.kernel_modules = tuple(sorted({"stream_ops", *getattr(self.left, "kernel_modules", ()),
                                            *getattr(self.right, "kernel_modules", ())}))

    def tensor_specs(self):
        return self.left.tensor_specs() + self.right.tensor_specs()

    def bind(self, loaded):
        self.left.bind(loaded)
        self.right.bind(loaded)

    def prepare(self, max_positions: int) -> None:
        for m in (self.left, self.right):
            if hasattr(m, "prepare"):
                m.prepare(max_positions)

    def cache_need(self):
        needs = []
        for m in (self.left, self.right):
            need = m.cache_need()
            needs.extend(need if isinstance(need, tuple) else [need])
        return tuple(n for n in needs if n.kind != "none")

    def forward(self, x, step, cache, as_pair=False):
        """`as_pair`: the caller's next kernel takes the weighted sum itself; it gets a WeightedPair."""
        a = self.left.forward(x, step, cache)
        b = self.right.forward(x, step, cache)
        if a.dtype != torch.float32 or b.dtype != torch.float32:
            raise ValueError("mixers that run side by side hand their outputs over in float32")
        if as_pair:
            return WeightedPair(a, self.spec.left_scale, b, self.spec.right_scale)
        out = torch.empty_like(a)
        K.weighted_sum(a, self.spec.left_scale, b, self.spec.right_scale, out)
        return out
