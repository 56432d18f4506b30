"""Norms fused with the residual add: RMS norm, and Dynamic Tanh (which takes no statistics).

y = x / sqrt(mean(x^2) + eps) * gamma; it stands before the mixer, before the feed-forward and once
after the last block (crates/burn-lm-llama/src/nn/transformer.rs:248-255,101; eps at :60-62 and
:211-216).  The sum of squares, the root and the product with gamma are fp32 in both paths.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from .. import kernels as K
from ..registry import register_part
from ..weights.loader import TensorSpec
from .base import Part
from .linear import NormedStream


@dataclass(frozen=True)
class RMSNormSpec:
    size: int
    eps: float


@register_part("norm", "rmsnorm")
class RMSNorm(Part):
    family = "norm"
    graph_safe = True
    roles = ("weight",)

    def tensor_specs(self):
        return [TensorSpec(self.tensor_names["weight"], (self.spec.size,), init="one_plus_normal:0.1")]

    def bind(self, loaded):
        self.gamma = loaded[self.tensor_names["weight"]]

    takes_handed_norm = True      # a product that writes the stream may leave this norm's input (parts.linear.NormHandoff)

    def add_norm(self, resid, delta, rows=None, lazy=False, handoff=None):
        """`lazy`: the caller can take a norm that is not computed yet (parts.linear.NormedStream);
        it gets one when nothing has to be added into the stream first.  `handoff`: where the writer of
        the stream may have left this norm's input."""
        handed = handoff.claim(resid, self.gamma) if handoff is not None else None
        if lazy and delta is None:
            return NormedStream(resid, self.gamma, self.spec.eps, rows, self.runtime.dtype, handed)
        n = rows.numel() if rows is not None else resid.shape[0]
        out = torch.empty((n, self.spec.size), dtype=self.runtime.dtype, device=resid.device)
        K.add_rmsnorm(resid, delta, self.gamma, self.spec.eps, out, rows)
        return out


@dataclass(frozen=True)
class DynamicTanhSpec:
    size: int


@register_part("norm", "dynamic_tanh")
class DynamicTanh(Part):
    """y = tanh(alpha x) * weight + bias with a learned scalar alpha: a squashing in the place of a norm, computed
    element by element in fp32 without a mean or a variance.  Weight, bias and alpha are kept in float32."""
    family = "norm"
    graph_safe = True
    roles = ("weight", "bias", "alpha")
    kernel_modules = ("elementwise",)
    takes_several = True          # `delta` may be a tuple of outputs that are all added into the stream

    def tensor_specs(self):
        t, n = self.tensor_names, self.spec.size
        return [TensorSpec(t["weight"], (n,), init="one_plus_normal:0.1"), TensorSpec(t["bias"], (n,), init="normal:0.1"),
                TensorSpec(t["alpha"], (), init="one_plus_normal:0.2")]

    def bind(self, loaded):
        t = self.tensor_names
        self.weight = loaded[t["weight"]].to(torch.float32).contiguous()
        self.bias = loaded[t["bias"]].to(torch.float32).contiguous()
        self.alpha = loaded[t["alpha"]].to(torch.float32).reshape(1).contiguous()

    def parameters(self):
        """(weight, bias, alpha) in float32, for a kernel that applies this norm in its own epilogue."""
        return self.weight, self.bias, self.alpha

    def add_norm(self, resid, delta, rows=None, lazy=False, handoff=None):
        deltas = list(delta) if isinstance(delta, (tuple, list)) else ([delta] if delta is not None else [])
        n = rows.numel() if rows is not None else resid.shape[0]
        out = torch.empty((n, self.spec.size), dtype=self.runtime.dtype, device=resid.device)
        K.add_dyt(resid, deltas, self.weight, self.bias, self.alpha, out, rows)
        return out
