"""Dense feed-forwards.  The gated one: (silu(x Wgate) * (x Wup)) Wdown, no biases
(crates/burn-lm-llama/src/nn/fftn.rs:26-36,44-46).  Gate and up run as one product with a fused
[gate; up] weight; the activation and the product of the two halves are fp32.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from .. import kernels as K
from ..registry import register_part
from ..weights.loader import TensorSpec
from .base import Part
from .linear import Linear


@dataclass(frozen=True)
class SwiGLUSpec:
    hidden_size: int
    intermediate_size: int


@register_part("feed_forward", "swiglu")
class SwiGLU(Part):
    family = "feed_forward"
    graph_safe = True
    roles = ("gate", "up", "down")

    def tensor_specs(self):
        s, t = self.spec, self.tensor_names
        return [TensorSpec(t["gate"], (s.intermediate_size, s.hidden_size)),
                TensorSpec(t["up"], (s.intermediate_size, s.hidden_size)),
                TensorSpec(t["down"], (s.hidden_size, s.intermediate_size))]

    def bind(self, loaded):
        t = self.tensor_names
        g, u = loaded[t["gate"]], loaded[t["up"]]
        if g.dtype != u.dtype:
            raise ValueError(f"{t['gate']} and {t['up']} are stored in different dtypes")
        inner = self.spec.intermediate_size
        if g.dtype == torch.bfloat16 and inner % K.GATE_TILE == 0:
            # tiles of 8 gate rows followed by the 8 up rows of the same outputs: the skinny kernel's
            # gated epilogue finds both halves of an output in one 16-row tile
            tile = K.GATE_TILE
            fused = torch.stack([g.view(inner // tile, tile, -1), u.view(inner // tile, tile, -1)], dim=1).reshape(2 * inner, -1)
            self.gate_up = Linear(fused.contiguous(), gate_tile=tile)
        else:
            self.gate_up = Linear(torch.cat([g, u], dim=0).contiguous())
        self.down = Linear(loaded[t["down"]])

    takes_pending_norm = True
    adds_to_stream = True

    def forward(self, x, step, stream=None):
        rt = self.runtime
        act = self.gate_up.gated(x, rt.dtype)
        return self.down.into_stream(act, stream, rt.dtype, handoff=getattr(step, "handoff", None))


@dataclass(frozen=True)
class BiasedMLPSpec:
    hidden_size: int
    intermediate_size: int
    activation: str = "xielu"


@register_part("feed_forward", "biased_mlp")
class BiasedMLP(Part):
    """W_down act(W_up h + b_up) + b_down.  Activation "xielu" has two learned numbers (p, q): for z > 0,
    softplus(p) z^2 + z / 2; for z <= 0, (1/2 + softplus(q)) (exp(z) - 1 - z) + z / 2.  The bias and the activation are
    taken in fp32 on the product's fp32 sums.  The down projection's bias is handed on with the output (a pair), for the
    kernel that reads the output next to add it."""
    family = "feed_forward"
    graph_safe = True
    roles = ("up", "up_bias", "down", "down_bias", "act")
    kernel_modules = ("stream_ops",)

    def __init__(self, spec, tensors, runtime):
        super().__init__(spec, tensors, runtime)
        if spec.activation != "xielu":
            raise ValueError(f"activation {spec.activation!r}; this feed-forward knows 'xielu'")

    def tensor_specs(self):
        s, t = self.spec, self.tensor_names
        return [TensorSpec(t["up"], (s.intermediate_size, s.hidden_size)), TensorSpec(t["up_bias"], (s.intermediate_size,), init="normal:0.1"),
                TensorSpec(t["down"], (s.hidden_size, s.intermediate_size)), TensorSpec(t["down_bias"], (s.hidden_size,), init="normal:0.1"),
                TensorSpec(t["act"], (2,), init="normal:0.5")]

    def bind(self, loaded):
        t = self.tensor_names
        self.up, self.down = Linear(loaded[t["up"]]), Linear(loaded[t["down"]])
        f32 = lambda x: x.to(torch.float32).contiguous()
        self.up_bias, self.down_bias, self.params = f32(loaded[t["up_bias"]]), f32(loaded[t["down_bias"]]), f32(loaded[t["act"]])

    def forward(self, x, step):
        z = self.up(x, out_dtype=torch.float32)
        act = torch.empty(z.shape, dtype=self.runtime.dtype, device=z.device)
        K.bias_act(z, self.up_bias, act, K.ACT_XIELU, self.params)
        return self.down(act, out_dtype=torch.float32), self.down_bias
