"""The windowed attention mixer with kept first tokens, a sink in its softmax, a norm over the whole query and key
projections, values blended across layers, and a gate per head.

q = Wq h, k = Wk h, v = Wv h without biases; q and k are each divided by the root mean square of the whole
projection (all heads at once) and multiplied by a weight of that size; there is no rotation.  Query head h reads
key/value head h // (heads / kv heads); keys have `head_dim` lanes and values `value_dim`.  The query at position i
sees the key at j when j <= i and (i - j < window or j < keep_first).  p_j = exp(s_j) / (1 + sum exp(s_j)) with
s = scale q.k: a sink of score 0 that carries no value.  Layers that blend their values replace v by
(1 - lambda) v + lambda v_first, v_first being the values of the same token in the first blending layer of the step's
forward pass, and cache the blended v.  Head h's output is multiplied by sigmoid(Wg h)_h before the output projection.

The four projections run as one product with a fused [q; k; v; g] weight whose result stays in fp32 for the norms.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from .. import kernels as K
from ..registry import register_part
from ..weights.loader import TensorSpec
from .base import CacheNeed, Part
from .linear import Linear

BLOCKS_PER_SM = 4     # blocks of the row kernel a step should offer every multiprocessor


@dataclass(frozen=True)
class SinkAttentionSpec:
    hidden_size: int
    n_heads: int
    n_kv_heads: int
    head_dim: int                 # lanes of a head's query and key
    value_dim: int                # lanes of a head's value
    scale: float
    window: int
    keep_first: int = 0
    sink: bool = True             # one more entry of score 0 in the softmax's denominator
    qk_norm_eps: Optional[float] = None   # None: q and k are not normed
    head_gate: bool = True
    value_blend: Optional[str] = None     # None; "source": later layers blend this layer's values in; "blend": this layer
                                          # blends the source's values into its own
    blend_group: str = "values"           # layers that share a source name the same group


@register_part("mixer", "sink_attention")
class SinkAttention(Part):
    family = "mixer"
    graph_safe = True
    roles = ("q", "k", "v", "o", "g", "q_norm", "k_norm", "blend")
    kernel_modules = ("elementwise", "attention_sink")

    def __init__(self, spec, tensors, runtime):
        super().__init__(spec, tensors, runtime)
        if spec.n_heads % spec.n_kv_heads:
            raise ValueError(f"{spec.n_heads} heads do not divide into {spec.n_kv_heads} kv heads")
        if spec.value_dim > 512:
            raise ValueError(f"value_dim {spec.value_dim}: the attention kernels take values of up to 512 lanes")
        if spec.value_blend not in (None, "source", "blend"):
            raise ValueError(f"value_blend is None, 'source' or 'blend', not {spec.value_blend!r}")

    def tensor_specs(self):
        s, t = self.spec, self.tensor_names
        specs = [TensorSpec(t["q"], (s.n_heads * s.head_dim, s.hidden_size)),
                 TensorSpec(t["k"], (s.n_kv_heads * s.head_dim, s.hidden_size)),
                 TensorSpec(t["v"], (s.n_kv_heads * s.value_dim, s.hidden_size)),
                 TensorSpec(t["o"], (s.hidden_size, s.n_heads * s.value_dim))]
        if s.head_gate:
            specs.append(TensorSpec(t["g"], (s.n_heads, s.hidden_size)))
        if s.qk_norm_eps is not None:
            specs += [TensorSpec(t["q_norm"], (s.n_heads * s.head_dim,), init="one_plus_normal:0.1"),
                      TensorSpec(t["k_norm"], (s.n_kv_heads * s.head_dim,), init="one_plus_normal:0.1")]
        if "blend" in t:       # the source layer's scalar is stored but unread
            specs.append(TensorSpec(t["blend"], (), init="normal:0.3", optional=s.value_blend != "blend"))
        return specs

    def bind(self, loaded):
        s, t = self.spec, self.tensor_names
        ws = [loaded[t["q"]], loaded[t["k"]], loaded[t["v"]]] + ([loaded[t["g"]]] if s.head_gate else [])
        if len({w.dtype for w in ws}) != 1:
            raise ValueError(f"the projections of {t['q']} and its neighbours are stored in different dtypes")
        self.proj = Linear(torch.cat(ws, dim=0).contiguous())
        self.o = Linear(loaded[t["o"]])
        f32 = lambda x: x.to(torch.float32).contiguous()
        self.q_weight = f32(loaded[t["q_norm"]]) if s.qk_norm_eps is not None else None
        self.k_weight = f32(loaded[t["k_norm"]]) if s.qk_norm_eps is not None else None
        self.blend = f32(loaded[t["blend"]]).reshape(1) if s.value_blend == "blend" else None

    def cache_need(self) -> CacheNeed:
        s = self.spec
        return CacheNeed("kv", n_kv_heads=s.n_kv_heads, head_dim=s.head_dim, window=s.window, value_dim=s.value_dim,
                         keep_first=s.keep_first)

    def _splits(self, step) -> int:
        """Over how many blocks the row kernel cuts a row's keys: a few tokens with long windows leave most of the
        multiprocessors idle otherwise.  Every block should still have some chunks of 32 keys."""
        s = self.spec
        if K.attention_sink_prompt_takes(self.runtime.dtype, s.head_dim, s.value_dim, step.max_q_len, s.n_heads):
            return 1
        seen = min(step.max_kv_len, s.window + s.keep_first)
        blocks = step.n_tokens * s.n_kv_heads
        want = BLOCKS_PER_SM * K.sm_count(self.runtime.device)
        if K.attention_sink_decode_takes(self.runtime.dtype, s.head_dim, s.value_dim, s.n_heads, s.n_kv_heads):
            pages = seen // K.PAGE + 1                       # that kernel cuts by pages: some to every block, and its blocks
            want //= 2                                       # hold three pages each: half as many fill a multiprocessor
            return max(1, min((want + blocks - 1) // blocks, pages // 4, 32))
        return max(1, min((want + blocks - 1) // blocks, seen // 128, 32))

    adds_to_stream = True

    def forward(self, x, step, cache, stream=None):
        s, rt = self.spec, self.runtime
        if not cache.writes:
            raise ValueError("this mixer appends to a cache line of its own; it cannot read another run's")
        n = step.n_tokens
        proj = self.proj(x, out_dtype=torch.float32)            # [N, q | k | v | g] in fp32
        q = torch.empty((n, s.n_heads * s.head_dim), dtype=rt.dtype, device=proj.device)
        v_cols = s.n_kv_heads * s.value_dim
        values_in = values_out = None
        key = ("value_blend", s.blend_group)
        if s.value_blend == "source":
            values_out = step.memo[key] = torch.empty((n, v_cols), dtype=torch.float32, device=proj.device)
        elif s.value_blend == "blend":
            values_in = step.memo.get(key)
            if values_in is None or tuple(values_in.shape) != (n, v_cols):
                raise ValueError("a layer blends values in, but no earlier layer of the step has left values of that size")
        K.qk_norm_append(proj, step, cache.pool, cache.block_table, q, s.n_heads, s.n_kv_heads, s.head_dim, s.value_dim,
                         q_weight=self.q_weight, k_weight=self.k_weight, eps=s.qk_norm_eps or 0.0, blend=self.blend,
                         values_in=values_in, values_out=values_out)
        out = torch.empty((n, s.n_heads * s.value_dim), dtype=rt.dtype, device=proj.device)
        gate_at = (s.n_heads + s.n_kv_heads) * s.head_dim + v_cols
        n_splits = self._splits(step)
        scratch = None
        if n_splits > 1:
            scratch = step.workspace.scratch("attention_sink", K.attention_sink_scratch_floats(n, s.n_heads, s.value_dim, n_splits))
        K.attention_sink(q, step, cache.pool, cache.block_table, out, s.n_heads, s.n_kv_heads, s.head_dim, s.value_dim, s.scale,
                         s.window, s.keep_first, sink=s.sink, gate=proj[:, gate_at:] if s.head_gate else None,
                         gate_stride=proj.stride(0), max_q_len=step.max_q_len, n_splits=n_splits, scratch=scratch)
        return self.o.into_stream(out, stream, rt.dtype, handoff=None)
