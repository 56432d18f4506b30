"""Attention without a softmax, whose heads' weights are mixed before they meet the values.

q = Wq h + bq, k = Wk h + bk, v = Wv h + bv; the first `rotary_dim` lanes of every q and k head are rotated (lane i
with lane i + rotary_dim / 2, angle position * base^(-2i / rotary_dim), taken in fp64 and applied in fp32); query head h reads
key/value head h // (heads / kv heads); keys have `head_dim` lanes and values `value_dim`.  s = scale q.k, then
softcap tanh(s / softcap) when a cap is set; the weight of a visible key (j <= i) is sigmoid(s + head_bias_h), not
normalised over the keys; weights are mixed across heads, w'_h = sum_g talk[h, g] w_g, and head h applies w'_h to the
values of its own key/value head; then the output projection.
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
from .mamba2 import f32

BLOCKS_PER_SM = 2     # blocks a step should offer every multiprocessor before keys are cut into ranges
RANGE_KEYS = 256      # a range of keys is not made shorter than this


@dataclass(frozen=True)
class SigmoidAttentionSpec:
    hidden_size: int
    n_heads: int
    n_kv_heads: int
    head_dim: int                 # lanes of a head's query and key
    value_dim: int
    scale: float
    softcap: Optional[float] = None      # None: scores are not capped
    rotary_dim: int = 0
    rotary_base: float = 10000.0
    projection_bias: bool = True
    head_bias: bool = True               # a number per head added to the score inside the sigmoid
    talking_heads: bool = True           # the heads' weights are mixed by a [heads, heads] matrix


@register_part("mixer", "sigmoid_attention")
class SigmoidAttention(Part):
    family = "mixer"
    graph_safe = True
    roles = ("q", "k", "v", "o", "q_bias", "k_bias", "v_bias", "talk", "head_bias")
    kernel_modules = ("attention_sigmoid",)

    def __init__(self, spec, tensors, runtime):
        super().__init__(spec, tensors, runtime)
        s = spec
        if s.n_heads % s.n_kv_heads:
            raise ValueError(f"{s.n_heads} heads do not divide into {s.n_kv_heads} kv heads")
        if s.rotary_dim % 2 or not 0 <= s.rotary_dim <= s.head_dim:
            raise ValueError(f"{s.rotary_dim} rotated lanes: an even number of at most head_dim {s.head_dim}")
        half = s.rotary_dim // 2
        self.freq = torch.tensor([s.rotary_base ** (-2.0 * i / s.rotary_dim) for i in range(half)], dtype=torch.float64) \
            .to(runtime.device) if half else None

    def tensor_specs(self):
        s, t = self.spec, self.tensor_names
        qw, kw, vw = s.n_heads * s.head_dim, s.n_kv_heads * s.head_dim, s.n_kv_heads * s.value_dim
        specs = [TensorSpec(t["q"], (qw, s.hidden_size)), TensorSpec(t["k"], (kw, s.hidden_size)),
                 TensorSpec(t["v"], (vw, s.hidden_size)), TensorSpec(t["o"], (s.hidden_size, s.n_heads * s.value_dim))]
        if s.projection_bias:
            specs += [TensorSpec(t["q_bias"], (qw,), init="normal:0.1"), TensorSpec(t["k_bias"], (kw,), init="normal:0.1"),
                      TensorSpec(t["v_bias"], (vw,), init="normal:0.1")]
        if s.talking_heads:
            specs.append(TensorSpec(t["talk"], (s.n_heads, s.n_heads), init="normal:0.4"))
        if s.head_bias:
            specs.append(TensorSpec(t["head_bias"], (s.n_heads,), init="normal:1.0"))
        return specs

    def bind(self, loaded):
        s, t = self.spec, self.tensor_names
        ws = [loaded[t["q"]], loaded[t["k"]], loaded[t["v"]]]
        if len({w.dtype for w in ws}) != 1:
            raise ValueError(f"{t['q']}, {t['k']}, {t['v']} are stored in different dtypes")
        self.qkv = Linear(torch.cat(ws, dim=0).contiguous())
        self.o = Linear(loaded[t["o"]])
        self.bias = torch.cat([f32(loaded[t[r]]) for r in ("q_bias", "k_bias", "v_bias")]).contiguous() if s.projection_bias else None
        self.talk = f32(loaded[t["talk"]]) if s.talking_heads else None
        self.head_bias = f32(loaded[t["head_bias"]]) if s.head_bias else None
        if self.runtime.device.type == "cuda" and not K.sigmoid_attention_takes(self.runtime.dtype, s.n_heads, s.n_kv_heads,
                                                                                s.head_dim, s.value_dim):
            raise ValueError(f"{s.n_heads} heads of {s.head_dim} + {s.value_dim} lanes are beyond what the attention kernel holds")

    def cache_need(self) -> CacheNeed:
        s = self.spec
        return CacheNeed("kv", n_kv_heads=s.n_kv_heads, head_dim=s.head_dim, window=None, value_dim=s.value_dim)

    def _ranges(self, step) -> int:
        """Over how many blocks a query's keys are cut: nothing is normalised over the keys, so partial outputs just add.
        Few query rows with long pasts (decoding) would leave most multiprocessors idle otherwise."""
        tiles = step.n_seqs * ((step.max_q_len + 15) // 16)
        want = (4 if step.max_q_len == 1 else BLOCKS_PER_SM) * K.sm_count(self.runtime.device)      # single rows: small blocks, four an SM
        shortest = K.PAGE if step.max_q_len == 1 else RANGE_KEYS                  # a single row's range may be one page
        return max(1, min((want + tiles - 1) // tiles, step.max_kv_len // shortest, 64))

    def forward(self, x, step, cache):
        s, rt = self.spec, self.runtime
        if not cache.writes:
            raise ValueError("this mixer appends to a cache line of its own; it cannot read another run's")
        n = step.n_tokens
        proj = self.qkv(x, out_dtype=torch.float32)                  # [N, q | k | v] in fp32
        q = torch.empty((n, s.n_heads * s.head_dim), dtype=rt.dtype, device=proj.device)
        K.bias_rope_append(proj, self.bias, self.freq, s.rotary_dim, q, cache.pool, cache.block_table, step, s.n_heads,
                           s.n_kv_heads, s.head_dim, s.value_dim)
        out = torch.zeros((n, s.n_heads * s.value_dim), dtype=rt.dtype, device=proj.device)   # rows of no sequence stay zero
        ranges = self._ranges(step)
        partial = None
        if ranges > 1:
            partial = step.workspace.scratch("sigmoid_attention", ranges * n * s.n_heads * s.value_dim)
        K.sigmoid_attention(q, cache.pool, cache.block_table, step, out, s.n_heads, s.n_kv_heads, s.head_dim, s.value_dim, s.scale,
                            softcap=s.softcap or 0.0, talk=self.talk, head_bias=self.head_bias, ranges=ranges, partial=partial)
        return self.o(out, out_dtype=torch.float32)
