"""The Fobilorn decoder as a plan of parts: the registry entry "Fobilorn".

Token embedding plus a hashed embedding of token pairs, squashed by a Dynamic Tanh norm; parallel blocks (one
Dynamic Tanh norm whose output both the mixer and the feed-forward read); windowed attention with kept first
tokens, a sink in the softmax, a norm over the whole query and key projections, values blended with the first
blending layer's, and a gate per head; a dense gated feed-forward or a mixture of experts with sigmoid scores whose
weights multiply the experts' inputs, beside a shared expert; a last Dynamic Tanh norm and the output projection.
Every layer brings its own sizes.  Stored names: 'embed', 'bigram', 'embed.norm', 'l<i>.norm1', 'l<i>.mix.*',
'l<i>.mlp.*', 'final.norm', 'head'; a norm's bias and scalar lie beside its weight as '<name>.b' and '<name>.alpha'.
"""
from __future__ import annotations

from ..config.fobilorn import FobilornConfig
from ..config.reader import ConfigError
from ..parts.embedding import HeadSpec, PairEmbeddingSpec
from ..parts.feed_forward import SwiGLUSpec
from ..parts.moe import SigmoidMoESpec
from ..parts.norm import DynamicTanhSpec
from ..parts.sink_attention import SinkAttentionSpec
from ..plan import LayerPlan, ModelPlan, NamedPart, PartPlan, ScheduleEntry
from ..registry import Architecture, register_architecture

MAX_POSITIONS = 1 << 20     # nothing in the design depends on the position itself; the cache sets the real limit


def _norm(width: int, name: str) -> PartPlan:
    return PartPlan("dynamic_tanh", DynamicTanhSpec(width), {"weight": name, "bias": name + ".b", "alpha": name + ".alpha"})


def _gated(width: int, inner: int, prefix: str) -> PartPlan:
    return PartPlan("swiglu", SwiGLUSpec(width, inner), {"gate": prefix + "gate", "up": prefix + "up", "down": prefix + "down"})


def fobilorn_plan(cfg: FobilornConfig) -> ModelPlan:
    width = cfg.width
    layers = []
    blends = False       # whether an earlier layer already is the source of blended values
    blended = None       # lanes of those values (kv heads x value size): the same in every layer that blends
    for i, layer in enumerate(cfg.layers):
        p, m = f"l{i}.", layer.mixer
        tensors = {"q": p + "mix.q", "k": p + "mix.k", "v": p + "mix.v", "o": p + "mix.o", "g": p + "mix.g",
                   "q_norm": p + "mix.q.norm", "k_norm": p + "mix.k.norm"}
        blend = None
        if m.v_mix:
            blend = "blend" if blends else "source"
            blends = True
            if blended is not None and blended != m.kv_heads * m.vdim:
                raise ConfigError(f"config key 'layers[{i}].mixer': v_mix blends values of {m.kv_heads} x {m.vdim} lanes with "
                                  f"the {blended} lanes of the first layer that has v_mix")
            blended = m.kv_heads * m.vdim
            tensors["blend"] = p + "mix.vmix"      # stored in the source layer too, where nothing reads it
        parts = [NamedPart("norm", "norm", _norm(width, p + "norm1")),
                 NamedPart("mixer", "mixer", PartPlan("sink_attention", SinkAttentionSpec(
                     hidden_size=width, n_heads=m.heads, n_kv_heads=m.kv_heads, head_dim=m.dim, value_dim=m.vdim, scale=m.scale,
                     window=m.window, keep_first=m.keep_first, sink=True, qk_norm_eps=cfg.eps, head_gate=True,
                     value_blend=blend), tensors))]
        f = layer.mlp
        if f is not None and f.kind == "dense":
            parts.append(NamedPart("feed_forward", "feed_forward", _gated(width, f.ff, p + "mlp.")))
        elif f is not None:
            shared = _gated(width, f.shared_ff, p + "mlp.shared.") if f.shared_ff is not None else None
            parts.append(NamedPart("feed_forward", "feed_forward", PartPlan(
                "sigmoid_moe", SigmoidMoESpec(width, f.experts, f.top, f.ff, weight_on="input", shared=shared),
                {"router": p + "mlp.router", "gate": p + "mlp.e{}.gate", "up": p + "mlp.e{}.up", "down": p + "mlp.e{}.down"})))
        layers.append(LayerPlan("parallel", tuple(parts)))
    b = cfg.bigram
    return ModelPlan(
        architecture=cfg.architecture,
        vocab_size=cfg.vocab,
        hidden_size=width,
        embedding=PartPlan("token_pairs", PairEmbeddingSpec(cfg.vocab, width, b.buckets, b.mul_prev, b.mul_cur,
                                                            norm=_norm(width, "embed.norm")),
                           {"table": "embed", "pairs": "bigram"}),
        layers=tuple(layers),
        schedule=tuple(ScheduleEntry(n) for n in range(len(layers))),
        final_norm=_norm(width, "final.norm"),
        head=PartPlan("linear", HeadSpec(cfg.vocab, width), {"weight": "head"}),
        max_positions=MAX_POSITIONS,
        # a writer may store the blend's scalar in layers that do not blend; nothing reads it there
        ignorable_tensors=(r"l\d+\.mix\.vmix",),
    )


FOBILORN = register_architecture(Architecture(
    name="Fobilorn", config_class=FobilornConfig, plan=fobilorn_plan, aliases=("fobilorn",),
    description="parallel blocks: windowed sink attention with gated heads, dense or mixture-of-experts feed-forward, "
                "Dynamic Tanh norms, token-pair embedding"))
