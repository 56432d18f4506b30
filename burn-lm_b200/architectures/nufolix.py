"""The Nufolix decoder as a plan of parts: the registry entry "Nufolix".

A scaled token embedding; layers whose sublayers stand between two RMS norms each, the normed output multiplied by one
model-wide number before it joins the stream (block "sandwich"); a mixer per layer that is either a state-space scan
(Mamba-2) or two mixers side by side, attention without a softmax (biased projections, partial rotation, capped scores,
a sigmoid per key, weights mixed across heads) beside a gated delta rule; a dense feed-forward with biases and the xIELU
activation, or none; a last RMS norm and the embedding table as the output projection.  Every layer brings its own
sizes.  Stored names: 'embed', 'l<i>.norm1', 'l<i>.norm1b', 'l<i>.norm2', 'l<i>.norm2b', 'l<i>.mix.*', 'l<i>.mlp.*',
'final.norm'; a projection's bias lies beside its weight as '<name>.b', a convolution's taps as '<name>.conv'.
"""
from __future__ import annotations

from ..config.nufolix import NufolixConfig
from ..parts.embedding import HeadSpec, ScaledEmbeddingSpec
from ..parts.feed_forward import BiasedMLPSpec
from ..parts.gated_delta import GatedDeltaSpec
from ..parts.mamba2 import Mamba2Spec
from ..parts.norm import PostRMSNormSpec, RMSNormSpec
from ..parts.parallel_mixers import ParallelMixersSpec
from ..parts.sigmoid_attention import SigmoidAttentionSpec
from ..plan import LayerPlan, ModelPlan, NamedPart, PartPlan, ScheduleEntry
from ..registry import Architecture, register_architecture

MAX_POSITIONS = 1 << 20     # the rotation takes any position; the cache sets the real limit


def nufolix_plan(cfg: NufolixConfig) -> ModelPlan:
    width, eps = cfg.width, cfg.eps
    pre = lambda name: PartPlan("rmsnorm", RMSNormSpec(width, eps), {"weight": name})
    post = lambda name: PartPlan("rms_post", PostRMSNormSpec(width, eps, cfg.residual_mult), {"weight": name})
    layers = []
    for i, layer in enumerate(cfg.layers):
        p, m = f"l{i}.", layer.mixer
        if layer.type == "mamba2":
            mixer = PartPlan("mamba2", Mamba2Spec(width, m.heads, m.vdim, m.state, m.groups, m.conv, m.norm_groups, eps),
                             {"in": p + "mix.in", "conv": p + "mix.conv", "conv_bias": p + "mix.conv.b", "dt_bias": p + "mix.dt_bias",
                              "A_log": p + "mix.A_log", "D": p + "mix.D", "norm": p + "mix.norm", "o": p + "mix.o"})
        else:
            lf, rg = m.left, m.right
            a, b = p + "mix.left.", p + "mix.right."
            left = PartPlan("sigmoid_attention", SigmoidAttentionSpec(
                hidden_size=width, n_heads=lf.heads, n_kv_heads=lf.kv_heads, head_dim=lf.dim, value_dim=lf.vdim, scale=lf.scale,
                softcap=lf.softcap, rotary_dim=lf.rot_dims, rotary_base=lf.rot_base, projection_bias=True, head_bias=True,
                talking_heads=True),
                {"q": a + "q", "k": a + "k", "v": a + "v", "o": a + "o", "q_bias": a + "q.b", "k_bias": a + "k.b", "v_bias": a + "v.b",
                 "talk": a + "talk", "head_bias": a + "pb"})
            right = PartPlan("gated_delta", GatedDeltaSpec(
                hidden_size=width, n_heads=rg.heads, qk_heads=rg.kv_heads, key_dim=rg.dim, value_dim=rg.vdim, conv=rg.conv, eps=eps),
                {"q": b + "q", "q_conv": b + "q.conv", "k": b + "k", "k_conv": b + "k.conv", "v": b + "v", "v_conv": b + "v.conv",
                 "b": b + "b", "A_log": b + "A_log", "norm": b + "norm", "a1": b + "a1", "a2": b + "a2", "dt_bias": b + "dt_bias",
                 "g1": b + "g1", "g2": b + "g2", "o": b + "o"})
            mixer = PartPlan("parallel_mixers", ParallelMixersSpec(left, right, m.left_scale, m.right_scale))
        parts = [NamedPart("mixer_norm", "norm", pre(p + "norm1")), NamedPart("mixer", "mixer", mixer),
                 NamedPart("mixer_post_norm", "norm", post(p + "norm1b"))]
        if layer.ff is not None:
            parts += [NamedPart("feed_forward_norm", "norm", pre(p + "norm2")),
                      NamedPart("feed_forward", "feed_forward", PartPlan(
                          "biased_mlp", BiasedMLPSpec(width, layer.ff, "xielu"),
                          {"up": p + "mlp.up", "up_bias": p + "mlp.up.b", "down": p + "mlp.down", "down_bias": p + "mlp.down.b",
                           "act": p + "mlp.act"})),
                      NamedPart("feed_forward_post_norm", "norm", post(p + "norm2b"))]
        layers.append(LayerPlan("sandwich", tuple(parts)))
    return ModelPlan(
        architecture=cfg.architecture,
        vocab_size=cfg.vocab,
        hidden_size=width,
        embedding=PartPlan("scaled_table", ScaledEmbeddingSpec(cfg.vocab, width, cfg.embedding_scale), {"table": "embed"}),
        layers=tuple(layers),
        schedule=tuple(ScheduleEntry(n) for n in range(len(layers))),
        final_norm=pre("final.norm"),
        head=PartPlan("linear", HeadSpec(cfg.vocab, width), {"weight": "embed"}),      # the table itself, without the scale
        max_positions=MAX_POSITIONS,
    )


NUFOLIX = register_architecture(Architecture(
    name="Nufolix", config_class=NufolixConfig, plan=nufolix_plan, aliases=("nufolix",),
    description="sandwich-normed layers: a Mamba-2 scan, or sigmoid attention with mixed heads beside a gated delta rule; "
                "dense xIELU feed-forward; tied output table"))
