"""The typed configuration of the Fobilorn decoder, read from its own config.json keys.

    architecture   "Fobilorn"
    vocab, width   sizes of the token table and of the residual stream
    embedding      {"bigram": {"buckets", "mul_prev", "mul_cur"}}: the hashed table of token pairs
    norm           {"eps"}: the eps of the root mean squares inside the mixers
    layers         a list; every entry has "type" (its mixer: "attention"), "mixer" (the mixer's sizes and
                   constants) and "mlp" (its feed-forward, or null for none)

An attention mixer: heads, kv_heads, dim (query/key size of a head), vdim (value size), scale, v_mix,
mask {size, keep_first}.  A feed-forward: {"kind": "dense", "ff"} or {"kind": "moe", "router": {"experts",
"top"}, "expert": {"ff"}, "shared": {"ff"} or null}.  Every layer carries its own sizes: two layers of one
model may differ in all of them.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional

from .reader import ConfigError, KeyReader


@dataclass(frozen=True)
class BigramConfig:
    buckets: int
    mul_prev: int
    mul_cur: int


@dataclass(frozen=True)
class AttentionMixerConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    v_mix: bool
    window: int
    keep_first: int


@dataclass(frozen=True)
class FeedForwardConfig:
    kind: str                          # "dense" or "moe"
    ff: int                            # inner size (of one expert for "moe")
    experts: int = 0
    top: int = 0
    shared_ff: Optional[int] = None    # inner size of the expert every token uses; None: there is none


@dataclass(frozen=True)
class FobilornLayerConfig:
    type: str
    mixer: AttentionMixerConfig
    mlp: Optional[FeedForwardConfig]


@dataclass(frozen=True)
class FobilornConfig:
    vocab: int
    width: int
    bigram: BigramConfig
    eps: float
    layers: tuple
    architecture: str = "Fobilorn"
    torch_dtype: Optional[str] = None
    raw: dict = field(default_factory=dict, compare=False, repr=False)

    @classmethod
    def from_dict(cls, data: dict) -> "FobilornConfig":
        r = KeyReader(data)
        emb = KeyReader(r.obj("embedding"), "embedding.")
        big = KeyReader(emb.obj("bigram"), "embedding.bigram.")
        bigram = BigramConfig(big.integer("buckets", minimum=1), big.integer("mul_prev", minimum=0),
                              big.integer("mul_cur", minimum=0))
        eps = KeyReader(r.obj("norm"), "norm.").number("eps", positive=True)
        raw_layers = data.get("layers")
        if not isinstance(raw_layers, list) or not raw_layers:
            raise ConfigError("config key 'layers' must be a non-empty list")
        layers = []
        for i, entry in enumerate(raw_layers):
            where = f"layers[{i}]."
            if not isinstance(entry, dict):
                raise ConfigError(f"config key 'layers[{i}]' must be an object")
            lr = KeyReader(entry, where)
            kind = lr.string("type")
            if kind != "attention":
                raise ConfigError(f"config key '{where}type' is {kind!r}; this decoder knows 'attention'")
            m = KeyReader(lr.obj("mixer"), where + "mixer.")
            mask = KeyReader(m.obj("mask"), where + "mixer.mask.")
            mixer = AttentionMixerConfig(
                heads=m.integer("heads", minimum=1), kv_heads=m.integer("kv_heads", minimum=1),
                dim=m.integer("dim", minimum=1), vdim=m.integer("vdim", minimum=1),
                scale=m.number("scale", positive=True), v_mix=m.boolean("v_mix", default=False),
                window=mask.integer("size", minimum=1), keep_first=mask.integer("keep_first", default=0, minimum=0))
            if mixer.heads % mixer.kv_heads:
                raise ConfigError(f"config key '{where}mixer.kv_heads' ({mixer.kv_heads}) must divide 'heads' ({mixer.heads})")
            mlp = None
            f = lr.obj("mlp", default=None)
            if f is not None:
                fr = KeyReader(f, where + "mlp.")
                fkind = fr.string("kind")
                if fkind == "dense":
                    mlp = FeedForwardConfig("dense", fr.integer("ff", minimum=1))
                elif fkind == "moe":
                    router = KeyReader(fr.obj("router"), where + "mlp.router.")
                    experts, top = router.integer("experts", minimum=1), router.integer("top", minimum=1)
                    if top > experts:
                        raise ConfigError(f"config key '{where}mlp.router.top' ({top}) exceeds 'experts' ({experts})")
                    shared = fr.obj("shared", default=None)
                    mlp = FeedForwardConfig(
                        "moe", KeyReader(fr.obj("expert"), where + "mlp.expert.").integer("ff", minimum=1), experts, top,
                        KeyReader(shared, where + "mlp.shared.").integer("ff", minimum=1) if shared is not None else None)
                else:
                    raise ConfigError(f"config key '{where}mlp.kind' is {fkind!r}; this decoder knows 'dense' and 'moe'")
            layers.append(FobilornLayerConfig(kind, mixer, mlp))
        return cls(vocab=r.integer("vocab", minimum=1), width=r.integer("width", minimum=1), bigram=bigram, eps=eps,
                   layers=tuple(layers), architecture=r.string("architecture", default="Fobilorn"),
                   torch_dtype=r.string("torch_dtype", default=None) or r.string("dtype", default=None), raw=dict(data))

    def to_dict(self) -> dict:
        """The config.json content of this configuration."""
        layers = []
        for layer in self.layers:
            m = layer.mixer
            mlp = None
            if layer.mlp is not None and layer.mlp.kind == "dense":
                mlp = {"kind": "dense", "ff": layer.mlp.ff}
            elif layer.mlp is not None:
                mlp = {"kind": "moe", "router": {"experts": layer.mlp.experts, "top": layer.mlp.top},
                       "expert": {"ff": layer.mlp.ff},
                       "shared": {"ff": layer.mlp.shared_ff} if layer.mlp.shared_ff is not None else None}
            layers.append({"type": layer.type, "mlp": mlp,
                           "mixer": {"heads": m.heads, "kv_heads": m.kv_heads, "dim": m.dim, "vdim": m.vdim, "scale": m.scale,
                                     "v_mix": m.v_mix, "mask": {"size": m.window, "keep_first": m.keep_first}}})
        d = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
             "embedding": {"bigram": {"buckets": self.bigram.buckets, "mul_prev": self.bigram.mul_prev,
                                      "mul_cur": self.bigram.mul_cur}},
             "norm": {"eps": self.eps}, "layers": layers}
        if self.torch_dtype:
            d["torch_dtype"] = self.torch_dtype
        return d
