"""The typed configuration of the Nufolix decoder, read from its own config.json keys.

    architecture    "Nufolix"
    vocab, width    sizes of the token table and of the residual stream
    embedding       {"scale"}: what a token's row is multiplied by
    norm            {"eps"}
    residual_mult   what a sublayer's normed output is multiplied by before it joins the stream
    layers          a list; every entry has "type" ("mamba2" or "parallel"), "mixer" (its sizes and constants) and "mlp"
                    ({"kind": "dense", "ff"} or null)

A "mamba2" mixer: heads, vdim, state, groups, conv, norm_groups.  A "parallel" mixer: left {heads, kv_heads, dim, vdim,
scale, softcap, rot {dims, base}}, right {heads, kv_heads, dim, vdim, conv}, left_scale, right_scale.  Every layer
carries its own sizes.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional, Union

from .reader import ConfigError, KeyReader


@dataclass(frozen=True)
class Mamba2MixerConfig:
    heads: int
    vdim: int
    state: int
    groups: int
    conv: int
    norm_groups: int


@dataclass(frozen=True)
class LeftMixerConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    softcap: float
    rot_dims: int
    rot_base: float


@dataclass(frozen=True)
class RightMixerConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int


@dataclass(frozen=True)
class ParallelMixerConfig:
    left: LeftMixerConfig
    right: RightMixerConfig
    left_scale: float
    right_scale: float


@dataclass(frozen=True)
class NufolixLayerConfig:
    type: str
    mixer: Union[Mamba2MixerConfig, ParallelMixerConfig]
    ff: Optional[int]                  # inner size of the dense feed-forward; None: the layer has none


def _divides(where, small_key, small, big_key, big):
    if big % small:
        raise ConfigError(f"config key '{where}{small_key}' ({small}) must divide '{big_key}' ({big})")


@dataclass(frozen=True)
class NufolixConfig:
    vocab: int
    width: int
    embedding_scale: float
    eps: float
    residual_mult: float
    layers: tuple
    architecture: str = "Nufolix"
    torch_dtype: Optional[str] = None
    raw: dict = field(default_factory=dict, compare=False, repr=False)

    @classmethod
    def from_dict(cls, data: dict) -> "NufolixConfig":
        r = KeyReader(data)
        scale = KeyReader(r.obj("embedding"), "embedding.").number("scale")
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
            m = KeyReader(lr.obj("mixer"), where + "mixer.")
            if kind == "mamba2":
                mixer = Mamba2MixerConfig(
                    heads=m.integer("heads", minimum=1), vdim=m.integer("vdim", minimum=1), state=m.integer("state", minimum=1),
                    groups=m.integer("groups", minimum=1), conv=m.integer("conv", minimum=1),
                    norm_groups=m.integer("norm_groups", minimum=1))
                _divides(where + "mixer.", "groups", mixer.groups, "heads", mixer.heads)
                _divides(where + "mixer.", "norm_groups", mixer.norm_groups, "heads * vdim", mixer.heads * mixer.vdim)
            elif kind == "parallel":
                lw, rw = where + "mixer.left.", where + "mixer.right."
                lt, rt = KeyReader(m.obj("left"), lw), KeyReader(m.obj("right"), rw)
                rot = KeyReader(lt.obj("rot"), lw + "rot.")
                left = LeftMixerConfig(
                    heads=lt.integer("heads", minimum=1), kv_heads=lt.integer("kv_heads", minimum=1), dim=lt.integer("dim", minimum=1),
                    vdim=lt.integer("vdim", minimum=1), scale=lt.number("scale", positive=True),
                    softcap=lt.number("softcap", positive=True), rot_dims=rot.integer("dims", minimum=0),
                    rot_base=rot.number("base", positive=True))
                _divides(lw, "kv_heads", left.kv_heads, "heads", left.heads)
                if left.rot_dims % 2 or left.rot_dims > left.dim:
                    raise ConfigError(f"config key '{lw}rot.dims' ({left.rot_dims}) must be even and at most 'dim' ({left.dim})")
                right = RightMixerConfig(
                    heads=rt.integer("heads", minimum=1), kv_heads=rt.integer("kv_heads", minimum=1), dim=rt.integer("dim", minimum=1),
                    vdim=rt.integer("vdim", minimum=1), conv=rt.integer("conv", minimum=1))
                _divides(rw, "kv_heads", right.kv_heads, "heads", right.heads)
                mixer = ParallelMixerConfig(left, right, m.number("left_scale"), m.number("right_scale"))
            else:
                raise ConfigError(f"config key '{where}type' is {kind!r}; this decoder knows 'mamba2' and 'parallel'")
            ff = None
            f = lr.obj("mlp", default=None)
            if f is not None:
                fr = KeyReader(f, where + "mlp.")
                fkind = fr.string("kind")
                if fkind != "dense":
                    raise ConfigError(f"config key '{where}mlp.kind' is {fkind!r}; this decoder knows 'dense'")
                ff = fr.integer("ff", minimum=1)
            layers.append(NufolixLayerConfig(kind, mixer, ff))
        return cls(vocab=r.integer("vocab", minimum=1), width=r.integer("width", minimum=1), embedding_scale=scale, eps=eps,
                   residual_mult=r.number("residual_mult"), layers=tuple(layers),
                   architecture=r.string("architecture", default="Nufolix"),
                   torch_dtype=r.string("torch_dtype", default=None) or r.string("dtype", default=None), raw=dict(data))

    def to_dict(self) -> dict:
        """The config.json content of this configuration."""
        layers = []
        for layer in self.layers:
            m = layer.mixer
            if layer.type == "mamba2":
                mixer = {"heads": m.heads, "vdim": m.vdim, "state": m.state, "groups": m.groups, "conv": m.conv,
                         "norm_groups": m.norm_groups}
            else:
                lf, rg = m.left, m.right
                mixer = {"left": {"heads": lf.heads, "kv_heads": lf.kv_heads, "dim": lf.dim, "vdim": lf.vdim, "scale": lf.scale,
                                  "softcap": lf.softcap, "rot": {"dims": lf.rot_dims, "base": lf.rot_base}},
                         "right": {"heads": rg.heads, "kv_heads": rg.kv_heads, "dim": rg.dim, "vdim": rg.vdim, "conv": rg.conv},
                         "left_scale": m.left_scale, "right_scale": m.right_scale}
            layers.append({"type": layer.type, "mixer": mixer,
                           "mlp": {"kind": "dense", "ff": layer.ff} if layer.ff is not None else None})
        d = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
             "embedding": {"scale": self.embedding_scale}, "norm": {"eps": self.eps}, "residual_mult": self.residual_mult,
             "layers": layers}
        if self.torch_dtype:
            d["torch_dtype"] = self.torch_dtype
        return d
