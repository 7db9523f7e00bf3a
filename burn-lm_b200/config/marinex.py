"""The typed configuration of the Marinex decoder, read from its own config.json keys.

    architecture    "Marinex"
    vocab, width    sizes of the token table and of the residual stream
    norm            {"eps"}
    layers          a list; every entry has "type" ("attention" or "latent_attention"), "mixer" (its sizes and
                    constants) and "mlp" ({"kind": "moe", "expert": {"ff"}, "router": {"experts", "top",
                    "groups": {"count", "keep"}}} or null)

An "attention" mixer: heads, kv_heads, dim, vdim, scale, softcap, rot {dims, base}.  A "latent_attention" mixer: heads,
dim, rot_dim, vdim, q_rank, kv_rank, scale, mask {size}, rot {dims, base}.  Every layer carries its own sizes.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional, Union

from .reader import ConfigError, KeyReader


@dataclass(frozen=True)
class AttentionMixerConfig:
    heads: int
    kv_heads: int
    dim: int            # query/key lanes of a head
    vdim: int           # value lanes of a head
    scale: float
    softcap: float
    rot_dims: int       # how many of a head's first lanes turn
    rot_base: float


@dataclass(frozen=True)
class LatentMixerConfig:
    heads: int
    dim: int            # unrotated query/key lanes of a head
    rot_dim: int        # rotated query/key lanes of a head (the key's are shared by the heads)
    vdim: int
    q_rank: int         # lanes of the queries' latent
    kv_rank: int        # lanes of the cached latent
    scale: float
    window: int         # a position sees itself and the window - 1 positions before it
    rot_dims: int
    rot_base: float


@dataclass(frozen=True)
class ExpertsConfig:
    experts: int
    top: int
    ff: int
    groups: int         # the experts form this many equal groups of neighbours
    keep: int           # of which the best `keep` can be chosen from


@dataclass(frozen=True)
class MarinexLayerConfig:
    type: str
    mixer: Union[AttentionMixerConfig, LatentMixerConfig]
    mlp: Optional[ExpertsConfig]


def _rotation(m: KeyReader, where: str, lanes: int):
    rot = KeyReader(m.obj("rot"), where + "rot.")
    dims, base = rot.integer("dims", minimum=0), rot.number("base", positive=True)
    if dims % 2 or dims > lanes:
        raise ConfigError(f"config key '{where}rot.dims' ({dims}) must be even and at most {lanes}")
    return dims, base


@dataclass(frozen=True)
class MarinexConfig:
    vocab: int
    width: int
    eps: float
    layers: tuple
    architecture: str = "Marinex"
    torch_dtype: Optional[str] = None
    raw: dict = field(default_factory=dict, compare=False, repr=False)

    @classmethod
    def from_dict(cls, data: dict) -> "MarinexConfig":
        r = KeyReader(data)
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
            mw = where + "mixer."
            m = KeyReader(lr.obj("mixer"), mw)
            if kind == "attention":
                dim = m.integer("dim", minimum=1)
                dims, base = _rotation(m, mw, dim)
                mixer = AttentionMixerConfig(
                    heads=m.integer("heads", minimum=1), kv_heads=m.integer("kv_heads", minimum=1), dim=dim,
                    vdim=m.integer("vdim", minimum=1), scale=m.number("scale", positive=True),
                    softcap=m.number("softcap", positive=True), rot_dims=dims, rot_base=base)
                if mixer.heads % mixer.kv_heads:
                    raise ConfigError(f"config key '{mw}heads' ({mixer.heads}) must be a multiple of 'kv_heads' ({mixer.kv_heads})")
            elif kind == "latent_attention":
                rot_dim = m.integer("rot_dim", minimum=0)
                dims, base = _rotation(m, mw, rot_dim)
                mixer = LatentMixerConfig(
                    heads=m.integer("heads", minimum=1), dim=m.integer("dim", minimum=1), rot_dim=rot_dim,
                    vdim=m.integer("vdim", minimum=1), q_rank=m.integer("q_rank", minimum=1), kv_rank=m.integer("kv_rank", minimum=1),
                    scale=m.number("scale", positive=True),
                    window=KeyReader(m.obj("mask"), mw + "mask.").integer("size", minimum=1), rot_dims=dims, rot_base=base)
            else:
                raise ConfigError(f"config key '{where}type' is {kind!r}; this decoder knows 'attention' and 'latent_attention'")
            mlp = None
            f = lr.obj("mlp", default=None)
            if f is not None:
                fr = KeyReader(f, where + "mlp.")
                fkind = fr.string("kind")
                if fkind != "moe":
                    raise ConfigError(f"config key '{where}mlp.kind' is {fkind!r}; this decoder knows 'moe'")
                er, rr = KeyReader(fr.obj("expert"), where + "mlp.expert."), KeyReader(fr.obj("router"), where + "mlp.router.")
                gr = KeyReader(rr.obj("groups"), where + "mlp.router.groups.")
                mlp = ExpertsConfig(experts=rr.integer("experts", minimum=1), top=rr.integer("top", minimum=1),
                                    ff=er.integer("ff", minimum=1), groups=gr.integer("count", minimum=1),
                                    keep=gr.integer("keep", minimum=1))
                if mlp.experts % mlp.groups:
                    raise ConfigError(f"config key '{where}mlp.router.groups.count' ({mlp.groups}) must divide 'experts' ({mlp.experts})")
                if mlp.keep > mlp.groups:
                    raise ConfigError(f"config key '{where}mlp.router.groups.keep' ({mlp.keep}) must be at most 'count' ({mlp.groups})")
                if mlp.top > mlp.keep * (mlp.experts // mlp.groups):
                    raise ConfigError(f"config key '{where}mlp.router.top' ({mlp.top}) must be at most the experts of the kept "
                                      f"groups ({mlp.keep * (mlp.experts // mlp.groups)})")
            layers.append(MarinexLayerConfig(kind, mixer, mlp))
        return cls(vocab=r.integer("vocab", minimum=1), width=r.integer("width", minimum=1), eps=eps, layers=tuple(layers),
                   architecture=r.string("architecture", default="Marinex"),
                   torch_dtype=r.string("torch_dtype", default=None) or r.string("dtype", default=None), raw=dict(data))

    def to_dict(self) -> dict:
        """The config.json content of this configuration."""
        layers = []
        for layer in self.layers:
            m = layer.mixer
            rot = {"dims": m.rot_dims, "base": m.rot_base}
            if layer.type == "attention":
                mixer = {"heads": m.heads, "kv_heads": m.kv_heads, "dim": m.dim, "vdim": m.vdim, "scale": m.scale,
                         "softcap": m.softcap, "rot": rot}
            else:
                mixer = {"heads": m.heads, "dim": m.dim, "rot_dim": m.rot_dim, "vdim": m.vdim, "q_rank": m.q_rank,
                         "kv_rank": m.kv_rank, "scale": m.scale, "mask": {"size": m.window}, "rot": rot}
            f = layer.mlp
            layers.append({"type": layer.type, "mixer": mixer,
                           "mlp": {"kind": "moe", "expert": {"ff": f.ff},
                                   "router": {"experts": f.experts, "top": f.top,
                                              "groups": {"count": f.groups, "keep": f.keep}}} if f is not None else None})
        d = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.eps}, "layers": layers}
        if self.torch_dtype:
            d["torch_dtype"] = self.torch_dtype
        return d
