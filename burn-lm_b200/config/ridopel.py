"""The typed configuration of the Ridopel decoder, read from its own config.json keys.

    architecture    "Ridopel"
    vocab, width    sizes of the token table and of the residual stream
    norm            {"eps"}
    canon           {"taps"}: taps of the causal convolution in front of every mixer
    logit_softcap   logits are squashed into (-cap, cap); absent or null: they are not
    loop            {"start", "stop", "times"}: layers start .. stop - 1 run `times` times in a row; absent: no loop
    layers          a list; every entry has "type" ("latent_attention", "hgrn2" or "wkv"), "mixer" (its sizes and
                    constants) and "mlp" ({"kind": "moe", "expert": {"ff", "limit"}, "router": {"experts", "top"}} or null)

A "latent_attention" mixer: heads, dim, rot_dim, vdim, kv_rank, scale, rot {dims, base}.  An "hgrn2" mixer: heads, dim,
vdim.  A "wkv" mixer: heads, dim.  Every layer carries its own sizes.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional, Union

from .reader import ConfigError, KeyReader


@dataclass(frozen=True)
class LatentMixerConfig:
    heads: int
    dim: int            # unrotated query/key lanes of a head
    rot_dim: int        # rotated query/key lanes of a head (the key's are shared by the heads)
    vdim: int
    kv_rank: int
    scale: float
    rot_dims: int       # how many of the rot_dim lanes turn
    rot_base: float


@dataclass(frozen=True)
class Hgrn2MixerConfig:
    heads: int
    dim: int
    vdim: int


@dataclass(frozen=True)
class WkvMixerConfig:
    heads: int
    dim: int


@dataclass(frozen=True)
class ExpertsConfig:
    experts: int
    top: int
    ff: int
    limit: float


@dataclass(frozen=True)
class RidopelLayerConfig:
    type: str
    mixer: Union[LatentMixerConfig, Hgrn2MixerConfig, WkvMixerConfig]
    mlp: Optional[ExpertsConfig]


@dataclass(frozen=True)
class LoopConfig:
    start: int
    stop: int
    times: int


@dataclass(frozen=True)
class RidopelConfig:
    vocab: int
    width: int
    eps: float
    taps: int
    layers: tuple
    loop: Optional[LoopConfig] = None
    logit_softcap: Optional[float] = None
    architecture: str = "Ridopel"
    torch_dtype: Optional[str] = None
    raw: dict = field(default_factory=dict, compare=False, repr=False)

    @classmethod
    def from_dict(cls, data: dict) -> "RidopelConfig":
        r = KeyReader(data)
        eps = KeyReader(r.obj("norm"), "norm.").number("eps", positive=True)
        taps = KeyReader(r.obj("canon"), "canon.").integer("taps", minimum=1)
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
            if kind == "latent_attention":
                rot = KeyReader(m.obj("rot"), where + "mixer.rot.")
                mixer = LatentMixerConfig(
                    heads=m.integer("heads", minimum=1), dim=m.integer("dim", minimum=1), rot_dim=m.integer("rot_dim", minimum=0),
                    vdim=m.integer("vdim", minimum=1), kv_rank=m.integer("kv_rank", minimum=1), scale=m.number("scale", positive=True),
                    rot_dims=rot.integer("dims", minimum=0), rot_base=rot.number("base", positive=True))
                if mixer.rot_dims % 2 or mixer.rot_dims > mixer.rot_dim:
                    raise ConfigError(f"config key '{where}mixer.rot.dims' ({mixer.rot_dims}) must be even and at most "
                                      f"'rot_dim' ({mixer.rot_dim})")
            elif kind == "hgrn2":
                mixer = Hgrn2MixerConfig(heads=m.integer("heads", minimum=1), dim=m.integer("dim", minimum=1),
                                         vdim=m.integer("vdim", minimum=1))
            elif kind == "wkv":
                mixer = WkvMixerConfig(heads=m.integer("heads", minimum=1), dim=m.integer("dim", minimum=1))
            else:
                raise ConfigError(f"config key '{where}type' is {kind!r}; this decoder knows 'latent_attention', 'hgrn2' and 'wkv'")
            mlp = None
            f = lr.obj("mlp", default=None)
            if f is not None:
                fr = KeyReader(f, where + "mlp.")
                fkind = fr.string("kind")
                if fkind != "moe":
                    raise ConfigError(f"config key '{where}mlp.kind' is {fkind!r}; this decoder knows 'moe'")
                er, rr = KeyReader(fr.obj("expert"), where + "mlp.expert."), KeyReader(fr.obj("router"), where + "mlp.router.")
                mlp = ExpertsConfig(experts=rr.integer("experts", minimum=1), top=rr.integer("top", minimum=1),
                                    ff=er.integer("ff", minimum=1), limit=er.number("limit", positive=True))
                if mlp.top > mlp.experts:
                    raise ConfigError(f"config key '{where}mlp.router.top' ({mlp.top}) must be at most 'experts' ({mlp.experts})")
            layers.append(RidopelLayerConfig(kind, mixer, mlp))
        loop = None
        lp = r.obj("loop", default=None)
        if lp is not None:
            lo = KeyReader(lp, "loop.")
            loop = LoopConfig(lo.integer("start", minimum=0), lo.integer("stop", minimum=0), lo.integer("times", minimum=1))
            if not loop.start <= loop.stop <= len(layers):
                raise ConfigError(f"config key 'loop': layers {loop.start} .. {loop.stop} - 1 of {len(layers)}")
        cap = r.number("logit_softcap", default=None, positive=True)
        return cls(vocab=r.integer("vocab", minimum=1), width=r.integer("width", minimum=1), eps=eps, taps=taps,
                   layers=tuple(layers), loop=loop, logit_softcap=cap, architecture=r.string("architecture", default="Ridopel"),
                   torch_dtype=r.string("torch_dtype", default=None) or r.string("dtype", default=None), raw=dict(data))

    def to_dict(self) -> dict:
        """The config.json content of this configuration."""
        layers = []
        for layer in self.layers:
            m = layer.mixer
            if layer.type == "latent_attention":
                mixer = {"heads": m.heads, "dim": m.dim, "rot_dim": m.rot_dim, "vdim": m.vdim, "kv_rank": m.kv_rank, "scale": m.scale,
                         "rot": {"dims": m.rot_dims, "base": m.rot_base}}
            elif layer.type == "hgrn2":
                mixer = {"heads": m.heads, "dim": m.dim, "vdim": m.vdim}
            else:
                mixer = {"heads": m.heads, "dim": m.dim}
            f = layer.mlp
            layers.append({"type": layer.type, "mixer": mixer,
                           "mlp": {"kind": "moe", "expert": {"ff": f.ff, "limit": f.limit},
                                   "router": {"experts": f.experts, "top": f.top}} if f is not None else None})
        d = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.eps},
             "canon": {"taps": self.taps}, "layers": layers}
        if self.loop is not None:
            d["loop"] = {"start": self.loop.start, "stop": self.loop.stop, "times": self.loop.times}
        if self.logit_softcap is not None:
            d["logit_softcap"] = self.logit_softcap
        if self.torch_dtype:
            d["torch_dtype"] = self.torch_dtype
        return d
