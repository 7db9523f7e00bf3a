"""The Marinex decoder as a plan of parts: the registry entry "Marinex".

A token embedding; layers whose sublayers read the residual stream itself and whose outputs are RMS-normed before
they join it (block "postnorm"): x <- x + norm1(mixer(x)), then x <- x + norm2(feed_forward(x)); a mixer per layer
that is grouped-query attention with normed heads, a number per head on the scores, capped scores and a sink of
score 0 (mixer "normed_attention"), or attention over a cached latent with a latent for the queries as well, a
window, a learned sink and a gate per head (mixer "latent_attention"); a mixture of experts without gates
(W_down gelu(W_up h)) whose sigmoid router chooses among the experts of the best groups, or no feed-forward; a last
RMS norm and the output projection.  Every layer brings its own sizes.  Stored names: 'embed', 'l<i>.norm1',
'l<i>.norm2', 'l<i>.mix.*', 'l<i>.mlp.*', 'final.norm', 'head'.
"""
from __future__ import annotations

from ..config.marinex import MarinexConfig
from ..parts.embedding import EmbeddingSpec, HeadSpec
from ..parts.latent_attention import LatentAttentionSpec
from ..parts.moe import RoutedMoESpec
from ..parts.norm import PostRMSNormSpec, RMSNormSpec
from ..parts.normed_attention import NormedAttentionSpec
from ..plan import LayerPlan, ModelPlan, NamedPart, PartPlan, ScheduleEntry
from ..registry import Architecture, register_architecture

MAX_POSITIONS = 1 << 20     # the rotation takes any position; the cache sets the real limit


def _mixer(width: int, eps: float, kind: str, m, p: str) -> PartPlan:
    a = p + "mix."
    if kind == "attention":
        return PartPlan("normed_attention", NormedAttentionSpec(
            hidden_size=width, n_heads=m.heads, n_kv_heads=m.kv_heads, head_dim=m.dim, value_dim=m.vdim, scale=m.scale, eps=eps,
            rotary_dims=m.rot_dims, rotary_base=m.rot_base, rotary_halves=False, qk_norm=True, value_norm=True,
            head_temperature=True, softcap=m.softcap, sink=True, window=None),
            {"q": a + "q", "k": a + "k", "v": a + "v", "o": a + "o", "q_norm": a + "q.norm", "k_norm": a + "k.norm",
             "temperature": a + "temp"})
    return PartPlan("latent_attention", LatentAttentionSpec(
        hidden_size=width, n_heads=m.heads, key_dim=m.dim, rot_dim=m.rot_dim, value_dim=m.vdim, rank=m.kv_rank, scale=m.scale,
        rotary_dims=m.rot_dims, rotary_base=m.rot_base, eps=eps, output_gate=True, q_rank=m.q_rank, rotary_halves=True,
        window=m.window, sink=True, gate_per_head=True),
        {"dq": a + "dq", "q_norm": a + "dq.norm", "uq": a + "uq", "dkv": a + "dkv", "c_norm": a + "dkv.norm", "uk": a + "uk",
         "uv": a + "uv", "g": a + "g", "o": a + "o", "sink": a + "sink"})


def marinex_plan(cfg: MarinexConfig) -> ModelPlan:
    width, eps = cfg.width, cfg.eps
    post = lambda name: PartPlan("rms_post", PostRMSNormSpec(width, eps), {"weight": name})
    layers = []
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        parts = [NamedPart("mixer", "mixer", _mixer(width, eps, layer.type, layer.mixer, p)),
                 NamedPart("mixer_post_norm", "norm", post(p + "norm1"))]
        f = layer.mlp
        if f is not None:
            parts += [NamedPart("feed_forward", "feed_forward", PartPlan(
                "routed_moe", RoutedMoESpec(width, f.experts, f.top, f.ff, scores="sigmoid", correction=True, renormalise=False,
                                            n_groups=f.groups, keep_groups=f.keep, unit="gelu"),
                {"router": p + "mlp.router", "correction": p + "mlp.correction", "up": p + "mlp.e{}.up",
                 "down": p + "mlp.e{}.down"})),
                NamedPart("feed_forward_post_norm", "norm", post(p + "norm2"))]
        layers.append(LayerPlan("postnorm", tuple(parts)))
    return ModelPlan(
        architecture=cfg.architecture,
        vocab_size=cfg.vocab,
        hidden_size=width,
        embedding=PartPlan("table", EmbeddingSpec(cfg.vocab, width), {"table": "embed"}),
        layers=tuple(layers),
        schedule=tuple(ScheduleEntry(i) for i in range(len(layers))),
        final_norm=PartPlan("rmsnorm", RMSNormSpec(width, eps), {"weight": "final.norm"}),
        head=PartPlan("linear", HeadSpec(cfg.vocab, width), {"weight": "head"}),
        max_positions=MAX_POSITIONS,
    )


MARINEX = register_architecture(Architecture(
    name="Marinex", config_class=MarinexConfig, plan=marinex_plan, aliases=("marinex",),
    description="layers normed behind their sublayers: grouped-query attention with normed heads, capped scores and a sink, "
                "or windowed latent attention with a learned sink; ungated experts chosen among the best groups"))
