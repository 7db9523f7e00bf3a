"""The Ridopel decoder as a plan of parts: the registry entry "Ridopel".

A token embedding that is RMS-normed; pre-norm layers whose mixer reads its normed input through a short causal
convolution with the input itself added (block "prenorm_filtered"); a mixer per layer that is attention over a cached
latent with a shared rotated key part and an output gate, HGRN2 (linear attention written through its forget gate), or
WKV (token-shifted linear attention with a decay per token and key channel); a mixture of experts with softmax scores, a
correction of the choice, renormalised weights and a clamped gated unit, or no feed-forward; a last RMS norm, the output
projection, and logits squashed by a tanh cap.  A span of the layers may run several times in a row with the same
weights, every pass with a cache line or state of its own, and before each pass the stream is rewritten from itself and
the embedding's output (stream part "concat_projection").  Every layer brings its own sizes.  Stored names: 'embed',
'embed.norm', 'loop.in', 'l<i>.norm1', 'l<i>.norm2', 'l<i>.canon1', 'l<i>.mix.*', 'l<i>.mlp.*', 'final.norm', 'head'.
"""
from __future__ import annotations

from ..config.ridopel import RidopelConfig
from ..parts.embedding import CappedHeadSpec, NormedEmbeddingSpec
from ..parts.filter import ShortConvSpec
from ..parts.hgrn2 import Hgrn2Spec
from ..parts.latent_attention import LatentAttentionSpec
from ..parts.moe import RoutedMoESpec
from ..parts.norm import RMSNormSpec
from ..parts.stream import ConcatProjectionSpec
from ..parts.wkv import WkvSpec
from ..plan import LayerPlan, ModelPlan, NamedPart, PartPlan, ScheduleEntry
from ..registry import Architecture, register_architecture

MAX_POSITIONS = 1 << 20     # the rotation takes any position; the cache sets the real limit
EXPERT_ALPHA = 1.702        # the slope inside the experts' gate, fixed by the design


def _mixer(width: int, eps: float, kind: str, m, p: str) -> PartPlan:
    a = p + "mix."
    if kind == "latent_attention":
        return PartPlan("latent_attention", LatentAttentionSpec(
            hidden_size=width, n_heads=m.heads, key_dim=m.dim, rot_dim=m.rot_dim, value_dim=m.vdim, rank=m.kv_rank, scale=m.scale,
            rotary_dims=m.rot_dims, rotary_base=m.rot_base, eps=eps, output_gate=True),
            {"q": a + "q", "dkv": a + "dkv", "c_norm": a + "dkv.norm", "uk": a + "uk", "uv": a + "uv", "g": a + "g", "o": a + "o"})
    if kind == "hgrn2":
        return PartPlan("hgrn2", Hgrn2Spec(hidden_size=width, n_heads=m.heads, key_dim=m.dim, value_dim=m.vdim, eps=eps),
                        {"q": a + "q", "f": a + "f", "f_bias": a + "f.b", "lower": a + "lower", "v": a + "v", "norm": a + "norm",
                         "o": a + "o"})
    tensors = {"mu_" + s: a + "mu." + s for s in "rkvgw"}
    tensors.update({s: a + s for s in ("r", "k", "v", "g", "w1", "w2", "w0", "u", "norm", "o")})
    return PartPlan("wkv", WkvSpec(hidden_size=width, n_heads=m.heads, head_dim=m.dim, eps=eps), tensors)


def run_order(n_layers: int, loop) -> list:
    """[(layer, whether a pass of the loop starts with this run)]: the looped span `times` times in a row, the rest once."""
    if loop is None:
        return [(i, False) for i in range(n_layers)]
    order = [(i, False) for i in range(loop.start)]
    for _ in range(loop.times):
        order += [(i, i == loop.start) for i in range(loop.start, loop.stop)]
    return order + [(i, False) for i in range(loop.stop, n_layers)]


def ridopel_plan(cfg: RidopelConfig) -> ModelPlan:
    width, eps = cfg.width, cfg.eps
    norm = lambda name: PartPlan("rmsnorm", RMSNormSpec(width, eps), {"weight": name})
    layers = []
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        parts = [NamedPart("mixer_norm", "norm", norm(p + "norm1")),
                 NamedPart("input_filter", "filter", PartPlan("short_conv", ShortConvSpec(width, cfg.taps, residual=True),
                                                              {"taps": p + "canon1"})),
                 NamedPart("mixer", "mixer", _mixer(width, eps, layer.type, layer.mixer, p))]
        f = layer.mlp
        if f is not None:
            parts += [NamedPart("feed_forward_norm", "norm", norm(p + "norm2")),
                      NamedPart("feed_forward", "feed_forward", PartPlan(
                          "routed_moe", RoutedMoESpec(width, f.experts, f.top, f.ff, scores="softmax", correction=True,
                                                      renormalise=True, clamp_limit=f.limit, clamp_alpha=EXPERT_ALPHA),
                          {"router": p + "mlp.router", "correction": p + "mlp.correction", "gate": p + "mlp.e{}.gate",
                           "up": p + "mlp.e{}.up", "down": p + "mlp.e{}.down"}))]
        layers.append(LayerPlan("prenorm_filtered", tuple(parts)))
    stream_parts = ()
    if cfg.loop is not None:
        stream_parts = (PartPlan("concat_projection", ConcatProjectionSpec(width), {"weight": "loop.in"}),)
    return ModelPlan(
        architecture=cfg.architecture,
        vocab_size=cfg.vocab,
        hidden_size=width,
        embedding=PartPlan("normed_table", NormedEmbeddingSpec(cfg.vocab, width, eps), {"table": "embed", "norm": "embed.norm"}),
        layers=tuple(layers),
        schedule=tuple(ScheduleEntry(i, before=0 if first else None) for i, first in run_order(len(layers), cfg.loop)),
        final_norm=norm("final.norm"),
        head=PartPlan("capped_linear", CappedHeadSpec(cfg.vocab, width, cfg.logit_softcap), {"weight": "head"}),
        max_positions=MAX_POSITIONS,
        stream_parts=stream_parts,
        ignorable_tensors=(r"loop\.in",) if cfg.loop is None else (),
    )


RIDOPEL = register_architecture(Architecture(
    name="Ridopel", config_class=RidopelConfig, plan=ridopel_plan, aliases=("ridopel",),
    description="pre-norm layers behind a short input convolution: latent attention, HGRN2 or WKV; softmax-routed experts "
                "with a clamped unit; a looped span of layers fed the embedding again; capped logits"))
