"""How a layer's parts stand around the residual stream: one after the other behind norms of their own
(pre-norm), or side by side behind one norm (parallel).

Pre-norm: h = x + mixer(norm(x)); out = h + feed_forward(norm(h))
(crates/burn-lm-llama/src/nn/transformer.rs:241-256).  The residual stream is fp32; a part's
output is added into it by the next norm's fused kernel, so a block takes the pending output of
the block before it (`delta`) and returns its own.
"""
from __future__ import annotations

from .. import kernels as K
from ..registry import register_part
from .linear import NormHandoff


def _add_norm(norm, resid, delta, lazy, handoff):
    if getattr(norm, "takes_handed_norm", False):
        return norm.add_norm(resid, delta, lazy=lazy, handoff=handoff)
    return norm.add_norm(resid, delta, lazy=lazy)


@register_part("block", "prenorm")
class PreNormBlock:
    family = "block"
    graph_safe = True     # it only calls its parts: a step of graph-safe parts can be captured

    NAMES = ("mixer_norm", "mixer", "feed_forward_norm", "feed_forward")

    def __init__(self, parts: dict):
        if set(parts) != set(self.NAMES):
            raise ValueError(f"the prenorm block arranges parts named {self.NAMES}; the layer has {sorted(parts)}")
        self.mixer_norm, self.mixer = parts["mixer_norm"], parts["mixer"]
        self.feed_forward_norm, self.feed_forward = parts["feed_forward_norm"], parts["feed_forward"]

    def first_norm(self):
        """The norm that reads the stream first in this block: the block before may prepare its input."""
        return self.mixer_norm

    def forward(self, resid, delta, step, cache_view, next_norm=None):
        # Two optional abilities of a mixer or feed-forward shorten the path: `takes_pending_norm`
        # (its first product normalises on the fly) and `adds_to_stream` (its last product adds its
        # result into the residual stream itself and returns None).  A part that adds into the stream
        # is told, through the step's handoff, which norm reads the stream next (`next_norm` after this
        # block), and may leave that norm's input beside its sum.
        mixer, ff = self.mixer, self.feed_forward
        if step.handoff is None:
            step.handoff = NormHandoff()
        handoff = step.handoff
        x = _add_norm(self.mixer_norm, resid, delta, getattr(mixer, "takes_pending_norm", False), handoff)
        if getattr(mixer, "adds_to_stream", False):
            handoff.expect(self.feed_forward_norm)
            a = mixer.forward(x, step, cache_view, stream=resid)
        else:
            a = mixer.forward(x, step, cache_view)
        x = _add_norm(self.feed_forward_norm, resid, a, getattr(ff, "takes_pending_norm", False), handoff)
        if getattr(ff, "adds_to_stream", False):
            handoff.expect(next_norm)
            return ff.forward(x, step, stream=resid)
        return ff.forward(x, step)


@register_part("block", "parallel")
class ParallelBlock:
    """h = norm(x); x <- x + (mixer(h) + feed_forward(h)): one norm, and both parts read its output.  The layer
    may have no feed-forward.  What the parts return is handed, as a tuple, to the norm that reads the stream next
    when that norm adds several outputs at once (`takes_several`); else it is added into the stream here."""
    family = "block"
    graph_safe = True

    NAMES = ("norm", "mixer", "feed_forward")

    def __init__(self, parts: dict):
        if not {"norm", "mixer"} <= set(parts) <= set(self.NAMES):
            raise ValueError(f"the parallel block arranges parts named {self.NAMES} (the last may be absent); the layer has {sorted(parts)}")
        self.norm, self.mixer, self.feed_forward = parts["norm"], parts["mixer"], parts.get("feed_forward")

    def first_norm(self):
        return self.norm

    def forward(self, resid, delta, step, cache_view, next_norm=None):
        if getattr(step, "handoff", None) is not None:
            step.handoff.expect(None)          # no product of this block prepares a norm's input
        h = self.norm.add_norm(resid, delta)
        if not isinstance(h, type(resid)):
            h = h.materialize()                # both parts read it
        pending = []
        mixer, ff = self.mixer, self.feed_forward
        a = mixer.forward(h, step, cache_view, stream=resid) if getattr(mixer, "adds_to_stream", False) else mixer.forward(h, step, cache_view)
        if a is not None:
            pending.append(a)
        if ff is not None:
            f = ff.forward(h, step, stream=resid) if getattr(ff, "adds_to_stream", False) else ff.forward(h, step)
            if f is not None:
                pending.append(f)
        if not pending:
            return None
        if len(pending) == 1:
            return pending[0]
        if getattr(next_norm, "takes_several", False):
            return tuple(pending)
        K.add_dyt(resid, pending, None, None, None, None)     # only the sum into the stream
        return None


@register_part("block", "sandwich")
class SandwichBlock:
    """Norms before and behind each sublayer: x <- x + m * post1(mixer(pre1(x))), then x <- x + m * post2(ff(pre2(x))); the
    multiplier m belongs to the norms behind (norm kind "rms_post").  A layer may have no feed-forward.  The norm behind a
    sublayer is not run by itself: its input travels as a pending output (parts.norm.PostNormed) to the norm that reads
    the stream next (the next sublayer's, the next block's, or the model's last), whose kernel norms it, adds it and
    norms the sum."""
    family = "block"
    graph_safe = True

    NAMES = ("mixer_norm", "mixer", "mixer_post_norm", "feed_forward_norm", "feed_forward", "feed_forward_post_norm")

    def __init__(self, parts: dict):
        if not set(self.NAMES[:3]) <= set(parts) <= set(self.NAMES) or len(parts) not in (3, 6):
            raise ValueError(f"the sandwich block arranges parts named {self.NAMES} (the last three may be absent); the layer has {sorted(parts)}")
        self.mixer_norm, self.mixer, self.mixer_post = parts["mixer_norm"], parts["mixer"], parts["mixer_post_norm"]
        self.ff_norm, self.ff, self.ff_post = (parts.get("feed_forward_norm"), parts.get("feed_forward"),
                                               parts.get("feed_forward_post_norm"))
        for norm in (self.mixer_norm, self.ff_norm):
            if norm is not None and not getattr(norm, "takes_post_normed", False):
                raise ValueError("the norms in front of a sandwich block's sublayers must take a pending normed output")

    def first_norm(self):
        return self.mixer_norm

    @staticmethod
    def _pending(post, result):
        """A sublayer returns its output; or (output, bias) when its last product's bias is still to be added; or a
        parts.parallel_mixers.WeightedPair when it is a weighted sum of two outputs that is still to be taken."""
        if isinstance(result, tuple):
            return post.pending(result[0], result[1])
        if hasattr(result, "scale_a"):
            return post.pending(result.a, second=(result.scale_a, result.b, result.scale_b))
        return post.pending(result)

    def forward(self, resid, delta, step, cache_view, next_norm=None):
        if getattr(step, "handoff", None) is not None:
            step.handoff.expect(None)          # no product of this block prepares a norm's input
        h = self.mixer_norm.add_norm(resid, delta)
        if getattr(self.mixer, "gives_pairs", False):      # two mixers side by side: the norm's kernel takes their weighted sum
            pending = self._pending(self.mixer_post, self.mixer.forward(h, step, cache_view, as_pair=True))
        else:
            pending = self._pending(self.mixer_post, self.mixer.forward(h, step, cache_view))
        if self.ff is not None:
            h = self.ff_norm.add_norm(resid, pending)
            pending = self._pending(self.ff_post, self.ff.forward(h, step))
        if getattr(next_norm, "takes_post_normed", False):
            return pending
        self.mixer_post.add(resid, pending)
        return None


@register_part("block", "prenorm_filtered")
class FilteredPreNormBlock:
    """The pre-norm block with a filter over time between the first norm and the mixer: h = filter(norm1(x));
    x <- x + mixer(h); x <- x + feed_forward(norm2(x)).  The layer may have no feed-forward.  The norm hands its rows on
    unrounded (float32); the filter (family "filter") returns them filtered, in float32 and in the compute dtype, and the
    mixer reads the one it asks for (`takes_float32_input`).  What the filter carries per sequence lies at the start of
    the run's state block; a mixer with a state of its own finds it behind that (`state_offset` of its view), and a mixer
    that keeps keys gets a state block beside its pages."""
    family = "block"
    graph_safe = True

    NAMES = ("mixer_norm", "input_filter", "mixer", "feed_forward_norm", "feed_forward")

    def __init__(self, parts: dict):
        if not set(self.NAMES[:3]) <= set(parts) <= set(self.NAMES) or len(parts) not in (3, 5):
            raise ValueError(f"the filtered pre-norm block arranges parts named {self.NAMES} (the last two may be absent); "
                             f"the layer has {sorted(parts)}")
        self.mixer_norm, self.filter, self.mixer = parts["mixer_norm"], parts["input_filter"], parts["mixer"]
        self.feed_forward_norm, self.feed_forward = parts.get("feed_forward_norm"), parts.get("feed_forward")
        self.kernel_modules = ("elementwise",)

    def first_norm(self):
        return self.mixer_norm

    def cache_need(self):
        from .base import CacheNeed
        own = self.filter.state_floats()
        need = self.mixer.cache_need()
        needs = list(need) if isinstance(need, tuple) else [need]
        states = [n for n in needs if n.kind == "state"]
        if len(states) > 1:
            raise ValueError("a mixer behind a filter keeps at most one state block")
        if states:
            st = states[0]
            if len(st.state_shape) != 2 or st.state_shape[0] != 2 or st.state_dtype != "float32":
                raise ValueError("a mixer behind a filter keeps its state as two float32 copies")
            merged = CacheNeed("state", state_shape=(2, own + st.state_shape[1]))
            rest = [n for n in needs if n.kind not in ("state", "none")]
            return tuple(rest + [merged]) if rest else merged
        rest = [n for n in needs if n.kind != "none"]
        mine = CacheNeed("state", state_shape=(2, own))
        return tuple(rest + [mine]) if rest else mine

    def forward(self, resid, delta, step, cache_view, next_norm=None):
        import dataclasses

        import torch
        if getattr(step, "handoff", None) is not None:
            step.handoff.expect(None)          # no product of this block prepares a norm's input
        h = self.mixer_norm.add_norm(resid, delta, out_dtype=torch.float32)
        wide, rounded = self.filter.forward(h, step, cache_view.state, 0)
        view = dataclasses.replace(cache_view, state_offset=self.filter.state_floats())
        x = wide if getattr(self.mixer, "takes_float32_input", False) else rounded
        a = self.mixer.forward(x, step, view)
        if self.feed_forward is None:
            return a
        x = self.feed_forward_norm.add_norm(resid, a)
        return self.feed_forward.forward(x, step)


class _StreamReader:
    """What stands where a block's first norm would: the block reads the stream itself, and the kernel that hands it
    the stream's rows can first norm, scale and add a pending sublayer output (parts.norm.PostNormed)."""
    takes_post_normed = True


@register_part("block", "postnorm")
class PostNormBlock:
    """Norms behind the sublayers only: x <- x + post1(mixer(x)), then x <- x + post2(feed_forward(x)).  Both sublayers
    read the stream itself, not a normed copy; what they return is RMS-normed (norm kind "rms_post") before it joins the
    stream.  A layer may have no feed-forward.  The norm behind a sublayer is not run by itself: its input travels as a
    pending output to whoever reads the stream next, whose kernel norms it, adds it (fp32) and hands the sum on: here the
    kernel that gives the next sublayer its rows in the compute dtype (in the 32-bit path the sublayer reads the stream's
    own rows), else the next block's first norm or the model's last."""
    family = "block"
    graph_safe = True
    kernel_modules = ("stream_ops",)

    NAMES = ("mixer", "mixer_post_norm", "feed_forward", "feed_forward_post_norm")

    def __init__(self, parts: dict):
        if not set(self.NAMES[:2]) <= set(parts) <= set(self.NAMES) or len(parts) not in (2, 4):
            raise ValueError(f"the postnorm block arranges parts named {self.NAMES} (the last two may be absent); the layer has {sorted(parts)}")
        self.mixer, self.mixer_post = parts["mixer"], parts["mixer_post_norm"]
        self.ff, self.ff_post = parts.get("feed_forward"), parts.get("feed_forward_post_norm")
        self.reader = _StreamReader()

    def first_norm(self):
        return self.reader

    def _read(self, resid, delta):
        """The stream's rows for a sublayer, after `delta` (None, a plain output, or a pending normed one) has joined them."""
        import torch

        from .norm import PostNormed, PostRMSNorm
        dtype = self.mixer.runtime.dtype
        if isinstance(delta, PostNormed):
            if dtype == torch.float32:
                PostRMSNorm.add(resid, delta)
                return resid
            out = torch.empty(resid.shape, dtype=dtype, device=resid.device)
            K.sandwich_norm(resid, delta.output, delta.weight, delta.mult, delta.eps, None, 0.0, out, delta_bias=delta.bias,
                            second=delta.second)
            return out
        if delta is None and dtype == torch.float32:
            return resid
        out = torch.empty(resid.shape, dtype=dtype, device=resid.device)
        K.pack_cols(resid, delta, out, 0)
        return out

    def forward(self, resid, delta, step, cache_view, next_norm=None):
        if getattr(step, "handoff", None) is not None:
            step.handoff.expect(None)          # no product of this block prepares a norm's input
        x = self._read(resid, delta)
        pending = SandwichBlock._pending(self.mixer_post, self.mixer.forward(x, step, cache_view))
        if self.ff is not None:
            x = self._read(resid, pending)
            pending = SandwichBlock._pending(self.ff_post, self.ff.forward(x, step))
        if getattr(next_norm, "takes_post_normed", False):
            return pending
        self.mixer_post.add(resid, pending)
        return None
