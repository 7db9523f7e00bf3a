"""Norms fused with the residual add: RMS norm, Dynamic Tanh (which takes no statistics), and the RMS norm that
stands behind a sublayer and scales what it adds to the stream.

y = x / sqrt(mean(x^2) + eps) * gamma; it stands before the mixer, before the feed-forward and once
after the last block (crates/burn-lm-llama/src/nn/transformer.rs:248-255,101; eps at :60-62 and
:211-216).  The sum of squares, the root and the product with gamma are fp32 in both paths.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from .. import kernels as K
from ..registry import register_part
from ..weights.loader import TensorSpec
from .base import Part
from .linear import NormedStream


@dataclass(frozen=True)
class RMSNormSpec:
    size: int
    eps: float


@dataclass
class PostNormed:
    """A sublayer's raw output that is still to be normed, scaled and added to the stream:
    stream += mult * (output (+ bias)) / rms(output (+ bias)) * weight.  The norm that reads the stream next does it in
    its own kernel (a norm with `takes_post_normed`), or `PostRMSNorm.add` does it alone."""
    output: torch.Tensor          # [N, D] float32 or the compute dtype
    weight: torch.Tensor          # float32 [D]
    eps: float
    mult: float
    bias: Optional[torch.Tensor] = None     # float32 [D]: a bias of the sublayer's last product, not added yet
    second: Optional[tuple] = None          # (scale_a, output_b, scale_b): the sublayer's output is scale_a * output +
                                            # scale_b * output_b (two mixers side by side), summed by the same kernel


@register_part("norm", "rmsnorm")
class RMSNorm(Part):
    family = "norm"
    graph_safe = True
    roles = ("weight",)

    def tensor_specs(self):
        return [TensorSpec(self.tensor_names["weight"], (self.spec.size,), init="one_plus_normal:0.1")]

    def bind(self, loaded):
        self.gamma = loaded[self.tensor_names["weight"]]

    takes_handed_norm = True      # a product that writes the stream may leave this norm's input (parts.linear.NormHandoff)
    takes_post_normed = True      # `delta` may be a PostNormed: normed, scaled and added by this norm's kernel

    def add_norm(self, resid, delta, rows=None, lazy=False, handoff=None, out_dtype=None):
        """`lazy`: the caller can take a norm that is not computed yet (parts.linear.NormedStream);
        it gets one when nothing has to be added into the stream first.  `handoff`: where the writer of
        the stream may have left this norm's input.  `out_dtype` float32: the normed rows unrounded, for a reader
        that works on them before a product does (`delta` is then float32 or None)."""
        if out_dtype is not None and out_dtype != self.runtime.dtype:
            if handoff is not None:
                handoff.claim(resid, self.gamma)
            n = rows.numel() if rows is not None else resid.shape[0]
            out = torch.empty((n, self.spec.size), dtype=out_dtype, device=resid.device)
            K.add_rmsnorm(resid, delta, self.gamma, self.spec.eps, out, rows)
            return out
        if isinstance(delta, PostNormed):
            if handoff is not None:
                handoff.claim(resid, self.gamma)          # nothing a product left fits a stream that changes now
            n = rows.numel() if rows is not None else resid.shape[0]
            out = torch.empty((n, self.spec.size), dtype=self.runtime.dtype, device=resid.device)
            if getattr(self, "_gamma32", None) is None:
                self._gamma32 = self.gamma.to(torch.float32).contiguous()
            K.sandwich_norm(resid, delta.output, delta.weight, delta.mult, delta.eps, self._gamma32, self.spec.eps, out,
                            rows=rows, delta_bias=delta.bias, second=delta.second)
            return out
        handed = handoff.claim(resid, self.gamma) if handoff is not None else None
        if lazy and delta is None:
            return NormedStream(resid, self.gamma, self.spec.eps, rows, self.runtime.dtype, handed)
        n = rows.numel() if rows is not None else resid.shape[0]
        out = torch.empty((n, self.spec.size), dtype=self.runtime.dtype, device=resid.device)
        K.add_rmsnorm(resid, delta, self.gamma, self.spec.eps, out, rows)
        return out


@dataclass(frozen=True)
class PostRMSNormSpec:
    size: int
    eps: float
    mult: float = 1.0             # what the normed output is multiplied by before it joins the stream


@register_part("norm", "rms_post")
class PostRMSNorm(Part):
    """The RMS norm behind a sublayer: x <- x + mult * norm(sublayer output).  It computes nothing by itself: `pending`
    wraps the output for the norm that reads the stream next, which adds and norms in one kernel."""
    family = "norm"
    graph_safe = True
    roles = ("weight",)
    kernel_modules = ("stream_ops",)

    def tensor_specs(self):
        return [TensorSpec(self.tensor_names["weight"], (self.spec.size,), init="one_plus_normal:0.1")]

    def bind(self, loaded):
        self.weight = loaded[self.tensor_names["weight"]].to(torch.float32).contiguous()

    def pending(self, output, bias=None, second=None) -> PostNormed:
        return PostNormed(output, self.weight, self.spec.eps, self.spec.mult, bias, second)

    @staticmethod
    def add(resid, pending: PostNormed) -> None:
        """Only the add into the stream (no norm reads it next)."""
        K.sandwich_norm(resid, pending.output, pending.weight, pending.mult, pending.eps, None, 0.0, None, delta_bias=pending.bias,
                        second=pending.second)


@dataclass(frozen=True)
class DynamicTanhSpec:
    size: int


@register_part("norm", "dynamic_tanh")
class DynamicTanh(Part):
    """y = tanh(alpha x) * weight + bias with a learned scalar alpha: a squashing in the place of a norm, computed
    element by element in fp32 without a mean or a variance.  Weight, bias and alpha are kept in float32."""
    family = "norm"
    graph_safe = True
    roles = ("weight", "bias", "alpha")
    kernel_modules = ("elementwise",)
    takes_several = True          # `delta` may be a tuple of outputs that are all added into the stream

    def tensor_specs(self):
        t, n = self.tensor_names, self.spec.size
        return [TensorSpec(t["weight"], (n,), init="one_plus_normal:0.1"), TensorSpec(t["bias"], (n,), init="normal:0.1"),
                TensorSpec(t["alpha"], (), init="one_plus_normal:0.2")]

    def bind(self, loaded):
        t = self.tensor_names
        self.weight = loaded[t["weight"]].to(torch.float32).contiguous()
        self.bias = loaded[t["bias"]].to(torch.float32).contiguous()
        self.alpha = loaded[t["alpha"]].to(torch.float32).reshape(1).contiguous()

    def parameters(self):
        """(weight, bias, alpha) in float32, for a kernel that applies this norm in its own epilogue."""
        return self.weight, self.bias, self.alpha

    def add_norm(self, resid, delta, rows=None, lazy=False, handoff=None):
        deltas = list(delta) if isinstance(delta, (tuple, list)) else ([delta] if delta is not None else [])
        n = rows.numel() if rows is not None else resid.shape[0]
        out = torch.empty((n, self.spec.size), dtype=self.runtime.dtype, device=resid.device)
        K.add_dyt(resid, deltas, self.weight, self.bias, self.alpha, out, rows)
        return out
