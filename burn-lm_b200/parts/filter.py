"""Filters over time that stand between a layer's norm and its mixer.

Kind "short_conv": a causal convolution per channel, y_t = sum_j w[:, j] x_(t - (K - 1) + j) with zeros before a
sequence's start and no bias; with `residual` the token's own input joins the sum, y_t = x_t + conv(x)_t.  The last
K - 1 inputs of a sequence are part of what it keeps: `state_floats()` says how many floats of a state copy the filter
wants, and the block that arranges it hands over the state block and the place in it.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from .. import kernels as K
from ..registry import register_part
from ..weights.loader import TensorSpec
from .base import Part


@dataclass(frozen=True)
class ShortConvSpec:
    channels: int
    taps: int
    residual: bool = True


@register_part("filter", "short_conv")
class ShortConv(Part):
    """forward(x float32 [N, C], step, state, state_offset) -> (y float32 [N, C], y in the compute dtype)."""
    family = "filter"
    graph_safe = True
    roles = ("taps",)
    kernel_modules = ("recurrent",)

    def tensor_specs(self):
        return [TensorSpec(self.tensor_names["taps"], (self.spec.channels, self.spec.taps), init="normal:0.2")]

    def bind(self, loaded):
        self.taps = loaded[self.tensor_names["taps"]].to(torch.float32).contiguous()

    def state_floats(self) -> int:
        """Floats of a state copy: the carried inputs [taps - 1, channels] (one float when a single tap carries none, so
        that the filter always has a place of its own)."""
        return (self.spec.taps - 1) * self.spec.channels or 1

    def forward(self, x, step, state, state_offset):
        s = self.spec
        y = torch.empty((step.n_tokens, s.channels), dtype=torch.float32, device=x.device)
        rounded = None
        if self.runtime.dtype == torch.bfloat16:
            rounded = torch.empty((step.n_tokens, s.channels), dtype=torch.bfloat16, device=x.device)
        K.causal_conv(x, 0, s.channels, self.taps, None, y, 0, step, state, state_offset, silu=False, out_bf16=rounded,
                      residual=s.residual)
        return y, (rounded if rounded is not None else y)
