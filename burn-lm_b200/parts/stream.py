"""Rewrites of the residual stream that stand between runs of layers (family "stream").

A stream part takes the stream, what the run before left to be added to it, and the embedding's output of the step, and
returns the stream that the next run reads: forward(resid, delta, embedded, step) -> resid.  A plan lists its stream
parts and names, per run of its schedule, the one that stands in front of it.

Kind "concat_projection": x <- W [x; x0] with W [width, 2 width] (the stream's columns first) and x0 the embedding's
output: a loop over some layers feeds the input in again at the start of every pass.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from .. import kernels as K
from ..registry import register_part
from ..weights.loader import TensorSpec
from .base import Part
from .linear import Linear


@dataclass(frozen=True)
class ConcatProjectionSpec:
    hidden_size: int


@register_part("stream", "concat_projection")
class ConcatProjection(Part):
    family = "stream"
    graph_safe = True
    needs_embedding = True        # the model keeps the embedding's output of the step for this part
    roles = ("weight",)
    kernel_modules = ("stream_ops",)

    def tensor_specs(self):
        d = self.spec.hidden_size
        return [TensorSpec(self.tensor_names["weight"], (d, 2 * d))]

    def bind(self, loaded):
        self.linear = Linear(loaded[self.tensor_names["weight"]])

    def forward(self, resid, delta, embedded, step):
        n, d = resid.shape
        both = torch.empty((n, 2 * d), dtype=self.linear.weight.dtype, device=resid.device)
        K.pack_cols(resid, delta, both, 0)          # the pending output joins the stream on the way (fp32)
        K.pack_cols(embedded, None, both, d)
        return self.linear(both, out_dtype=torch.float32)
