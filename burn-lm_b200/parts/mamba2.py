"""The state-space mixer (Mamba-2, the scalar-decay form of state-space duality).

One input projection gives [z | x | B | C | dt]; x, B and C pass a short causal convolution per channel (with a bias)
and silu; per head h with its group g: dt = softplus(dt + dt_bias_h), S <- exp(-exp(A_log_h) dt) S + dt B x^T (S is
state x value_dim), y = S^T C + D_h x.  The heads' outputs are multiplied by silu(z), RMS-normed in `norm_groups` equal
parts of the row (the gate comes before the norm), scaled by a weight and projected out.  The convolution's last inputs
and S (fp32) are what a sequence carries from token to token.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from .. import kernels as K
from ..registry import register_part
from ..weights.loader import TensorSpec
from .base import CacheNeed, Part
from .linear import Linear


@dataclass(frozen=True)
class Mamba2Spec:
    hidden_size: int
    n_heads: int
    value_dim: int                # lanes of a head
    state: int                    # rows of a head's state
    groups: int                   # heads // groups heads share a B and a C
    conv: int                     # taps of the convolution
    norm_groups: int
    eps: float


def f32(t):
    return t.to(torch.float32).contiguous()


@register_part("mixer", "mamba2")
class Mamba2(Part):
    family = "mixer"
    graph_safe = True
    roles = ("in", "conv", "conv_bias", "dt_bias", "A_log", "D", "norm", "o")
    kernel_modules = ("recurrent",)

    def __init__(self, spec, tensors, runtime):
        super().__init__(spec, tensors, runtime)
        s = spec
        if s.n_heads % s.groups:
            raise ValueError(f"{s.n_heads} heads do not divide into {s.groups} groups")
        self.inner = s.n_heads * s.value_dim
        if self.inner % s.norm_groups:
            raise ValueError(f"{s.norm_groups} norm groups do not divide the {self.inner} lanes of the heads")
        self.conv_channels = self.inner + 2 * s.groups * s.state
        self.width = 2 * self.inner + 2 * s.groups * s.state + s.n_heads          # z | x | B | C | dt
        # one copy of what a sequence carries: the convolution's last inputs, then the heads' states
        self.hist_floats = (s.conv - 1) * self.conv_channels
        self.state_floats = self.hist_floats + K.scan_state_floats(s.n_heads, s.state, s.value_dim)

    def tensor_specs(self):
        s, t = self.spec, self.tensor_names
        return [TensorSpec(t["in"], (self.width, s.hidden_size)),
                TensorSpec(t["conv"], (self.conv_channels, s.conv), init="normal:0.3"),
                TensorSpec(t["conv_bias"], (self.conv_channels,), init="normal:0.1"),
                TensorSpec(t["dt_bias"], (s.n_heads,), init="normal:0.5"),
                TensorSpec(t["A_log"], (s.n_heads,), init="normal:0.5"),
                TensorSpec(t["D"], (s.n_heads,), init="one_plus_normal:0.1"),
                TensorSpec(t["norm"], (self.inner,), init="one_plus_normal:0.1"),
                TensorSpec(t["o"], (s.hidden_size, self.inner))]

    def bind(self, loaded):
        t = self.tensor_names
        self.proj = Linear(loaded[t["in"]])
        self.o = Linear(loaded[t["o"]])
        self.taps, self.conv_bias = f32(loaded[t["conv"]]), f32(loaded[t["conv_bias"]])
        self.dt_bias, self.a_log, self.d_skip = f32(loaded[t["dt_bias"]]), f32(loaded[t["A_log"]]), f32(loaded[t["D"]])
        self.norm_weight = f32(loaded[t["norm"]])

    def cache_need(self) -> CacheNeed:
        return CacheNeed("state", state_shape=(2, self.state_floats))

    def forward(self, x, step, cache):
        s, rt = self.spec, self.runtime
        if not cache.writes:
            raise ValueError("this mixer carries a state of its own; it cannot read another run's")
        n, inner, gn = step.n_tokens, self.inner, s.groups * s.state
        proj = self.proj(x, out_dtype=torch.float32)                       # [N, z | x | B | C | dt] in fp32
        xbc = torch.empty((n, self.conv_channels), dtype=torch.float32, device=proj.device)
        K.causal_conv(proj, inner, self.conv_channels, self.taps, self.conv_bias, xbc, 0, step, cache.state, cache.state_offset, silu=True)
        y = torch.zeros((n, inner), dtype=torch.float32, device=proj.device)      # rows of no sequence stay zero
        K.ssm_scan(xbc, 0, inner, inner + gn, proj, 2 * inner + 2 * gn, self.dt_bias, self.a_log, self.d_skip, y,
                   s.n_heads, s.groups, s.state, s.value_dim, step, cache.state, cache.state_offset + self.hist_floats, wide_sums=rt.exact)
        gated = torch.empty((n, inner), dtype=rt.dtype, device=proj.device)
        K.gated_group_norm(y, proj, 0, self.norm_weight, inner // s.norm_groups, K.GATE_FIRST, s.eps, gated)
        return self.o(gated, out_dtype=torch.float32)
