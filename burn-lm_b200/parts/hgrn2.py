"""The HGRN2 mixer: linear attention whose forget gate also decides what is written.

q = silu(Wq h) (heads x key_dim), v = Wv h (heads x value_dim); the forget gate per head and key channel is
f = low + (1 - low) sigmoid(Wf h + b) with a stored lower bound `low`.  Per head, S [key_dim x value_dim]:
S <- diag(f) S + (1 - f) v^T, then o = S^T q: the write's key is 1 - f, there is no other key and no scale.  Each head's o
is RMS-normed over its value lanes with a weight shared by the heads; the heads are concatenated and projected.  S (fp32)
is carried per sequence; gate, bound and state are fp32 in both dtypes.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from .. import kernels as K
from ..registry import register_part
from ..weights.loader import TensorSpec
from .base import CacheNeed, Part
from .linear import Linear
from .mamba2 import f32


@dataclass(frozen=True)
class Hgrn2Spec:
    hidden_size: int
    n_heads: int
    key_dim: int
    value_dim: int
    eps: float


@register_part("mixer", "hgrn2")
class Hgrn2(Part):
    family = "mixer"
    graph_safe = True
    roles = ("q", "f", "f_bias", "lower", "v", "norm", "o")
    kernel_modules = ("recurrent",)

    def __init__(self, spec, tensors, runtime):
        super().__init__(spec, tensors, runtime)
        self.kw, self.vw = spec.n_heads * spec.key_dim, spec.n_heads * spec.value_dim
        self.state_floats = K.scan_state_floats(spec.n_heads, spec.key_dim, spec.value_dim)

    def tensor_specs(self):
        s, t = self.spec, self.tensor_names
        d = s.hidden_size
        return [TensorSpec(t["q"], (self.kw, d)), TensorSpec(t["f"], (self.kw, d)),
                TensorSpec(t["f_bias"], (self.kw,), init="normal:1.0"), TensorSpec(t["lower"], (self.kw,), init="sigmoid_normal:1.0"),
                TensorSpec(t["v"], (self.vw, d)), TensorSpec(t["norm"], (s.value_dim,), init="one_plus_normal:0.1"),
                TensorSpec(t["o"], (d, self.vw))]

    def bind(self, loaded):
        t = self.tensor_names
        ws = [loaded[t[r]] for r in ("q", "f", "v")]
        if len({w.dtype for w in ws}) != 1:
            raise ValueError(f"the projections of {t['q']} and its neighbours are stored in different dtypes")
        self.proj = Linear(torch.cat(ws, dim=0).contiguous())         # [q | f | v], kept in fp32 for the gate and the scan
        self.o = Linear(loaded[t["o"]])
        self.f_bias, self.lower, self.norm_weight = f32(loaded[t["f_bias"]]), f32(loaded[t["lower"]]), f32(loaded[t["norm"]])

    def cache_need(self) -> CacheNeed:
        return CacheNeed("state", state_shape=(2, self.state_floats))

    def forward(self, x, step, cache):
        s, rt = self.spec, self.runtime
        if not cache.writes:
            raise ValueError("this mixer carries a state of its own; it cannot read another run's")
        n = step.n_tokens
        proj = self.proj(x, out_dtype=torch.float32)
        o = torch.zeros((n, self.vw), dtype=torch.float32, device=proj.device)           # rows of no sequence stay zero
        K.decay_scan(proj, 0, None, 0, proj, 2 * self.kw, proj, self.kw, self.f_bias, self.lower, o, s.n_heads, s.key_dim,
                     s.value_dim, K.DECAY_LOWER_BOUND, False, step, cache.state, cache.state_offset, wide_sums=rt.exact)
        normed = torch.empty((n, self.vw), dtype=rt.dtype, device=proj.device)
        K.gated_group_norm(o, None, 0, self.norm_weight, s.value_dim, K.GATE_NONE, s.eps, normed)
        return self.o(normed, out_dtype=torch.float32)
