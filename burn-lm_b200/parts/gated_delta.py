"""The gated delta rule mixer: a matrix state per head that is decayed per key channel, corrected by the error of its
own prediction, and read out after the write.

q = Wq h and k = Wk h (qk_heads x key_dim), v = Wv h (heads x value_dim); each passes a short causal convolution per
channel (no bias) and silu; q and k become unit vectors per head (x / sqrt(sum x^2 + 1e-6)), q also times key_dim^-1/2;
beta = sigmoid(Wb h) per head; g = exp(-exp(A_log_h) softplus(Wa2 (Wa1 h) + dt_bias)) per head and key channel.  Per
head (head h uses q/k head h // (heads / qk_heads)), S [key_dim x value_dim]:  S <- g S (rows);  u = beta (v - S^T k);
S <- S + k u^T;  o = S^T q.  Each head's o is divided by its root mean square, times a weight shared by the heads,
times sigmoid(Wg2 (Wg1 h)); then the output projection.  S (fp32) and the convolutions' last inputs are carried.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from .. import kernels as K
from ..registry import register_part
from ..weights.loader import TensorSpec
from .base import CacheNeed, Part
from .linear import Linear
from .mamba2 import f32


@dataclass(frozen=True)
class GatedDeltaSpec:
    hidden_size: int
    n_heads: int
    qk_heads: int
    key_dim: int
    value_dim: int
    conv: int
    eps: float
    decay_rank: Optional[int] = None     # inner size of the two-step projection of the decays; None: read off the stored
    gate_rank: Optional[int] = None      # tensors (no configuration key names it); the same for the output gate's


@register_part("mixer", "gated_delta")
class GatedDelta(Part):
    family = "mixer"
    graph_safe = True
    roles = ("q", "q_conv", "k", "k_conv", "v", "v_conv", "b", "A_log", "norm", "a1", "a2", "dt_bias", "g1", "g2", "o")
    kernel_modules = ("recurrent",)

    def __init__(self, spec, tensors, runtime):
        super().__init__(spec, tensors, runtime)
        s = spec
        if s.n_heads % s.qk_heads:
            raise ValueError(f"{s.n_heads} heads do not divide into {s.qk_heads} query/key heads")
        self.qk, self.vw = s.qk_heads * s.key_dim, s.n_heads * s.value_dim
        self.conv_channels = 2 * self.qk + self.vw                          # q | k | v
        self.hist_floats = (s.conv - 1) * self.conv_channels
        self.state_floats = self.hist_floats + K.scan_state_floats(s.n_heads, s.key_dim, s.value_dim)

    def tensor_specs(self):
        s, t = self.spec, self.tensor_names
        d = s.hidden_size
        free = max(4, d // 8)       # what a rank that nothing names is made when weights are drawn rather than read
        ra, rg = s.decay_rank or -1, s.gate_rank or -1
        return [TensorSpec(t["q"], (self.qk, d)), TensorSpec(t["q_conv"], (self.qk, s.conv), init="normal:0.3"),
                TensorSpec(t["k"], (self.qk, d)), TensorSpec(t["k_conv"], (self.qk, s.conv), init="normal:0.3"),
                TensorSpec(t["v"], (self.vw, d)), TensorSpec(t["v_conv"], (self.vw, s.conv), init="normal:0.3"),
                TensorSpec(t["b"], (s.n_heads, d)), TensorSpec(t["A_log"], (s.n_heads,), init="normal:0.5"),
                TensorSpec(t["norm"], (s.value_dim,), init="one_plus_normal:0.1"),
                TensorSpec(t["a1"], (ra, d), free=free), TensorSpec(t["a2"], (s.n_heads * s.key_dim, ra), init="normal:0.1", free=free),
                TensorSpec(t["dt_bias"], (s.n_heads * s.key_dim,), init="normal:0.5"),
                TensorSpec(t["g1"], (rg, d), free=free), TensorSpec(t["g2"], (self.vw, rg), init="normal:0.1", free=free),
                TensorSpec(t["o"], (d, self.vw))]

    def bind(self, loaded):
        s, t = self.spec, self.tensor_names
        ws = [loaded[t[r]] for r in ("q", "k", "v", "b")]
        low = [loaded[t["a1"]], loaded[t["g1"]]]
        a2, g2 = loaded[t["a2"]], loaded[t["g2"]]
        if len({w.dtype for w in ws + low + [a2, g2]}) != 1:
            raise ValueError(f"the projections of {t['q']} and its neighbours are stored in different dtypes")
        # two products read the layer's input: q | k | v | b (kept in fp32), and the first steps of the decays' and the
        # gate's projections a1 | g1; their second steps run as one product with the weight [[a2, 0], [0, g2]]
        self.proj = Linear(torch.cat(ws, dim=0).contiguous())
        self.low = Linear(torch.cat(low, dim=0).contiguous())
        ra, rg = low[0].shape[0], low[1].shape[0]
        if a2.shape[1] != ra or g2.shape[1] != rg:
            raise ValueError(f"{t['a2']} and {t['g2']} do not continue {t['a1']} ({ra} rows) and {t['g1']} ({rg} rows)")
        second = torch.zeros((a2.shape[0] + g2.shape[0], ra + rg), dtype=a2.dtype, device=a2.device)
        second[:a2.shape[0], :ra] = a2
        second[a2.shape[0]:, ra:] = g2
        self.second = Linear(second.contiguous())
        self.o = Linear(loaded[t["o"]])
        self.taps = torch.cat([f32(loaded[t["q_conv"]]), f32(loaded[t["k_conv"]]), f32(loaded[t["v_conv"]])], dim=0).contiguous()
        self.dt_bias, self.a_log, self.norm_weight = f32(loaded[t["dt_bias"]]), f32(loaded[t["A_log"]]), f32(loaded[t["norm"]])

    def cache_need(self) -> CacheNeed:
        return CacheNeed("state", state_shape=(2, self.state_floats))

    def forward(self, x, step, cache):
        s, rt = self.spec, self.runtime
        if not cache.writes:
            raise ValueError("this mixer carries a state of its own; it cannot read another run's")
        n = step.n_tokens
        proj = self.proj(x, out_dtype=torch.float32)                         # [N, q | k | v | b] in fp32
        dev = proj.device
        conv = torch.empty((n, self.conv_channels), dtype=torch.float32, device=dev)
        K.causal_conv(proj, 0, self.conv_channels, self.taps, None, conv, 0, step, cache.state, cache.state_offset, silu=True)
        wide = self.second(self.low(x, out_dtype=rt.dtype), out_dtype=torch.float32)      # [N, decays | gate] in fp32
        o = torch.zeros((n, self.vw), dtype=torch.float32, device=dev)                    # rows of no sequence stay zero
        K.delta_scan(conv, 0, conv, self.qk, conv, 2 * self.qk, proj, self.conv_channels, wide, 0, self.dt_bias, self.a_log, o,
                     s.n_heads, s.qk_heads, s.key_dim, s.value_dim, step, cache.state, cache.state_offset + self.hist_floats)
        gated = torch.empty((n, self.vw), dtype=rt.dtype, device=dev)
        K.gated_group_norm(o, wide, s.n_heads * s.key_dim, self.norm_weight, s.value_dim, K.GATE_LAST, s.eps, gated)
        return self.o(gated, out_dtype=torch.float32)
