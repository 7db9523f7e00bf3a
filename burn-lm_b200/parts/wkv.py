"""The WKV mixer: RWKV-style time mixing with a decay per key channel that depends on the token.

With h' the input of the token before (zeros for a sequence's first), each of r, k, v, g, w reads its own mix
h + (h' - h) mu_s.  r, k, v = Wr, Wk, Wv of their mixes (heads x dim each), gate = silu(Wg mix_g), and the decay
w = exp(-exp(W2 tanh(W1 mix_w) + w0)) per head and key channel.  Per head, S [dim x dim]:
o = (S + diag(u) k v^T)^T r with the state before the token (u: a bonus for the current token only), then
S <- diag(w) S + k v^T.  Each head's o is divided by its root mean square; the concatenated heads are multiplied by a
weight of their size and by the gate, then projected.  S (fp32) and the last input h are carried per sequence; mixes,
decays and state are fp32 in both dtypes.
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

MIXES = ("r", "k", "v", "g", "w")


@dataclass(frozen=True)
class WkvSpec:
    hidden_size: int
    n_heads: int
    head_dim: int
    eps: float
    decay_rank: Optional[int] = None     # inner size of the decays' two-step projection; None: read off the stored tensors


@register_part("mixer", "wkv")
class Wkv(Part):
    family = "mixer"
    graph_safe = True
    takes_float32_input = True           # the mixes are taken from the unrounded input
    roles = tuple("mu_" + m for m in MIXES) + ("r", "k", "v", "g", "w1", "w2", "w0", "u", "norm", "o")
    kernel_modules = ("recurrent", "stream_ops", "gemm")

    def __init__(self, spec, tensors, runtime):
        super().__init__(spec, tensors, runtime)
        self.hk = spec.n_heads * spec.head_dim
        self.shift_floats = spec.hidden_size
        self.state_floats = self.shift_floats + K.scan_state_floats(spec.n_heads, spec.head_dim, spec.head_dim)

    def tensor_specs(self):
        s, t = self.spec, self.tensor_names
        d, rank = s.hidden_size, s.decay_rank or -1
        free = max(4, d // 16)
        return [TensorSpec(t["mu_" + m], (d,), init="sigmoid_normal:1.0") for m in MIXES] + \
               [TensorSpec(t[m], (self.hk, d)) for m in ("r", "k", "v", "g")] + \
               [TensorSpec(t["w1"], (rank, d), free=free), TensorSpec(t["w2"], (self.hk, rank), init="normal:0.1", free=free),
                TensorSpec(t["w0"], (self.hk,), init="normal:1.0"), TensorSpec(t["u"], (s.n_heads, s.head_dim), init="normal:0.5"),
                TensorSpec(t["norm"], (self.hk,), init="one_plus_normal:0.1"), TensorSpec(t["o"], (d, self.hk))]

    def bind(self, loaded):
        t = self.tensor_names
        ws = [loaded[t[m]] for m in ("r", "k", "v", "g")]
        if len({w.dtype for w in ws}) != 1:
            raise ValueError(f"the projections of {t['r']} and its neighbours are stored in different dtypes")
        self.rkvg = torch.stack(ws).contiguous()                     # [4, heads * dim, width]: a product per mix, one launch
        self.w1, self.w2, self.o = Linear(loaded[t["w1"]]), Linear(loaded[t["w2"]]), Linear(loaded[t["o"]])
        if loaded[t["w2"]].shape[1] != loaded[t["w1"]].shape[0]:
            raise ValueError(f"{t['w2']} does not continue {t['w1']}")
        self.mu = torch.stack([f32(loaded[t["mu_" + m]]) for m in MIXES]).contiguous()
        self.w0, self.u, self.norm_weight = f32(loaded[t["w0"]]), f32(loaded[t["u"]]).reshape(-1), f32(loaded[t["norm"]])

    def cache_need(self) -> CacheNeed:
        return CacheNeed("state", state_shape=(2, self.state_floats))

    def forward(self, x, step, cache):
        s, rt = self.spec, self.runtime
        if not cache.writes:
            raise ValueError("this mixer carries a state of its own; it cannot read another run's")
        if x.dtype != torch.float32:
            raise ValueError("this mixer takes its input unrounded (float32)")
        n, dev = step.n_tokens, x.device
        mixes = torch.empty((len(MIXES), n, s.hidden_size), dtype=self.rkvg.dtype, device=dev)
        K.shift_mix(x, self.mu, mixes, step, cache.state, cache.state_offset)
        rkvg = K.batched_product(mixes[:4], self.rkvg, out_dtype=torch.float32)          # [4, N, heads * dim] in fp32
        low = self.w1(mixes[4], out_dtype=torch.float32)
        squashed = torch.empty(low.shape, dtype=self.w2.weight.dtype, device=dev)
        K.bias_act(low, None, squashed, kind=K.ACT_TANH)
        decay = self.w2(squashed, out_dtype=torch.float32)                                # [N, heads * dim]; w0 joins in the scan
        o = torch.zeros((n, self.hk), dtype=torch.float32, device=dev)                   # rows of no sequence stay zero
        K.decay_scan(rkvg[0], 0, rkvg[1], 0, rkvg[2], 0, decay, 0, self.w0, self.u, o, s.n_heads, s.head_dim, s.head_dim,
                     K.DECAY_EXP_EXP, True, step, cache.state, cache.state_offset + self.shift_floats, wide_sums=rt.exact)
        gated = torch.empty((n, self.hk), dtype=rt.dtype, device=dev)
        K.gated_group_norm(o, rkvg[3], 0, self.norm_weight, s.head_dim, K.GATE_SILU_LAST, s.eps, gated)
        return self.o(gated, out_dtype=torch.float32)
