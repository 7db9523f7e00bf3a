"""Grouped-query attention whose queries, keys and values are normed head by head, with a number per head on the
scores, capped scores and a sink in the softmax.

q = Wq h, k = Wk h, v = Wv h without biases.  Every head of q and of k is divided by its root mean square and
multiplied by a weight of the head's size that all heads share (`qk_norm`); the first `rotary_dims` lanes of every q
and k head then turn by position * base^(-2i / rotary_dims), lanes (2i, 2i + 1) together (`rotary_halves`: lanes
(i, i + rotary_dims / 2)); every head of v is divided by its root mean square (`value_norm`, no weight) and cached so.
Query head h reads key/value head h // (heads / kv heads); keys have `head_dim` lanes, values `value_dim`.
s = scale * t_h * q.k (`head_temperature`: t a stored number per query head), then s <- cap tanh(s / cap)
(`softcap`); position i sees j <= i, or only 0 <= i - j < window; p_j = exp(s_j) / (sink + sum exp(s_j)) with `sink`
one more entry of score 0 that carries no value.  The heads' outputs are concatenated and projected by Wo.

Norms, rotation, scores, cap and softmax are fp32 in both dtypes.  The three projections run as one product with a
fused [q; k; v] weight whose result stays in fp32 for the norms; the attention kernels are the windowed family's
(`kernels.attention_sink`), which take the head's number, the cap and the sink as options.
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

BLOCKS_PER_SM = 4          # blocks of the single-token kernels a step should offer every multiprocessor
NO_WINDOW = 1 << 30        # what the kernels take for "every earlier key"


@dataclass(frozen=True)
class NormedAttentionSpec:
    hidden_size: int
    n_heads: int
    n_kv_heads: int
    head_dim: int                     # lanes of a head's query and key
    value_dim: int                    # lanes of a head's value
    scale: float
    eps: float                        # of the norms over heads
    rotary_dims: int = 0              # how many of a head's first lanes turn
    rotary_base: float = 10000.0
    rotary_halves: bool = False       # lanes (i, i + rotary_dims / 2) turn together instead of (2i, 2i + 1)
    qk_norm: bool = True              # RMS norm with a shared weight over every head of q and of k
    value_norm: bool = True           # every head of v divided by its root mean square
    head_temperature: bool = True     # a stored number per query head multiplies its scores
    softcap: Optional[float] = None   # s <- cap tanh(s / cap)
    sink: bool = True                 # one more entry of score 0 in the softmax's denominator
    window: Optional[int] = None      # None: every earlier key


@register_part("mixer", "normed_attention")
class NormedAttention(Part):
    family = "mixer"
    graph_safe = True
    roles = ("q", "k", "v", "o", "q_norm", "k_norm", "temperature")
    kernel_modules = ("elementwise", "attention_sink")

    def __init__(self, spec, tensors, runtime):
        super().__init__(spec, tensors, runtime)
        if spec.n_heads % spec.n_kv_heads:
            raise ValueError(f"{spec.n_heads} heads do not divide into {spec.n_kv_heads} kv heads")
        if spec.value_dim > 512:
            raise ValueError(f"value_dim {spec.value_dim}: the attention kernels take values of up to 512 lanes")
        if spec.rotary_dims % 2 or spec.rotary_dims > spec.head_dim:
            raise ValueError(f"{spec.rotary_dims} turning lanes of {spec.head_dim}: an even number, at most all of them")
        if spec.window is not None and spec.window < 1:
            raise ValueError(f"a window of {spec.window}")

    def tensor_specs(self):
        s, t = self.spec, self.tensor_names
        specs = [TensorSpec(t["q"], (s.n_heads * s.head_dim, s.hidden_size)),
                 TensorSpec(t["k"], (s.n_kv_heads * s.head_dim, s.hidden_size)),
                 TensorSpec(t["v"], (s.n_kv_heads * s.value_dim, s.hidden_size)),
                 TensorSpec(t["o"], (s.hidden_size, s.n_heads * s.value_dim))]
        if s.qk_norm:
            specs += [TensorSpec(t["q_norm"], (s.head_dim,), init="one_plus_normal:0.1"),
                      TensorSpec(t["k_norm"], (s.head_dim,), init="one_plus_normal:0.1")]
        if s.head_temperature:
            specs.append(TensorSpec(t["temperature"], (s.n_heads,), init="one_plus_normal:0.1"))
        return specs

    def bind(self, loaded):
        s, t = self.spec, self.tensor_names
        ws = [loaded[t["q"]], loaded[t["k"]], loaded[t["v"]]]
        if len({w.dtype for w in ws}) != 1:
            raise ValueError(f"the projections of {t['q']} and its neighbours are stored in different dtypes")
        self.proj = Linear(torch.cat(ws, dim=0).contiguous())
        self.o = Linear(loaded[t["o"]])
        f32 = lambda x: x.to(torch.float32).contiguous()
        self.q_weight = f32(loaded[t["q_norm"]]) if s.qk_norm else None
        self.k_weight = f32(loaded[t["k_norm"]]) if s.qk_norm else None
        self.temperature = f32(loaded[t["temperature"]]) if s.head_temperature else None
        self.freq = None
        if s.rotary_dims:
            self.freq = torch.tensor([s.rotary_base ** (-2.0 * i / s.rotary_dims) for i in range(s.rotary_dims // 2)],
                                     dtype=torch.float64).to(self.o.weight.device)

    def cache_need(self) -> CacheNeed:
        s = self.spec
        return CacheNeed("kv", n_kv_heads=s.n_kv_heads, head_dim=s.head_dim, window=s.window, value_dim=s.value_dim)

    def _splits(self, step) -> int:
        """Over how many blocks the single-token kernels cut a row's keys: a few tokens with many keys leave most of the
        multiprocessors idle otherwise."""
        s = self.spec
        if K.attention_sink_prompt_takes(self.runtime.dtype, s.head_dim, s.value_dim, step.max_q_len, s.n_heads):
            return 1
        seen = min(step.max_kv_len, s.window or step.max_kv_len)
        blocks = step.n_tokens * s.n_kv_heads
        want = BLOCKS_PER_SM * K.sm_count(self.runtime.device)
        if K.attention_sink_decode_takes(self.runtime.dtype, s.head_dim, s.value_dim, s.n_heads, s.n_kv_heads):
            pages = seen // K.PAGE + 1                       # that kernel cuts by pages, and its blocks hold several
            want //= 2
            return max(1, min((want + blocks - 1) // blocks, pages // 4, 32))
        return max(1, min((want + blocks - 1) // blocks, seen // 128, 32))

    def forward(self, x, step, cache):
        s, rt = self.spec, self.runtime
        if not cache.writes:
            raise ValueError("this mixer appends to a cache line of its own; it cannot read another run's")
        n = step.n_tokens
        proj = self.proj(x, out_dtype=torch.float32)            # [N, q | k | v] in fp32
        q = torch.empty((n, s.n_heads * s.head_dim), dtype=rt.dtype, device=proj.device)
        K.head_norm_rope_append(proj, step, cache.pool, cache.block_table, q, s.n_heads, s.n_kv_heads, s.head_dim, s.value_dim,
                                q_weight=self.q_weight, k_weight=self.k_weight, eps=s.eps, value_norm=s.value_norm, freq=self.freq,
                                rotary_dims=s.rotary_dims, halves=s.rotary_halves)
        out = torch.empty((n, s.n_heads * s.value_dim), dtype=rt.dtype, device=proj.device)
        n_splits = self._splits(step)
        scratch = None
        if n_splits > 1:
            scratch = step.workspace.scratch("attention_sink", K.attention_sink_scratch_floats(n, s.n_heads, s.value_dim, n_splits))
        K.attention_sink(q, step, cache.pool, cache.block_table, out, s.n_heads, s.n_kv_heads, s.head_dim, s.value_dim, s.scale,
                         s.window or NO_WINDOW, 0, sink=s.sink, max_q_len=step.max_q_len, n_splits=n_splits, scratch=scratch,
                         head_scale=self.temperature, softcap=s.softcap or 0.0)
        return self.o(out, out_dtype=torch.float32)
