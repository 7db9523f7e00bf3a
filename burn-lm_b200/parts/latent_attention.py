"""Attention over a cached latent: keys and values of all heads are made from one small vector per position.

q = Wq h, a head's lanes laid out as [key_dim unrotated | rot_dim rotated]; Wdkv h has rank + rot_dim rows: the first
`rank`, RMS-normed with a plain weight, are the latent c, the last rot_dim one rotated key part that all heads share.
Head i's unrotated key is Wuk_i c and its value Wuv_i c; its score is (q_nope . Wuk_i c + q_rot . k_rot) * scale, softmax
over the positions j <= i.  The rotation turns the lane pairs (2m, 2m + 1), m < rot_dims / 2, of the rotated parts by
position * base^(-2m / rot_dims); lanes from rot_dims on pass unchanged.  The concatenated heads are multiplied by
sigmoid(Wg h) and projected by Wo.

Options, all spec fields: the queries go through a latent of their own, q = Wuq RMSnorm(Wdq h) (`q_rank`); the turning
lanes are paired (m, m + rot_dims / 2) instead (`rotary_halves`); position i sees only j with 0 <= i - j < `window`; the
softmax's denominator also holds exp(sink_h), a stored number per head without key or value (`sink`); the gate is one
number per head, sigmoid(Wg h)_h with Wg [heads, width] (`gate_per_head`).

Only c and the rotated key part are cached (a paged line of rows of rank + rot_dim lanes).  Because key and value are
linear in c, the up-projections are taken off the cached side: q' = Wuk_i^T q_nope is a small batched product in front of
the attention kernel, which then works on the latent itself (score q' . c + q_rot . k_rot, output sum_j p_j c_j), and
Wuv_i is a batched product behind it.

Steps that bring 16 or more tokens of a sequence in bfloat16 go the other way round when a head's key ([unrotated |
rotated]) fits 128 lanes: the latents of the step's sequences are gathered, one product makes every head's unrotated
keys and values from them, and the grouped-query attention kernels (the tensor-core ones for prompts) run on those
pages with as many key/value heads as query heads.  A prompt's attention then costs what a dense decoder's costs
instead of (2 rank + rot_dim) / (key_dim + rot_dim + value_dim) times that; the expanded pages live for the step only.
With a window or a sink the expanded pages go through the windowed family's kernels (`kernels.attention_sink`), and a
windowed step only expands when its sequences are not much longer than what its tokens see.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import copy

import torch

from .. import kernels as K
from ..registry import register_part
from ..weights.loader import TensorSpec
from .base import CacheNeed, Part
from .linear import Linear

BLOCKS_PER_SM = 2     # blocks of the attention kernel a step should offer every multiprocessor
EXPAND_TOKENS = 16    # from this many new tokens of a sequence on, a bfloat16 step writes out keys and values of the heads
EXPAND_SPAN = 4       # ... with a window only while the longest sequence is at most this many times (new tokens + window) long
NO_WINDOW = 1 << 30   # what the windowed family's kernels take for "every earlier key"


@dataclass(frozen=True)
class LatentAttentionSpec:
    hidden_size: int
    n_heads: int
    key_dim: int                  # unrotated lanes of a head's query and key
    rot_dim: int                  # rotated lanes of a head's query; the key's are shared by the heads
    value_dim: int
    rank: int                     # lanes of the cached latent
    scale: float
    rotary_dims: int              # how many of the rot_dim lanes turn
    rotary_base: float
    eps: float                    # of the latent's norm
    output_gate: bool = True
    q_rank: Optional[int] = None  # lanes of the queries' latent; None: q = Wq h
    rotary_halves: bool = False   # lanes (m, m + rotary_dims / 2) turn together instead of (2m, 2m + 1)
    window: Optional[int] = None  # None: every earlier position
    sink: bool = False            # a stored number per head joins the softmax's denominator
    gate_per_head: bool = False   # the gate is a number per head instead of one per value lane


@register_part("mixer", "latent_attention")
class LatentAttention(Part):
    family = "mixer"
    graph_safe = True
    roles = ("q", "dq", "q_norm", "uq", "dkv", "c_norm", "uk", "uv", "g", "o", "sink")
    kernel_modules = ("elementwise", "attention_latent", "attention", "attention_sink", "gemm")

    def __init__(self, spec, tensors, runtime):
        super().__init__(spec, tensors, runtime)
        if spec.rotary_dims % 2 or spec.rotary_dims > spec.rot_dim:
            raise ValueError(f"{spec.rotary_dims} turning lanes of {spec.rot_dim}: an even number, at most all of them")
        if spec.window is not None and spec.window < 1:
            raise ValueError(f"a window of {spec.window}")
        self.q_cols = spec.n_heads * (spec.key_dim + spec.rot_dim)
        self.down_cols = spec.rank + spec.rot_dim
        self.v_cols = spec.n_heads * spec.value_dim
        self.gate_cols = spec.n_heads if spec.gate_per_head else self.v_cols
        # long portions run the grouped-query kernels on keys and values written out: the windowed family's with a window
        # or a sink, the dense decoder's without (only the one this mixer uses is compiled before the first step)
        self.kernel_modules = ("elementwise", "attention_latent", "gemm",
                               "attention_sink" if spec.window is not None or spec.sink else "attention")

    def tensor_specs(self):
        s, t = self.spec, self.tensor_names
        if s.q_rank:
            specs = [TensorSpec(t["dq"], (s.q_rank, s.hidden_size)), TensorSpec(t["q_norm"], (s.q_rank,), init="one_plus_normal:0.1"),
                     TensorSpec(t["uq"], (self.q_cols, s.q_rank))]
        else:
            specs = [TensorSpec(t["q"], (self.q_cols, s.hidden_size))]
        specs += [TensorSpec(t["dkv"], (self.down_cols, s.hidden_size)),
                 TensorSpec(t["c_norm"], (s.rank,), init="one_plus_normal:0.1"),
                 TensorSpec(t["uk"], (s.n_heads * s.key_dim, s.rank), init="normal:0.1"),
                 TensorSpec(t["uv"], (self.v_cols, s.rank), init="normal:0.1"),
                 TensorSpec(t["o"], (s.hidden_size, self.v_cols))]
        if s.output_gate:
            specs.append(TensorSpec(t["g"], (self.gate_cols, s.hidden_size)))
        if s.sink:
            specs.append(TensorSpec(t["sink"], (s.n_heads,), init="normal:1.0"))
        return specs

    def bind(self, loaded):
        s, t = self.spec, self.tensor_names
        ws = ([] if s.q_rank else [loaded[t["q"]]]) + [loaded[t["dkv"]]] + ([loaded[t["g"]]] if s.output_gate else [])
        if len({w.dtype for w in ws}) != 1:
            raise ValueError(f"the projections of {t['dkv']} and its neighbours are stored in different dtypes")
        self.proj = Linear(torch.cat(ws, dim=0).contiguous())        # [q | c, k_rot | gate], kept in fp32 for norm and rotation
        if s.q_rank:                                                 # the queries' own latent: down, norm, up
            self.dq, self.uq = Linear(loaded[t["dq"]]), Linear(loaded[t["uq"]])
            self.q_weight = loaded[t["q_norm"]].to(torch.float32).contiguous()
        self.sink = loaded[t["sink"]].to(torch.float32).contiguous() if s.sink else None
        self.o = Linear(loaded[t["o"]])
        dt = self.runtime.dtype
        # per head: [rank, key_dim] (the transposed up-projection of the keys) and [value_dim, rank]
        self.uk_t = loaded[t["uk"]].to(dt).view(s.n_heads, s.key_dim, s.rank).transpose(1, 2).contiguous()
        self.uv = loaded[t["uv"]].to(dt).view(s.n_heads, s.value_dim, s.rank).contiguous()
        self.c_weight = loaded[t["c_norm"]].to(torch.float32).contiguous()
        # whole heads for long prompts: [unrotated | rotated] keys padded to a head size the prompt kernels take
        wide = s.key_dim + s.rot_dim
        self.expand_hd = 64 if wide <= 64 else 128
        self.expands = dt == torch.bfloat16 and wide <= 128 and s.value_dim <= self.expand_hd
        if self.expands:
            self.up = Linear(torch.cat([loaded[t["uk"]], loaded[t["uv"]]], dim=0).to(dt).contiguous())   # [H dk + H dv, rank]
        self.freq = None
        if s.rotary_dims:
            self.freq = torch.tensor([s.rotary_base ** (-2.0 * i / s.rotary_dims) for i in range(s.rotary_dims // 2)],
                                     dtype=torch.float64).to(self.c_weight.device)

    def cache_need(self) -> CacheNeed:
        return CacheNeed("rows", n_kv_heads=1, head_dim=self.down_cols, window=self.spec.window)

    def _projections(self, x):
        """(q [N, heads * (key_dim + rot_dim)], [c | k_rot] [N, rank + rot_dim], gate or None): float32, column ranges of
        wider products."""
        s = self.spec
        proj = self.proj(x, out_dtype=torch.float32)
        if s.q_rank:
            wide = self.dq(x, out_dtype=torch.float32)
            cq = torch.empty(wide.shape, dtype=self.runtime.dtype, device=wide.device)
            K.add_rmsnorm(wide, None, self.q_weight, s.eps, cq)
            q, at = self.uq(cq, out_dtype=torch.float32), 0
        else:
            q, at = proj[:, :self.q_cols], self.q_cols
        gate = proj[:, at + self.down_cols:at + self.down_cols + self.gate_cols] if s.output_gate else None
        return q, proj[:, at:at + self.down_cols], gate

    def _gate(self, heads, gate):
        if gate is not None:
            K.sigmoid_gate(heads, gate, heads, share=self.spec.value_dim if self.spec.gate_per_head else 1)

    def _splits(self, step) -> int:
        """Over how many blocks a row's keys are cut: a few tokens with many keys leave most multiprocessors idle
        otherwise.  Every block should still have a few pages."""
        s = self.spec
        rows = K.latent_attention_tile_rows(self.runtime.dtype, s.n_heads, s.rank, s.rot_dim, step.max_q_len)
        tiles = (step.max_q_len * s.n_heads + rows - 1) // rows * step.n_seqs
        want = BLOCKS_PER_SM * K.sm_count(self.runtime.device)
        seen = step.max_kv_len if s.window is None else min(step.max_kv_len, s.window + step.max_q_len)
        return max(1, min(want // tiles, seen // (2 * K.PAGE), 32))                # no block left over for a second round

    def forward(self, x, step, cache):
        s, rt = self.spec, self.runtime
        if not cache.writes:
            raise ValueError("this mixer appends to a cache line of its own; it cannot read another run's")
        n, dev = step.n_tokens, x.device
        q_proj, down, gate = self._projections(x)                    # fp32
        if (self.expands and step.max_q_len >= EXPAND_TOKENS
                and (s.window is None or step.max_kv_len <= EXPAND_SPAN * (step.max_q_len + s.window))):
            return self._forward_expanded(q_proj, down, gate, step, cache)
        q_nope = torch.empty((s.n_heads, n, s.key_dim), dtype=rt.dtype, device=dev)
        q_rot = torch.empty((n, s.n_heads, s.rot_dim), dtype=torch.float32, device=dev)
        K.latent_prepare(q_proj, down, self.c_weight, s.eps, self.freq, s.rotary_dims, q_nope, q_rot, cache.pool, cache.block_table,
                         step, s.n_heads, s.key_dim, s.rot_dim, s.rank, halves=s.rotary_halves)
        q_lat = K.batched_product(q_nope, self.uk_t, out_dtype=torch.float32)            # [H, N, rank]
        mixed = torch.zeros((s.n_heads, n, s.rank), dtype=rt.dtype, device=dev)          # rows of no sequence stay zero
        n_splits = self._splits(step)
        partial = None
        if n_splits > 1:
            partial = step.workspace.scratch("latent_attention",
                                             K.latent_attention_scratch_floats(n, s.n_heads, s.rank, n_splits))
        K.latent_attention(q_lat, q_rot, cache.pool, cache.block_table, step, mixed, s.n_heads, s.rank, s.rot_dim, s.scale,
                           n_splits=n_splits, partial=partial, window=s.window or 0, sink=self.sink)
        heads = torch.empty((n, self.v_cols), dtype=rt.dtype, device=dev)
        K.batched_product(mixed, self.uv, out=heads.view(n, s.n_heads, s.value_dim).transpose(0, 1))
        self._gate(heads, gate)
        return self.o(heads, out_dtype=torch.float32)

    def _forward_expanded(self, q_proj, down, gate, step, cache):
        """Long prompts: attention on keys and values written out for all heads (see the module's head)."""
        s, rt, hd = self.spec, self.runtime, self.expand_hd
        n, dev, lanes = step.n_tokens, q_proj.device, self.down_cols
        q = torch.empty((n, s.n_heads, hd), dtype=rt.dtype, device=dev)
        K.latent_prepare(q_proj, down, self.c_weight, s.eps, self.freq, s.rotary_dims, None, None, cache.pool, cache.block_table,
                         step, s.n_heads, s.key_dim, s.rot_dim, s.rank, q_full=q, halves=s.rotary_halves)
        pages_each = (step.max_kv_len + K.PAGE - 1) // K.PAGE
        n_pages = step.n_seqs * pages_each
        rows = n_pages * K.PAGE
        page_elems = 2 * s.n_heads * K.PAGE * hd
        work = step.workspace.scratch("latent_expanded", (rows * lanes + n_pages * page_elems + 1) // 2 + 8).view(rt.dtype)
        gathered = work[:rows * lanes].view(rows, lanes)
        pages = work[(rows * lanes + 7) // 8 * 8:][:n_pages * page_elems].view(n_pages, 2, s.n_heads, K.PAGE, hd)
        K.latent_gather(cache.pool, cache.block_table, step, gathered, pages_each, lanes, window=s.window or 0)
        kv = self.up(gathered[:, :s.rank], out_dtype=rt.dtype)       # [rows, H key_dim | H value_dim]
        K.latent_expand(kv, gathered, pages, s.n_heads, s.key_dim, s.rot_dim, s.value_dim, s.rank)
        table = torch.arange(n_pages, dtype=torch.int32, device=dev).view(step.n_seqs, pages_each)
        own = torch.arange(step.n_seqs, dtype=torch.int32, device=dev)
        out = torch.zeros((n, s.n_heads * hd), dtype=rt.dtype, device=dev)               # rows of no sequence stay zero
        if s.window is None and self.sink is None:
            K.attention(q, s.n_heads * hd, pages, table, step.cu_seqlens, own, step.start_pos, out, n, step.n_seqs, step.max_q_len,
                        s.n_heads, s.n_heads, hd, s.scale, max_kv_len=step.max_kv_len)
        else:
            own_step = copy.copy(step)                     # the expanded pages have a table of their own: sequence s is its row s
            own_step.slot_of_seq = own
            K.attention_sink(q.view(n, s.n_heads * hd), own_step, pages, table, out, s.n_heads,
                             s.n_heads, hd, hd, s.scale, s.window or NO_WINDOW, 0, sink=self.sink is not None, sink_logit=self.sink,
                             max_q_len=step.max_q_len)
        heads = out
        if s.value_dim != hd:
            heads = torch.empty((n, self.v_cols), dtype=rt.dtype, device=dev)
            heads.view(n, s.n_heads, s.value_dim).copy_(out.view(n, s.n_heads, hd)[:, :, :s.value_dim])
        self._gate(heads, gate)
        return self.o(heads, out_dtype=torch.float32)
