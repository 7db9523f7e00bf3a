"""Attention over a cached latent: keys and values of all heads are made from one small vector per position.

q = Wq h, a head's lanes laid out as [key_dim unrotated | rot_dim rotated]; Wdkv h has rank + rot_dim rows: the first
`rank`, RMS-normed with a plain weight, are the latent c, the last rot_dim one rotated key part that all heads share.
Head i's unrotated key is Wuk_i c and its value Wuv_i c; its score is (q_nope . Wuk_i c + q_rot . k_rot) * scale, softmax
over the positions j <= i.  The rotation turns the lane pairs (2m, 2m + 1), m < rot_dims / 2, of the rotated parts by
position * base^(-2m / rot_dims); lanes from rot_dims on pass unchanged.  The concatenated heads are multiplied by
sigmoid(Wg h) and projected by Wo.

Only c and the rotated key part are cached (a paged line of rows of rank + rot_dim lanes).  Because key and value are
linear in c, the up-projections are taken off the cached side: q' = Wuk_i^T q_nope is a small batched product in front of
the attention kernel, which then works on the latent itself (score q' . c + q_rot . k_rot, output sum_j p_j c_j), and
Wuv_i is a batched product behind it.

Steps that bring 16 or more tokens of a sequence in bfloat16 go the other way round when a head's key ([unrotated |
rotated]) fits 128 lanes: the latents of the step's sequences are gathered, one product makes every head's unrotated
keys and values from them, and the grouped-query attention kernels (the tensor-core ones for prompts) run on those
pages with as many key/value heads as query heads.  A prompt's attention then costs what a dense decoder's costs
instead of (2 rank + rot_dim) / (key_dim + rot_dim + value_dim) times that; the expanded pages live for the step only.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from .. import kernels as K
from ..registry import register_part
from ..weights.loader import TensorSpec
from .base import CacheNeed, Part
from .linear import Linear

BLOCKS_PER_SM = 2     # blocks of the attention kernel a step should offer every multiprocessor
EXPAND_TOKENS = 16    # from this many new tokens of a sequence on, a bfloat16 step writes out keys and values of the heads


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


@register_part("mixer", "latent_attention")
class LatentAttention(Part):
    family = "mixer"
    graph_safe = True
    roles = ("q", "dkv", "c_norm", "uk", "uv", "g", "o")
    kernel_modules = ("elementwise", "attention_latent", "attention", "gemm")

    def __init__(self, spec, tensors, runtime):
        super().__init__(spec, tensors, runtime)
        if spec.rotary_dims % 2 or spec.rotary_dims > spec.rot_dim:
            raise ValueError(f"{spec.rotary_dims} turning lanes of {spec.rot_dim}: an even number, at most all of them")
        self.q_cols = spec.n_heads * (spec.key_dim + spec.rot_dim)
        self.down_cols = spec.rank + spec.rot_dim
        self.v_cols = spec.n_heads * spec.value_dim

    def tensor_specs(self):
        s, t = self.spec, self.tensor_names
        specs = [TensorSpec(t["q"], (self.q_cols, s.hidden_size)), TensorSpec(t["dkv"], (self.down_cols, s.hidden_size)),
                 TensorSpec(t["c_norm"], (s.rank,), init="one_plus_normal:0.1"),
                 TensorSpec(t["uk"], (s.n_heads * s.key_dim, s.rank), init="normal:0.1"),
                 TensorSpec(t["uv"], (self.v_cols, s.rank), init="normal:0.1"),
                 TensorSpec(t["o"], (s.hidden_size, self.v_cols))]
        if s.output_gate:
            specs.append(TensorSpec(t["g"], (self.v_cols, s.hidden_size)))
        return specs

    def bind(self, loaded):
        s, t = self.spec, self.tensor_names
        ws = [loaded[t["q"]], loaded[t["dkv"]]] + ([loaded[t["g"]]] if s.output_gate else [])
        if len({w.dtype for w in ws}) != 1:
            raise ValueError(f"the projections of {t['q']} and its neighbours are stored in different dtypes")
        self.proj = Linear(torch.cat(ws, dim=0).contiguous())        # [q | c, k_rot | gate], kept in fp32 for norm and rotation
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
        return CacheNeed("rows", n_kv_heads=1, head_dim=self.down_cols)

    def _splits(self, step) -> int:
        """Over how many blocks a row's keys are cut: a few tokens with many keys leave most multiprocessors idle
        otherwise.  Every block should still have a few pages."""
        s = self.spec
        rows = K.latent_attention_tile_rows(self.runtime.dtype, s.n_heads, s.rank, s.rot_dim, step.max_q_len)
        tiles = (step.max_q_len * s.n_heads + rows - 1) // rows * step.n_seqs
        want = BLOCKS_PER_SM * K.sm_count(self.runtime.device)
        return max(1, min(want // tiles, step.max_kv_len // (2 * K.PAGE), 32))     # no block left over for a second round

    def forward(self, x, step, cache):
        s, rt = self.spec, self.runtime
        if not cache.writes:
            raise ValueError("this mixer appends to a cache line of its own; it cannot read another run's")
        n, dev = step.n_tokens, x.device
        proj = self.proj(x, out_dtype=torch.float32)                 # [N, q | down | gate] in fp32
        if self.expands and step.max_q_len >= EXPAND_TOKENS:
            return self._forward_expanded(proj, step, cache)
        q_nope = torch.empty((s.n_heads, n, s.key_dim), dtype=rt.dtype, device=dev)
        q_rot = torch.empty((n, s.n_heads, s.rot_dim), dtype=torch.float32, device=dev)
        K.latent_prepare(proj[:, :self.q_cols], proj[:, self.q_cols:self.q_cols + self.down_cols], self.c_weight, s.eps,
                         self.freq, s.rotary_dims, q_nope, q_rot, cache.pool, cache.block_table, step, s.n_heads, s.key_dim,
                         s.rot_dim, s.rank)
        q_lat = K.batched_product(q_nope, self.uk_t, out_dtype=torch.float32)            # [H, N, rank]
        mixed = torch.zeros((s.n_heads, n, s.rank), dtype=rt.dtype, device=dev)          # rows of no sequence stay zero
        n_splits = self._splits(step)
        partial = None
        if n_splits > 1:
            partial = step.workspace.scratch("latent_attention",
                                             K.latent_attention_scratch_floats(n, s.n_heads, s.rank, n_splits))
        K.latent_attention(q_lat, q_rot, cache.pool, cache.block_table, step, mixed, s.n_heads, s.rank, s.rot_dim, s.scale,
                           n_splits=n_splits, partial=partial)
        heads = torch.empty((n, self.v_cols), dtype=rt.dtype, device=dev)
        K.batched_product(mixed, self.uv, out=heads.view(n, s.n_heads, s.value_dim).transpose(0, 1))
        if s.output_gate:
            gate_at = self.q_cols + self.down_cols
            K.sigmoid_gate(heads, proj[:, gate_at:gate_at + self.v_cols], heads)
        return self.o(heads, out_dtype=torch.float32)

    def _forward_expanded(self, proj, step, cache):
        """Long prompts: attention on keys and values written out for all heads (see the module's head)."""
        s, rt, hd = self.spec, self.runtime, self.expand_hd
        n, dev, lanes = step.n_tokens, proj.device, self.down_cols
        q = torch.empty((n, s.n_heads, hd), dtype=rt.dtype, device=dev)
        K.latent_prepare(proj[:, :self.q_cols], proj[:, self.q_cols:self.q_cols + self.down_cols], self.c_weight, s.eps,
                         self.freq, s.rotary_dims, None, None, cache.pool, cache.block_table, step, s.n_heads, s.key_dim,
                         s.rot_dim, s.rank, q_full=q)
        pages_each = (step.max_kv_len + K.PAGE - 1) // K.PAGE
        n_pages = step.n_seqs * pages_each
        rows = n_pages * K.PAGE
        page_elems = 2 * s.n_heads * K.PAGE * hd
        work = step.workspace.scratch("latent_expanded", (rows * lanes + n_pages * page_elems + 1) // 2 + 8).view(rt.dtype)
        gathered = work[:rows * lanes].view(rows, lanes)
        pages = work[(rows * lanes + 7) // 8 * 8:][:n_pages * page_elems].view(n_pages, 2, s.n_heads, K.PAGE, hd)
        K.latent_gather(cache.pool, cache.block_table, step, gathered, pages_each, lanes)
        kv = self.up(gathered[:, :s.rank], out_dtype=rt.dtype)       # [rows, H key_dim | H value_dim]
        K.latent_expand(kv, gathered, pages, s.n_heads, s.key_dim, s.rot_dim, s.value_dim, s.rank)
        table = torch.arange(n_pages, dtype=torch.int32, device=dev).view(step.n_seqs, pages_each)
        own = torch.arange(step.n_seqs, dtype=torch.int32, device=dev)
        out = torch.zeros((n, s.n_heads * hd), dtype=rt.dtype, device=dev)               # rows of no sequence stay zero
        K.attention(q, s.n_heads * hd, pages, table, step.cu_seqlens, own, step.start_pos, out, n, step.n_seqs, step.max_q_len,
                    s.n_heads, s.n_heads, hd, s.scale, max_kv_len=step.max_kv_len)
        heads = out
        if s.value_dim != hd:
            heads = torch.empty((n, self.v_cols), dtype=rt.dtype, device=dev)
            heads.view(n, s.n_heads, s.value_dim).copy_(out.view(n, s.n_heads, hd)[:, :, :s.value_dim])
        if s.output_gate:
            gate_at = self.q_cols + self.down_cols
            K.sigmoid_gate(heads, proj[:, gate_at:gate_at + self.v_cols], heads)
        return self.o(heads, out_dtype=torch.float32)
