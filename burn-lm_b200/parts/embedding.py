"""Token embedding (a row gather, no scale: crates/burn-lm-llama/src/nn/transformer.rs:95) and the
output projection to fp32 logits (transformer.rs:101-102; with tie_word_embeddings the head reads
the embedding table, which the reference leaves as a TODO at :82-84).
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from typing import Optional

from .. import kernels as K
from ..plan import PartPlan
from ..registry import part_class, register_part
from ..weights.loader import TensorSpec
from .base import CacheNeed, Part
from .linear import HandedNorm, Linear


@dataclass(frozen=True)
class EmbeddingSpec:
    vocab_size: int
    hidden_size: int


@register_part("embedding", "table")
class Embedding(Part):
    family = "embedding"
    graph_safe = True
    roles = ("table",)

    def tensor_specs(self):
        return [TensorSpec(self.tensor_names["table"], (self.spec.vocab_size, self.spec.hidden_size))]

    def bind(self, loaded):
        self.table = loaded[self.tensor_names["table"]]

    hands_norm_over = True      # forward() takes the step's handoff and may leave the first norm's input there

    def forward(self, tokens, out, handoff=None):
        """`handoff` (parts.linear.NormHandoff) with a norm expected: for a few tokens the kernel also leaves that
        norm's input (the stream times gamma, the rows' sums of squares), as the products that write the stream do."""
        norm = handoff.wanted if handoff is not None else None
        n = tokens.numel()
        if (norm is not None and n <= K.SQUARES_ROWS and self.runtime.dtype == torch.bfloat16 and out.is_cuda
                and getattr(norm, "gamma", None) is not None and norm.gamma.numel() == out.shape[1]):
            handed = HandedNorm(torch.empty((n, out.shape[1]), dtype=torch.bfloat16, device=out.device),
                                torch.empty((1, K.SQUARES_ROWS), dtype=torch.float32, device=out.device))
            K.embed(tokens, self.table, out, hand_over=(norm.gamma, handed.scaled, handed.squares))
            handoff.leave(out, norm.gamma, handed)
            return
        K.embed(tokens, self.table, out)


@dataclass(frozen=True)
class ScaledEmbeddingSpec:
    vocab_size: int
    hidden_size: int
    scale: float


@register_part("embedding", "scaled_table")
class ScaledEmbedding(Part):
    """x = table[token] * scale, the product taken in fp32; the table itself stays as stored (a tied head reads it unscaled)."""
    family = "embedding"
    graph_safe = True
    roles = ("table",)
    kernel_modules = ("stream_ops",)

    def tensor_specs(self):
        return [TensorSpec(self.tensor_names["table"], (self.spec.vocab_size, self.spec.hidden_size))]

    def bind(self, loaded):
        self.table = loaded[self.tensor_names["table"]]

    def forward(self, tokens, out):
        K.embed_scaled(tokens, self.table, out, self.spec.scale)


@dataclass(frozen=True)
class PairEmbeddingSpec:
    vocab_size: int
    hidden_size: int
    buckets: int                       # rows of the table of pairs, not counting its last row (a sequence's first token)
    mul_prev: int
    mul_cur: int
    norm: Optional[PartPlan] = None    # family "norm": applied to the sum before it enters the stream


@register_part("embedding", "token_pairs")
class PairEmbedding(Part):
    """x = table[token] + pairs[(previous token * mul_prev + token * mul_cur) mod buckets], the table's last row for a
    sequence's first token, then an optional norm.  The previous token is part of what a sequence keeps: the part
    asks the cache for a paged line of token ids, one per position, so that a step repeated or run ahead and
    forgotten leaves nothing wrong behind, as with keys and values."""
    family = "embedding"
    graph_safe = True
    roles = ("table", "pairs")
    kernel_modules = ("elementwise",)
    takes_step = True

    def __init__(self, spec, tensors, runtime):
        super().__init__(spec, tensors, runtime)
        self.norm = None
        if spec.norm is not None:
            self.norm = part_class("norm", spec.norm.kind)(spec.norm.spec, spec.norm.tensors, runtime)
            if not hasattr(self.norm, "parameters"):
                raise ValueError(f"the embedding applies its norm in its own kernel, which knows 'dynamic_tanh'; got {spec.norm.kind!r}")

    def tensor_specs(self):
        s, t = self.spec, self.tensor_names
        return [TensorSpec(t["table"], (s.vocab_size, s.hidden_size)), TensorSpec(t["pairs"], (s.buckets + 1, s.hidden_size))] \
            + (self.norm.tensor_specs() if self.norm is not None else [])

    def bind(self, loaded):
        self.table, self.pairs = loaded[self.tensor_names["table"]], loaded[self.tensor_names["pairs"]]
        if self.table.dtype != self.pairs.dtype:
            raise ValueError(f"{self.tensor_names['table']} and {self.tensor_names['pairs']} are stored in different dtypes")
        if self.norm is not None:
            self.norm.bind(loaded)

    def cache_need(self) -> CacheNeed:
        return CacheNeed("ids", window=2)       # a coming token looks one position back

    def forward(self, tokens, out, step=None, cache=None):
        s = self.spec
        K.embed_pairs(tokens, self.table, self.pairs, out, step, cache.pool, cache.block_table, s.buckets, s.mul_prev, s.mul_cur,
                      norm=self.norm.parameters() if self.norm is not None else None)


@dataclass(frozen=True)
class HeadSpec:
    vocab_size: int
    hidden_size: int


@register_part("head", "linear")
class Head(Part):
    """logits = x W^T in fp32; `weight` may name the embedding table (tied)."""
    family = "head"
    graph_safe = True
    roles = ("weight",)

    def tensor_specs(self):
        return [TensorSpec(self.tensor_names["weight"], (self.spec.vocab_size, self.spec.hidden_size))]

    def bind(self, loaded):
        self.linear = Linear(loaded[self.tensor_names["weight"]])

    takes_pending_norm = True

    def forward(self, x):
        return self.linear(x, out_dtype=torch.float32)


@dataclass(frozen=True)
class NormedEmbeddingSpec:
    vocab_size: int
    hidden_size: int
    eps: float


@register_part("embedding", "normed_table")
class NormedEmbedding(Part):
    """x = table[token] / sqrt(mean(table[token]^2) + eps) * weight: the row, RMS-normed in fp32 where it lies in the stream."""
    family = "embedding"
    graph_safe = True
    roles = ("table", "norm")
    kernel_modules = ("elementwise",)

    def tensor_specs(self):
        s, t = self.spec, self.tensor_names
        return [TensorSpec(t["table"], (s.vocab_size, s.hidden_size)),
                TensorSpec(t["norm"], (s.hidden_size,), init="one_plus_normal:0.1")]

    def bind(self, loaded):
        self.table = loaded[self.tensor_names["table"]]
        self.gamma = loaded[self.tensor_names["norm"]].to(torch.float32).contiguous()

    def forward(self, tokens, out):
        K.embed(tokens, self.table, out)
        K.add_rmsnorm(out, None, self.gamma, self.spec.eps, out)


@dataclass(frozen=True)
class CappedHeadSpec:
    vocab_size: int
    hidden_size: int
    cap: Optional[float] = None        # logits <- cap * tanh(logits / cap); None: as they are


@register_part("head", "capped_linear")
class CappedHead(Head):
    """logits = x W^T in fp32, then squashed into (-cap, cap)."""
    kernel_modules = ("elementwise", "stream_ops")

    def forward(self, x):
        logits = self.linear(x, out_dtype=torch.float32)
        if self.spec.cap:
            K.softcap(logits, self.spec.cap)
        return logits
