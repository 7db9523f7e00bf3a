"""The cache of a model: a slot per sequence, keys and values per run of the schedule, each
sequence with its own length, and a fixed-size state per sequence beside it.

Storage is sized in tokens.  Keys and values live in pages of 64 positions; a sequence holds as
many pages as its length needs, listed in its row of the block table, so `max_tokens` bounds the sum
over live sequences of their lengths rounded up to 64, whatever their number.  Runs of the schedule
whose mixers need the same thing (all keys of n heads of size d; a window; a state of some shape)
form a group with storage, page allocator and block table of its own.  A group whose mixers look
back over a window only gives a sequence's pages back as soon as every key in them lies before the
window of every token still to come, so a long sequence holds about window / 64 + 2 of its pages.
Pages and slots are given back when a sequence ends and are used again without being cleared: a
kernel never reads a position at or beyond a sequence's length, nor one before the window.  State
blocks are zeroed when a slot is acquired.

The reference preallocates [max_batch, kv heads, max_seq_len, head_dim] per layer with one length
for the whole batch (crates/burn-lm-llama/src/nn/attention/kv_cache.rs:14-34, nn/transformer.rs:
118-146); slots, pages and per-sequence lengths are this package's own.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from ..kernels import PAGE
from .allocators import CacheError, CacheFull, ContextLengthExceeded, IdAllocator


@dataclass
class CacheView:
    """What one run of the schedule sees of the cache."""
    kind: str                               # "kv", "ids", "rows", "state" or "none"; several joined by '+' 
    writes: bool                            # False: the line belongs to an earlier run; read only
    pool: Optional[torch.Tensor] = None     # kv: [pages, 2, n_kv_heads, PAGE, head_dim]; with values of another size than
                                            # the keys [pages, n_kv_heads * PAGE * (head_dim + value_dim)], a page's keys
                                            # [n_kv_heads, PAGE, head_dim] followed by its values [n_kv_heads, PAGE, value_dim];
                                            # ids: int32 [pages, PAGE]; rows: [pages, PAGE, head_dim]
    block_table: Optional[torch.Tensor] = None   # kv: int32 [max_seqs, max_pages_per_seq]
    state: Optional[torch.Tensor] = None    # state: [max_seqs, *state_shape]
    state_offset: int = 0                   # floats of a state copy that lie before the reader's own (a block that keeps
                                            # something of its own in the same state block puts its mixer behind it)
    window: Optional[int] = None
    keep_first: int = 0


class _KVGroup:
    def __init__(self, need, runs, n_pages, max_seqs, max_pages_per_seq, dtype, device):
        self.need, self.runs = need, list(runs)
        if need.kind == "ids":
            self.pool = torch.zeros((len(runs), n_pages, PAGE), dtype=torch.int32, device=device)
        elif need.kind == "rows":
            self.pool = torch.empty((len(runs), n_pages, PAGE, need.head_dim), dtype=dtype, device=device)
        elif need.value_dim is None or need.value_dim == need.head_dim:
            self.pool = torch.empty((len(runs), n_pages, 2, need.n_kv_heads, PAGE, need.head_dim), dtype=dtype, device=device)
        else:
            self.pool = torch.empty((len(runs), n_pages, need.n_kv_heads * PAGE * (need.head_dim + need.value_dim)),
                                    dtype=dtype, device=device)
        # leading pages that hold some of the first `keep_first` positions: a windowed group never gives them back
        self.kept_pages = (need.keep_first + PAGE - 1) // PAGE if need.window else 0
        self.pages = IdAllocator(n_pages, "cache page")
        self.block_table = torch.zeros((max_seqs, max_pages_per_seq), dtype=torch.int32, device=device)
        # pages_of[slot][i]: the page that holds positions 64 i .. 64 i + 63 of the slot's sequence, or None once a
        # windowed group has given it back; dropped[slot]: the pages kept_pages .. dropped - 1 have been given back
        self.pages_of: list[list] = [[] for _ in range(max_seqs)]
        self.dropped = [0] * max_seqs

    def live_pages(self, slot: int) -> list:
        return [p for p in self.pages_of[slot] if p is not None]

    def drop_before_window(self, slot: int, length: int) -> None:
        """`length`: how long the slot's sequence is now; the tokens still to come sit at positions >= length and see
        the keys from length - window + 1 on.  Pages that lie wholly before that are given back."""
        if not self.need.window:
            return
        first_needed = max(0, length - self.need.window + 1) // PAGE
        last = min(first_needed, len(self.pages_of[slot]))
        start = max(self.dropped[slot], self.kept_pages)
        if last > start:
            for i in range(start, last):
                self.pages.release(self.pages_of[slot][i])
                self.pages_of[slot][i] = None
            # the table's entries stay valid page numbers: no kernel reads them, but none may point outside the pool
            self.block_table[slot, start:last] = 0
            self.dropped[slot] = last

    def bytes(self):
        return self.pool.numel() * self.pool.element_size()


class _StateGroup:
    def __init__(self, need, runs, max_seqs, compute_dtype, device):
        self.need, self.runs = need, list(runs)
        dt = compute_dtype if need.state_dtype == "compute" else getattr(torch, need.state_dtype)
        self.state = torch.zeros((len(runs), max_seqs, *need.state_shape), dtype=dt, device=device)


class Cache:
    def __init__(self, needs: list, schedule, max_tokens: int, max_seqs: int, max_seq_len: int, dtype, device, named=None):
        """needs[run]: CacheNeed of every run of the schedule (None where the run reads another's).  `named`: what parts
        outside the layers keep per sequence (the embedding, say), name -> CacheNeed; their views are `named_view(name)`."""
        if max_tokens < 1 or max_seqs < 1 or max_seq_len < 1:
            raise CacheError("the cache needs room for at least one token of one sequence")
        self.max_tokens, self.max_seqs, self.max_seq_len = max_tokens, max_seqs, max_seq_len
        self.n_pages = (max_tokens + PAGE - 1) // PAGE
        self.max_pages_per_seq = min((max_seq_len + PAGE - 1) // PAGE, self.n_pages)
        self.dtype, self.device = dtype, device
        self.slots = IdAllocator(max_seqs, "sequence slot")
        self.seq_len = [0] * max_seqs
        self._kv_groups: list[_KVGroup] = []
        self._state_groups: list[_StateGroup] = []
        self._where: dict[int, tuple] = {}      # run -> ("kv" | "state" | "none", group, index in group)
        by_need: dict = {}
        several: dict[int, int] = {}            # run -> how many needs it has, when its mixer keeps several things
        for run, need in enumerate(needs):
            if isinstance(need, tuple):
                several[run] = len(need)
                for j, one in enumerate(need):
                    by_need.setdefault(one, []).append((run, j))
            elif need is not None:
                by_need.setdefault(need, []).append(run)
        for name, need in (named or {}).items():
            by_need.setdefault(need, []).append(("named", name))
        for need, runs in by_need.items():
            if need.kind in ("kv", "ids", "rows"):
                # (a windowed group has storage of its own; the window is applied in the kernels, and the
                # group gives the pages before it back as the sequence grows)
                g = _KVGroup(need, runs, self.n_pages, max_seqs, self.max_pages_per_seq, dtype, device)
                self._kv_groups.append(g)
                for i, r in enumerate(runs):
                    self._where[r] = ("kv", g, i)
            elif need.kind == "state":
                g = _StateGroup(need, runs, max_seqs, dtype, device)
                self._state_groups.append(g)
                for i, r in enumerate(runs):
                    self._where[r] = ("state", g, i)
            elif need.kind == "none":
                for r in runs:
                    self._where[r] = ("none", None, 0)
            else:
                raise CacheError(f"unknown cache need {need.kind!r}")
        self._views = []
        for run, entry in enumerate(schedule):
            src = run if entry.cache_of is None else entry.cache_of
            writes = entry.cache_of is None
            if src in several:
                self._views.append(self._merged([self._view_of(*self._where[(src, j)], writes) for j in range(several[src])]))
                continue
            kind, g, i = self._where[src]
            self._views.append(self._view_of(kind, g, i, writes))
        self._named_views = {name: self._view_of(*self._where[("named", name)], True) for name in (named or {})}

    @staticmethod
    def _view_of(kind, g, i, writes):
        if kind == "kv":
            return CacheView(g.need.kind, writes, pool=g.pool[i], block_table=g.block_table, window=g.need.window,
                             keep_first=g.need.keep_first)
        if kind == "state":
            return CacheView("state", writes, state=g.state[i])
        return CacheView("none", writes)

    @staticmethod
    def _merged(views):
        """One view of a run whose mixer keeps several things (keys and values beside a state, say): at most one of
        each kind; the fields of both are filled and `kind` names them joined by '+'."""
        kinds = [v.kind for v in views if v.kind != "none"]
        if len(set(kinds)) != len(kinds):
            raise CacheError(f"a run keeps two things of one kind: {kinds}")
        out = CacheView("+".join(kinds) if kinds else "none", views[0].writes)
        for v in views:
            if v.kind in ("kv", "ids", "rows"):
                out.pool, out.block_table, out.window, out.keep_first = v.pool, v.block_table, v.window, v.keep_first
            elif v.kind == "state":
                out.state = v.state
        return out

    # -- what the model sees -------------------------------------------------------------------------
    def view(self, run: int) -> CacheView:
        return self._views[run]

    def named_view(self, name: str) -> CacheView:
        return self._named_views[name]

    def bytes(self) -> int:
        return sum(g.bytes() for g in self._kv_groups)

    @property
    def free_pages(self) -> int:
        return min((g.pages.free_count for g in self._kv_groups), default=self.n_pages)

    # -- sequences -----------------------------------------------------------------------------------
    def acquire(self) -> int:
        """A free slot for a new sequence of length 0; its state blocks are zeroed."""
        slot = self.slots.acquire()
        self.seq_len[slot] = 0
        for g in self._state_groups:
            g.state[:, slot].zero_()
        return slot

    def release(self, slot: int) -> None:
        """Give the slot and all its pages back."""
        if not self.slots.held(slot):
            raise CacheError(f"sequence slot {slot} is released but not held")
        for g in self._kv_groups:
            for p in g.live_pages(slot):
                g.pages.release(p)
            g.pages_of[slot] = []
            g.dropped[slot] = 0
        self.seq_len[slot] = 0
        self.slots.release(slot)

    def release_all(self) -> None:
        for slot in range(self.max_seqs):
            if self.slots.held(slot):
                self.release(slot)

    def reserve(self, growth: list) -> None:
        """Make room for every (slot, new_length) pair, or acquire nothing and raise."""
        plan = []
        for slot, new_len in growth:
            if not self.slots.held(slot):
                raise CacheError(f"sequence slot {slot} is not held")
            if new_len > self.max_seq_len:
                raise ContextLengthExceeded(new_len, self.max_seq_len)
            plan.append((slot, (new_len + PAGE - 1) // PAGE))
        # what lies before the window of every token still to come goes back first (the sequence's length is that of
        # the steps already run: this step's tokens start there)
        for g in self._kv_groups:
            for slot, _ in plan:
                g.drop_before_window(slot, self.seq_len[slot])
        for g in self._kv_groups:
            extra = sum(max(0, pages - len(g.pages_of[slot])) for slot, pages in plan)
            if extra > g.pages.free_count:
                held = self.n_pages - g.pages.free_count
                raise CacheFull(f"the step needs {extra} more cache pages of {PAGE} tokens; {g.pages.free_count} of "
                                f"{self.n_pages} are free ({held * PAGE} of {self.n_pages * PAGE} token places held)")
        for g in self._kv_groups:
            cells, values = [], []              # all the step's new entries of the block table go over in one piece
            for slot, pages in plan:
                have = len(g.pages_of[slot])
                if pages > have:
                    new = g.pages.acquire_many(pages - have)
                    g.pages_of[slot].extend(new)
                    first = slot * self.max_pages_per_seq + have
                    cells.extend(range(first, first + len(new)))
                    values.extend(new)
            if cells:
                dev = g.block_table.device
                g.block_table.view(-1).index_put_((torch.tensor(cells, dtype=torch.int64).to(dev),),
                                                  torch.tensor(values, dtype=torch.int32).to(dev))

    def set_length(self, slot: int, length: int) -> None:
        self.seq_len[slot] = length
