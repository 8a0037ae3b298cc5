"""The cache of a model: keys and values in pages, per-sequence state, slots.

Each sequence of a batch holds a slot.  A slot owns, in every group of cache
entries, a list of pages (64 positions each) that grows with the sequence, and a
row of every state tensor.  Cache entries whose mixers ask for the same shape
(key/value heads, head size, window) form a group with storage and a page pool
of its own; a model whose layers differ (all keys here, a window there, state
elsewhere) gets several groups.  When a sequence ends its slot and pages go back
to the pools and are handed to the next sequence without being cleared;
a group whose mixers see a window of the last w positions gives a sequence's
pages back as soon as they lie wholly before every window still to come:
positions past a sequence's length are never read (the reference's argument for
not clearing its cache, runtime.go:1530-1531), and state rows are zeroed when a
slot is taken (runtime.go:1526-1539).

The reference keeps one cache per runner, position-major per layer
(model.go:1321-1357, 1385-1393); pages, slots and groups are this library's.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..parts.base import KVRequest, StateRequest
from .pool import CacheFull, IdPool

PAGE = 64
RELEASED = -1        # in a sequence's list of pages: this one lay before the window and went back to the pool


@dataclass
class KVView:
    """What a mixer gets for its run: this entry's pages of keys and values
    ([pages, kv_heads, PAGE, head_dim] each), the group whose page table
    (ctx.pages[group]) addresses them, and whether this run writes them."""
    group: int
    k: torch.Tensor
    v: torch.Tensor
    writes: bool = True


@dataclass
class StateView:
    """Per-sequence state of one entry: ``rows`` [max_slots, *shape] float32,
    indexed by ctx.seq_slot."""
    rows: torch.Tensor
    writes: bool = True


class _Group:
    def __init__(self, gid: int, req: KVRequest, n_pages: int):
        self.gid, self.req = gid, req
        self.entries: List[int] = []
        self.pool = IdPool(n_pages, f"page of cache group {gid}")
        self.storage: Optional[torch.Tensor] = None


class SequenceCache:
    """requests[i] is what cache entry i needs (KVRequest, StateRequest or None).

    max_tokens: positions all live sequences may hold together, each sequence
    rounded up to a whole page.  max_positions: the longest a sequence may get.
    """

    def __init__(self, requests: Sequence, max_tokens: int, max_positions: int,
                 dtype: torch.dtype, device, max_slots: Optional[int] = None, allocate: bool = True):
        self.dtype, self.device = dtype, device
        self.max_positions = int(max_positions)
        self.n_pages = max(1, -(-int(max_tokens) // PAGE))
        self.max_pages_per_seq = max(1, -(-self.max_positions // PAGE))
        self.max_slots = int(max_slots) if max_slots else min(self.n_pages, 1024)
        self.slots = IdPool(self.max_slots, "slot")
        self.groups: List[_Group] = []
        self._entry: Dict[int, Tuple[str, int, int]] = {}     # entry -> (kind, group/state index, index in it)
        self._states: List[torch.Tensor] = []
        by_shape: Dict[KVRequest, _Group] = {}
        for i, req in enumerate(requests):
            if req is None:
                continue
            if isinstance(req, KVRequest):
                g = by_shape.get(req)
                if g is None:
                    g = _Group(len(self.groups), req, self.n_pages)
                    by_shape[req] = g
                    self.groups.append(g)
                self._entry[i] = ("kv", g.gid, len(g.entries))
                g.entries.append(i)
            elif isinstance(req, StateRequest):
                rows = (torch.zeros((self.max_slots, *req.shape), dtype=torch.float32, device=device)
                        if allocate else None)
                self._entry[i] = ("state", len(self._states), 0)
                self._states.append(rows)
            else:
                raise TypeError(f"cache entry {i}: unknown request {req!r}")
        if allocate:
            for g in self.groups:
                r = g.req
                g.storage = torch.empty((len(g.entries), 2, self.n_pages, r.num_kv_heads, PAGE, r.head_dim),
                                        dtype=dtype, device=device)
        # per-slot bookkeeping
        self._length = [0] * self.max_slots
        self._pages: List[List[List[int]]] = [[[] for _ in self.groups] for _ in range(self.max_slots)]
        # per slot and group: pages before this index have been released (groups with a window only)
        self._first_page: List[List[int]] = [[0 for _ in self.groups] for _ in range(self.max_slots)]

    # -- sizes ------------------------------------------------------------
    def bytes(self) -> int:
        n = sum(g.storage.numel() * g.storage.element_size() for g in self.groups if g.storage is not None)
        return n + sum(s.numel() * 4 for s in self._states if s is not None)

    def bytes_per_position(self) -> int:
        """Key and value bytes one cached position occupies, all entries together."""
        es = torch.empty((), dtype=self.dtype).element_size()
        return sum(len(g.entries) * 2 * g.req.num_kv_heads * g.req.head_dim * es for g in self.groups)

    # -- views ------------------------------------------------------------
    def view(self, entry: int, writes: bool = True):
        if entry not in self._entry:
            return None
        kind, a, b = self._entry[entry]
        if kind == "kv":
            st = self.groups[a].storage
            return KVView(group=a, k=st[b, 0], v=st[b, 1], writes=writes)
        return StateView(rows=self._states[a], writes=writes)

    # -- sequences --------------------------------------------------------
    def open(self) -> int:
        """Take a slot for a new sequence of length 0; its state rows are zeroed."""
        slot = self.slots.take()
        self._length[slot] = 0
        for s in self._states:
            if s is not None:
                s[slot].zero_()
        return slot

    def state_snapshot(self, slots: Sequence[int]) -> List[torch.Tensor]:
        """Copies of these sequences' rows of every state tensor (the reference saves and restores
        such state around work that must leave no trace, qwen35.go:306-322)."""
        states = [s for s in self._states if s is not None]
        if not states:
            return []
        idx = torch.tensor([int(s) for s in slots], dtype=torch.int64).to(self.device)
        return [s.index_select(0, idx) for s in states]

    def state_restore(self, slots: Sequence[int], rows: Sequence[torch.Tensor]) -> None:
        """Put back what ``state_snapshot`` took for the same sequences."""
        states = [s for s in self._states if s is not None]
        if not states:
            return
        idx = torch.tensor([int(s) for s in slots], dtype=torch.int64).to(self.device)
        for s, r in zip(states, rows):
            s.index_copy_(0, idx, r)

    def length(self, slot: int) -> int:
        self._held(slot)
        return self._length[slot]

    def _held(self, slot: int) -> None:
        if not self.slots.is_held(slot):
            raise ValueError(f"slot {slot} is not in use")

    def pages_needed(self, slot: int, new_len: int) -> int:
        have = len(self._pages[slot][0]) if self.groups else 0
        return max(0, -(-new_len // PAGE) - have)

    def reserve(self, wants: Sequence[Tuple[int, int]]) -> None:
        """Make room for sequences to grow: wants = [(slot, new length)].  Either
        every sequence gets its pages or none does and CacheFull is raised."""
        need = 0
        for slot, new_len in wants:
            self._held(slot)
            if new_len > self.max_positions:
                raise CacheFull(f"sequence in slot {slot} would reach {new_len} positions, "
                                f"the cache holds {self.max_positions} per sequence")
            if new_len < self._length[slot]:
                raise ValueError(f"slot {slot}: cannot shrink from {self._length[slot]} to {new_len}")
            need += self.pages_needed(slot, new_len)
        for g in self.groups:
            if need > g.pool.free_count:
                raise CacheFull(f"{need} more pages of {PAGE} positions wanted, "
                                f"{g.pool.free_count} of {g.pool.n} free in cache group {g.gid}")
        for slot, new_len in wants:
            k = self.pages_needed(slot, new_len)
            for g in self.groups:
                self._pages[slot][g.gid].extend(g.pool.take_many(k))

    def commit(self, slot: int, new_len: int) -> None:
        """Record that positions up to new_len are now written.  In a group with a window w the next
        token (at position new_len) sees keys from new_len - w + 1 on and every later token later ones,
        so pages that end before that position are given back at once: a long sequence holds about
        w / 64 + 1 pages of such a group, not all of its positions."""
        self._held(slot)
        if -(-new_len // PAGE) > (len(self._pages[slot][0]) if self.groups else new_len):
            raise ValueError(f"slot {slot}: length {new_len} was not reserved")
        self._length[slot] = new_len
        for g in self.groups:
            w = g.req.window
            if w > 0:
                pg = self._pages[slot][g.gid]
                keep_from = min(max(0, new_len - w + 1) // PAGE, len(pg))
                for i in range(self._first_page[slot][g.gid], keep_from):
                    g.pool.give(pg[i])
                    pg[i] = RELEASED
                if keep_from > self._first_page[slot][g.gid]:
                    self._first_page[slot][g.gid] = keep_from

    def close(self, slot: int) -> None:
        """Give back a sequence's pages and slot."""
        self._held(slot)
        for g in self.groups:
            for p in self._pages[slot][g.gid]:
                if p != RELEASED:
                    g.pool.give(p)
            self._pages[slot][g.gid] = []
            self._first_page[slot][g.gid] = 0
        self._length[slot] = 0
        self.slots.give(slot)

    def page_rows(self, group: int, slots: Sequence[int], out: Optional[np.ndarray] = None) -> np.ndarray:
        """[len(slots), max_pages_per_seq] int32 page ids (the unused tail and pages released before a
        window are 0: no kernel reads them)."""
        if out is None:
            out = np.zeros((len(slots), self.max_pages_per_seq), dtype=np.int32)
        else:
            out[...] = 0
        for r, slot in enumerate(slots):
            pg = self._pages[slot][group]
            out[r, :len(pg)] = pg
            k = self._first_page[slot][group]
            if k:
                out[r, :k] = 0
        return out

    def live_slots(self) -> List[int]:
        return [i for i in range(self.max_slots) if self.slots.is_held(i)]

    def tokens_held(self) -> int:
        """Positions reserved by live sequences, each rounded up to whole pages."""
        if not self.groups:
            return sum(self._length[s] for s in self.live_slots())
        return sum(len(self._pages[s][0]) for s in self.live_slots()) * PAGE

    def check(self) -> None:
        """Invariants: no page lost, none owned twice, free slots own nothing."""
        self.slots.check()
        for g in self.groups:
            g.pool.check()
            owned: List[int] = []
            for s in range(self.max_slots):
                pg = self._pages[s][g.gid]
                if not self.slots.is_held(s):
                    assert not pg, f"free slot {s} still owns pages"
                k = self._first_page[s][g.gid]
                assert all(p == RELEASED for p in pg[:k]) and all(p != RELEASED for p in pg[k:]), \
                    f"slot {s}: released pages of group {g.gid} do not form the head of its list"
                owned.extend(pg[k:])
            assert len(owned) == len(set(owned)), f"a page of group {g.gid} is owned twice"
            assert len(owned) == g.pool.held_count, f"pages of group {g.gid} are lost"
