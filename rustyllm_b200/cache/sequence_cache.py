"""The cache of the engine: a slot for each live sequence; keys and values for each
layer in pages; storage groups for layers with different needs; and, beside it, a
state area of fixed size per sequence.

Reference counterpart: ``KVCache`` (src/model.rs:1328-1503) - per layer
``k[pos * k_dim ..]`` and ``v[..]``, an optional ring for a sliding window
(``slot = pos % window``, src/model.rs:1457-1464) and an optional fixed-size
recurrent state (``SsmState``, src/model.rs:1286-1315) - which belongs to one
sequence.  Here one pool serves every sequence of every batch:

  * a *slot* holds one sequence: its length, one row of each group's page table,
    and ``state_bytes`` of state that is zeroed when the slot is handed out;
  * a *group* is the storage of all layers with the same need (number of KV
    heads, width of a key head and of a value head, all keys or a window of them).
    It owns the keys ``[layers, pages, kv_heads, page_size, head_dim]``, the values
    ``[layers, pages, kv_heads, page_size, value_dim]`` and a page allocator;
    page p of a slot holds positions ``[p*page_size, (p+1)*page_size)`` of every
    layer of the group.  A window group gives pages back once every position in
    them has left the window;
  * slots and pages that are given back are used again without being cleared:
    nothing reads positions at or beyond a sequence's length (the reference
    relies on the same, src/session.rs:65-69).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..kernels import PAGE_SIZE
from ..staging import PinnedStaging
from .allocators import CacheFull, CacheMisuse, FreeList


@dataclass(frozen=True)
class KVNeed:
    """What one attention-like layer needs cached per position."""
    num_kv_heads: int
    head_dim: int                  # width of a key head
    window: Optional[int] = None   # None: all keys; W: only the last W positions are read
    value_dim: Optional[int] = None  # width of a value head; None: the same as head_dim

    def __post_init__(self):
        if self.value_dim == self.head_dim:        # one way to say "the same": equal needs share a group
            object.__setattr__(self, "value_dim", None)

    @property
    def v_dim(self) -> int:
        return self.head_dim if self.value_dim is None else self.value_dim


@dataclass(frozen=True)
class StateNeed:
    """Fixed-size per-sequence state of one layer, in bytes."""
    nbytes: int


class KVGroup:
    def __init__(self, need: KVNeed, layers: int, num_pages: int, max_slots: int,
                 max_pages_per_slot: int, dtype: torch.dtype, device: torch.device):
        self.need = need
        self.layers = layers
        self.num_pages = num_pages
        self.pages = FreeList(num_pages, "page")
        # zero-filled once: rows of a page beyond a sequence's length are never selected, but a
        # tensor-core attention kernel multiplies them by a probability of exactly 0, so they
        # must be finite (what earlier sequences left there is)
        self.keys = torch.zeros((layers, num_pages, need.num_kv_heads, PAGE_SIZE, need.head_dim),
                                dtype=dtype, device=device)
        self.values = torch.zeros((layers, num_pages, need.num_kv_heads, PAGE_SIZE, need.v_dim),
                                  dtype=dtype, device=device)
        self.page_table_host = torch.zeros((max_slots, max_pages_per_slot), dtype=torch.int32)
        self.page_table = self.page_table_host if device.type == "cpu" else \
            torch.zeros((max_slots, max_pages_per_slot), dtype=torch.int32, device=device)
        # per slot: page id of each logical page, or -1 once it was released (window groups)
        self.slot_pages: List[List[int]] = [[] for _ in range(max_slots)]

    def k_pool(self, layer: int) -> torch.Tensor:
        return self.keys[layer]

    def v_pool(self, layer: int) -> torch.Tensor:
        return self.values[layer]

    def bytes_per_token(self) -> int:
        return self.layers * self.need.num_kv_heads * (self.need.head_dim + self.need.v_dim) * self.keys.element_size()

    def memory_bytes(self) -> int:
        return (self.keys.numel() + self.values.numel()) * self.keys.element_size()

    def pages_needed(self, slot: int, new_len: int) -> int:
        have = len(self.slot_pages[slot])
        return max(0, -(-new_len // PAGE_SIZE) - have)


class SequenceCache:
    """All cache storage of one engine.

    ``kv_needs[i]`` / ``state_needs[i]`` describe cache entry i (one per layer run
    that owns a cache; a layer that reads another's cache has none).  ``max_tokens``
    is the most tokens live sequences hold at any time, each sequence's count
    rounded up to a whole page.
    """

    def __init__(self, kv_needs: Sequence[Optional[KVNeed]], state_needs: Sequence[Optional[StateNeed]],
                 max_tokens: int, dtype: torch.dtype, device, max_slots: Optional[int] = None,
                 max_seq_len: Optional[int] = None):
        device = torch.device(device)
        self.device = device
        self._staging: Optional[PinnedStaging] = None      # for page-table updates
        self.dtype = dtype
        self.page_size = PAGE_SIZE
        if max_tokens <= 0:
            raise ValueError("max_tokens must be > 0")
        num_pages = -(-max_tokens // PAGE_SIZE)
        self.num_pages = num_pages
        self.max_slots = max_slots if max_slots is not None else min(num_pages, 1024)
        if self.max_slots <= 0:
            raise ValueError("max_slots must be > 0")
        per_slot = num_pages if max_seq_len is None else min(num_pages, -(-max_seq_len // PAGE_SIZE))
        self.max_pages_per_slot = max(1, per_slot)
        self.max_seq_len = self.max_pages_per_slot * PAGE_SIZE if max_seq_len is None \
            else min(max_seq_len, self.max_pages_per_slot * PAGE_SIZE)

        # group the entries by need
        self.groups: List[KVGroup] = []
        self.entry_group: List[Optional[Tuple[int, int]]] = []   # entry -> (group, layer in group)
        by_need: Dict[KVNeed, List[int]] = {}
        for i, need in enumerate(kv_needs):
            if need is not None:
                by_need.setdefault(need, []).append(i)
        placement: Dict[int, Tuple[int, int]] = {}
        for gi, (need, entries) in enumerate(by_need.items()):
            pages = num_pages
            if need.window is not None:
                # a sequence holds at most the window plus one page in flight plus the step's tokens;
                # sized like the full group so that a long prompt step still fits
                pages = num_pages
            self.groups.append(KVGroup(need, len(entries), pages, self.max_slots,
                                       self.max_pages_per_slot, dtype, device))
            for li, e in enumerate(entries):
                placement[e] = (gi, li)
        for i in range(len(kv_needs)):
            self.entry_group.append(placement.get(i))

        # fixed-size state, one area per slot, entries laid out one after another (256-byte aligned)
        self.state_offsets: List[Optional[Tuple[int, int]]] = []
        off = 0
        for need in state_needs:
            if need is None or need.nbytes == 0:
                self.state_offsets.append(None)
            else:
                self.state_offsets.append((off, need.nbytes))
                off += -(-need.nbytes // 256) * 256
        self.state_bytes = off
        self.state = torch.zeros((self.max_slots, max(off, 1)), dtype=torch.uint8, device=device)

        self.slots = FreeList(self.max_slots, "slot")
        self.lengths: List[int] = [0] * self.max_slots

    # ------------------------------------------------------------------ slots
    def alloc_slot(self) -> int:
        (slot,) = self.slots.take(1)
        self.lengths[slot] = 0
        if self.state_bytes:
            self.state[slot].zero_()
        return slot

    def free_slot(self, slot: int) -> None:
        if not self.slots.is_held(slot):
            raise CacheMisuse(f"slot {slot} is freed but is not held")
        for g in self.groups:
            g.pages.give_back(p for p in g.slot_pages[slot] if p >= 0)
            g.slot_pages[slot] = []
        self.lengths[slot] = 0
        self.slots.give_back([slot])

    def length(self, slot: int) -> int:
        if not self.slots.is_held(slot):
            raise CacheMisuse(f"slot {slot} is not held")
        return self.lengths[slot]

    @property
    def free_pages(self) -> int:
        return min((g.pages.free_count for g in self.groups), default=self.num_pages)

    # ------------------------------------------------------------------ per step
    def prepare(self, slots: Sequence[int], counts: Sequence[int]) -> None:
        """Make room for ``counts[i]`` more tokens in ``slots[i]``: all or nothing."""
        if len(set(slots)) != len(slots):
            raise CacheMisuse(f"a slot appears twice in one step: {list(slots)}")
        for s, n in zip(slots, counts):
            if not self.slots.is_held(s):
                raise CacheMisuse(f"slot {s} is used in a step but is not held")
            if n <= 0:
                raise ValueError(f"slot {s}: a step must bring at least one token")
            if self.lengths[s] + n > self.max_seq_len:
                raise CacheFull(f"slot {s}: {self.lengths[s]} + {n} tokens exceed the longest "
                                f"sequence the cache holds ({self.max_seq_len})")
        for g in self.groups:
            want = sum(g.pages_needed(s, self.lengths[s] + n) for s, n in zip(slots, counts))
            if want > g.pages.free_count:
                raise CacheFull(f"{want} more pages of {PAGE_SIZE} tokens needed, "
                                f"{g.pages.free_count} of {g.num_pages} free")
        for g in self.groups:
            updates = []   # (slot, logical page, pool page)
            for s, n in zip(slots, counts):
                k = g.pages_needed(s, self.lengths[s] + n)
                if k == 0:
                    continue
                lo = len(g.slot_pages[s])
                new = g.pages.take(k)
                g.slot_pages[s].extend(new)
                updates.extend((s, lo + j, p) for j, p in enumerate(new))
            if updates:
                self._write_page_table(g, updates)

    def _write_page_table(self, g: KVGroup, updates) -> None:
        """Record new pages in the host copy and in the device copy of the page table.
        The device copy is written from a pinned buffer of a ring (a buffer is reused only
        after the copy that read it has finished), so later changes on the host cannot
        reach a step that is already queued."""
        u = np.asarray(updates, dtype=np.int64)
        flat = u[:, 0] * self.max_pages_per_slot + u[:, 1]
        g.page_table_host.view(-1).numpy()[flat] = u[:, 2]
        if g.page_table is not g.page_table_host:
            if self._staging is None:
                self._staging = PinnedStaging(self.device, torch.int32)
            n = flat.shape[0]
            dev = self._staging.upload(np.concatenate([flat, u[:, 2]]))      # places, then pages, in one copy
            g.page_table.view(-1).index_copy_(0, dev[:n].long(), dev[n:])

    def commit(self, slots: Sequence[int], counts: Sequence[int]) -> None:
        """The step ran: lengths grow; window groups release pages that fell out."""
        for s, n in zip(slots, counts):
            self.lengths[s] += n
        for g in self.groups:
            w = g.need.window
            if w is None:
                continue
            for s in slots:
                # the next query sits at position len; it reads positions >= len + 1 - w
                first_needed = max(0, self.lengths[s] + 1 - w)
                dead = first_needed // PAGE_SIZE   # logical pages wholly in front of it
                sp = g.slot_pages[s]
                gone = [sp[i] for i in range(min(dead, len(sp))) if sp[i] >= 0]
                if gone:
                    g.pages.give_back(gone)
                    for i in range(min(dead, len(sp))):
                        sp[i] = -1

    # ------------------------------------------------------------------ views for parts
    def kv_entry(self, entry: int) -> Tuple[KVGroup, int]:
        where = self.entry_group[entry]
        if where is None:
            raise CacheMisuse(f"cache entry {entry} has no key/value storage")
        return self.groups[where[0]], where[1]

    def state_entry(self, entry: int) -> Optional[torch.Tensor]:
        """``[max_slots, nbytes]`` view (uint8) of one entry's state, or None."""
        where = self.state_offsets[entry]
        if where is None:
            return None
        off, n = where
        return self.state[:, off:off + n]

    def check(self) -> None:
        """Invariants of the bookkeeping (tests call this after every operation)."""
        self.slots.check()
        for g in self.groups:
            g.pages.check()
            seen = set()
            for s in range(self.max_slots):
                held = [p for p in g.slot_pages[s] if p >= 0]
                if held and not self.slots.is_held(s):
                    raise CacheMisuse(f"free slot {s} still owns pages")
                for p in held:
                    if p in seen:
                        raise CacheMisuse(f"page {p} belongs to two sequences")
                    if not g.pages.is_held(p):
                        raise CacheMisuse(f"page {p} is used by slot {s} but marked free")
                    seen.add(p)
            if len(seen) != g.pages.held_count:
                raise CacheMisuse(f"{g.pages.held_count - len(seen)} held page(s) belong to no sequence")

    def memory_bytes(self) -> int:
        return sum(g.memory_bytes() for g in self.groups) + self.state.numel()
