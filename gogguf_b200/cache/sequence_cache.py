"""The cache: one slot per live sequence, paged keys and values per layer group, fixed-size state.

What each scheduled layer needs is asked of its mixer as a *request*:

* `KVRequest(num_kv_heads, head_dim, window)` - keys and values of every position (window None)
  or of the last `window` positions.  Layers with equal requests form a *group* with storage of
  its own: pools ``k, v [layer_in_group][page][kv_head][page_size][head_dim]`` and, per slot, the
  list of pages that hold its positions.  A windowed group gives pages back as soon as every
  position in them has left the window.
* `StateRequest(shape, dtype)` - a fixed-size state per sequence, ``[max_slots, *shape]`` for that
  layer, zeroed when a slot is opened.
* None - the layer keeps nothing.

A sequence's length lives here once, for all groups; a step first *plans* (checks capacity and
reserves pages for the tokens it brings, all or nothing), the kernels write keys and values at
positions length..length+n-1, and `commit` advances the length after the last layer - the same
two-phase rule as the reference's cache, whose Append does not move Len() until Advance()
(pkg/model/qwen3/cache.go:37-45).  The reference holds one sequence in growing float32 slices
(cache.go:4-29) and its GPU mirror as [max_seq, kv_dim] per layer (pkg/gpu/cuda/driver.c:534-565);
slots, pages and groups are this library's own.

Capacity is counted in tokens: `max_tokens` is the most that live sequences may hold, each
sequence's count rounded up to a whole page.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple, Union

import torch

from .allocators import CacheError, CacheFull, FreeList

PAGE_SIZE = 64


@dataclass(frozen=True)
class KVRequest:
    num_kv_heads: int
    head_dim: int
    window: Optional[int] = None


@dataclass(frozen=True)
class StateRequest:
    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32


Request = Union[KVRequest, StateRequest, None]


class KVGroup:
    """Storage and page bookkeeping of the layers that share one `KVRequest`."""

    def __init__(self, request: KVRequest, entries: List[int], n_pages: int, page_size: int,
                 dtype: torch.dtype, device):
        self.request = request
        self.entries = list(entries)          # schedule entries that own a layer of this group
        self.page_size = page_size
        self.n_pages = n_pages
        shape = (len(entries), n_pages, request.num_kv_heads, page_size, request.head_dim)
        # zero-filled once: a page that is handed out again holds old finite numbers, never NaN patterns
        self.k = torch.zeros(shape, dtype=dtype, device=device)
        self.v = torch.zeros(shape, dtype=dtype, device=device)
        self.pages = FreeList(n_pages, "page")
        self.seq_pages: Dict[int, List[int]] = {}   # slot -> page id per page index (-1 once given back)

    def pages_needed(self, slot: int, new_len: int) -> int:
        have = len(self.seq_pages.get(slot, ()))
        want = (new_len + self.page_size - 1) // self.page_size
        return max(0, want - have)

    def reserve(self, slot: int, new_len: int) -> None:
        n = self.pages_needed(slot, new_len)
        if n:
            self.seq_pages.setdefault(slot, []).extend(self.pages.take_many(n))

    def trim(self, slot: int, length: int) -> None:
        """Windowed group: give back pages all of whose positions are below length - window + 1."""
        w = self.request.window
        if w is None:
            return
        first_needed = length - w + 1
        pl = self.seq_pages.get(slot, [])
        for idx, pg in enumerate(pl):
            if (idx + 1) * self.page_size > first_needed:
                break
            if pg >= 0:
                self.pages.give(pg)
                pl[idx] = -1

    def can_shorten(self, slot: int, length: int) -> bool:
        """Are the positions that a token at position `length` reads still held?"""
        w = self.request.window
        if w is None:
            return True
        pl = self.seq_pages.get(slot, [])
        first_needed = max(0, length - w + 1)
        last = (length + self.page_size - 1) // self.page_size
        return all(pg >= 0 for pg in pl[first_needed // self.page_size:last])

    def shorten(self, slot: int, length: int) -> None:
        """Give back the pages beyond the first `length` positions."""
        pl = self.seq_pages.get(slot, [])
        keep = (length + self.page_size - 1) // self.page_size
        for pg in pl[keep:]:
            if pg >= 0:
                self.pages.give(pg)
        del pl[keep:]

    def release(self, slot: int) -> None:
        for pg in self.seq_pages.pop(slot, []):
            if pg >= 0:
                self.pages.give(pg)

    def table_row(self, slot: int, width: int) -> List[int]:
        pl = self.seq_pages.get(slot, [])
        if len(pl) > width:
            raise CacheError(f"page table width {width} is too small for {len(pl)} pages")
        # a page that was given back is never read (it lies before the window); 0 keeps the entry valid
        return [p if p >= 0 else 0 for p in pl] + [0] * (width - len(pl))


@dataclass
class KVView:
    """What a mixer gets for one scheduled layer: its slices of the group's pools."""
    group: int
    k: torch.Tensor            # [page][kv_head][page_size][head_dim]
    v: torch.Tensor
    page_size: int
    request: KVRequest


@dataclass
class StateView:
    state: torch.Tensor        # [max_slots, *shape]
    request: StateRequest


class SequenceCache:
    def __init__(self, requests: Sequence[Request], cache_of: Sequence[Optional[int]], max_tokens: int,
                 dtype: torch.dtype, device="cpu", page_size: int = PAGE_SIZE, max_slots: Optional[int] = None):
        """`requests[i]` is what schedule entry i asks for; `cache_of[i]` is None or the earlier entry
        whose cache entry i reads (then entry i gets that entry's view and no storage of its own)."""
        if max_tokens <= 0:
            raise ValueError("max_tokens must be positive")
        self.page_size = page_size
        self.n_pages = (max_tokens + page_size - 1) // page_size
        self.max_tokens = self.n_pages * page_size
        self.max_slots = max_slots if max_slots is not None else self.n_pages
        self.dtype = dtype
        self.device = torch.device(device)
        self.slots = FreeList(self.max_slots, "slot")
        self.lengths: List[int] = [0] * self.max_slots

        self.groups: List[KVGroup] = []
        self._views: Dict[int, Union[KVView, StateView, None]] = {}
        by_request: Dict[KVRequest, List[int]] = {}
        for i, (rq, src) in enumerate(zip(requests, cache_of)):
            if src is None and isinstance(rq, KVRequest):
                by_request.setdefault(rq, []).append(i)
        for rq, entries in by_request.items():
            g = KVGroup(rq, entries, self.n_pages, page_size, dtype, self.device)
            gi = len(self.groups)
            self.groups.append(g)
            for li, e in enumerate(entries):
                self._views[e] = KVView(group=gi, k=g.k[li], v=g.v[li], page_size=page_size, request=rq)
        self.states: Dict[int, torch.Tensor] = {}
        for i, (rq, src) in enumerate(zip(requests, cache_of)):
            if src is None and isinstance(rq, StateRequest):
                st = torch.zeros((self.max_slots,) + tuple(rq.shape), dtype=rq.dtype, device=self.device)
                self.states[i] = st
                self._views[i] = StateView(state=st, request=rq)
            elif src is None and rq is None:
                self._views[i] = None
        for i, src in enumerate(cache_of):
            if src is not None:
                if self._views.get(src) is None:
                    raise CacheError(f"schedule entry {i} reads the cache of entry {src}, which has none")
                self._views[i] = self._views[src]

    # ------------------------------------------------------------------ slots
    def open(self) -> int:
        """A slot for a new sequence: length 0, state zeroed, no pages yet."""
        s = self.slots.take()
        self.lengths[s] = 0
        for st in self.states.values():
            st[s].zero_()
        return s

    def close(self, slot: int) -> None:
        """Give back a sequence's slot and pages.  Nothing is cleared: reads are bounded by lengths."""
        if not self.slots.is_held(slot):
            raise CacheError(f"slot {slot} is not open")
        for g in self.groups:
            g.release(slot)
        self.lengths[slot] = 0
        self.slots.give(slot)

    def length(self, slot: int) -> int:
        if not self.slots.is_held(slot):
            raise CacheError(f"slot {slot} is not open")
        return self.lengths[slot]

    def truncate(self, slot: int, length: int) -> bool:
        """Shorten an open sequence to its first `length` tokens (a conversation that is rolled back,
        a sequence that ran one step further than its result).  Returns False and changes nothing
        where that cannot be done: a windowed group has already given back a page that the shorter
        sequence's next token reads, or a layer keeps a fixed-size state, in which all tokens are
        folded together.  The caller then starts the sequence again."""
        cur = self.length(slot)
        if length < 0 or length > cur:
            raise CacheError(f"slot {slot} holds {cur} tokens, cannot be cut to {length}")
        if length == cur:
            return True
        if self.states or not all(g.can_shorten(slot, length) for g in self.groups):
            return False
        for g in self.groups:
            g.shorten(slot, length)
        self.lengths[slot] = length
        return True

    def restart(self, slot: int) -> None:
        """An open slot as `open` hands it out: length 0, no pages, state zeroed."""
        if not self.slots.is_held(slot):
            raise CacheError(f"slot {slot} is not open")
        for g in self.groups:
            g.release(slot)
        self.lengths[slot] = 0
        for st in self.states.values():
            st[slot].zero_()

    @property
    def live_slots(self) -> int:
        return self.slots.held_count

    def free_tokens(self) -> int:
        return min((g.pages.free_count for g in self.groups), default=self.n_pages) * self.page_size

    # ------------------------------------------------------------------ steps
    def plan(self, slots: Sequence[int], counts: Sequence[int]) -> None:
        """Reserve pages for `counts[i]` new tokens of `slots[i]`; all or nothing."""
        if len(set(slots)) != len(slots):
            raise CacheError("a slot appears twice in one step")
        for s, n in zip(slots, counts):
            if not self.slots.is_held(s):
                raise CacheError(f"slot {s} is not open")
            if n <= 0:
                raise CacheError(f"slot {s}: a step must bring at least one token")
        for g in self.groups:
            need = sum(g.pages_needed(s, self.lengths[s] + n) for s, n in zip(slots, counts))
            if need > g.pages.free_count:
                raise CacheFull(
                    f"the step needs {need} more pages of {self.page_size} tokens but only "
                    f"{g.pages.free_count} of {g.n_pages} are free (cache sized for {self.max_tokens} tokens)")
        for g in self.groups:
            for s, n in zip(slots, counts):
                g.reserve(s, self.lengths[s] + n)

    def commit(self, slots: Sequence[int], counts: Sequence[int]) -> None:
        """Advance the lengths after the last layer of a step; windowed groups drop old pages."""
        for s, n in zip(slots, counts):
            self.lengths[s] += n
            for g in self.groups:
                g.trim(s, self.lengths[s])

    def table_width(self, slots: Sequence[int]) -> int:
        w = 1
        for g in self.groups:
            for s in slots:
                w = max(w, len(g.seq_pages.get(s, ())))
        return w

    def page_table(self, group: int, slots: Sequence[int], width: int) -> List[List[int]]:
        g = self.groups[group]
        return [g.table_row(s, width) for s in slots]

    def view(self, entry: int):
        return self._views[entry]

    def check(self) -> None:
        """Bookkeeping invariants (used by tests): nothing lost, nothing held twice."""
        self.slots.check()
        for g in self.groups:
            g.pages.check()
            held = [p for pl in g.seq_pages.values() for p in pl if p >= 0]
            if len(held) != len(set(held)):
                raise CacheError("a page is held by two sequences")
            if len(held) != g.pages.held_count:
                raise CacheError(f"{g.pages.held_count} pages are held but sequences list {len(held)}")
            for s in g.seq_pages:
                if not self.slots.is_held(s):
                    raise CacheError(f"pages are listed for slot {s}, which is not open")
