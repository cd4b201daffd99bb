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

The kinds of request are an open set.  Each request class is registered with the *store* class that
holds what it asks for (`register_cache_store`); `SequenceCache` looks the store up by the request's
type, lets requests with equal `group_key` share one store, and talks to every store through the
`CacheStore` interface only.  A per-token cache that is not a K/V pair of equal head size subclasses
`PagedStore` (page bookkeeping, page tables) and allocates its own tensors; a per-sequence state of
another shape subclasses `CacheStore` directly.
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


Request = Optional[object]       # an instance of any registered request class, or None

STORES: Dict[type, type] = {}     # request class -> store class


def register_cache_store(request_cls: type):
    """Class decorator: instances of `request_cls` are held by the decorated `CacheStore` class."""
    def deco(store_cls: type) -> type:
        if request_cls in STORES and STORES[request_cls] is not store_cls:
            raise ValueError(f"cache requests of type {request_cls.__name__} already have a store")
        STORES[request_cls] = store_cls
        return store_cls
    return deco


class CacheStore:
    """What the cache asks of the storage behind one kind of request.

    Built as ``Store(request, entries, n_pages=..., page_size=..., max_slots=..., dtype=..., device=...)``
    for the schedule entries `entries` that share it.  The defaults describe storage that does not
    grow with the sequence; a paged store overrides the page methods (see `PagedStore`).
    """

    paged = False                 # True: has `pages`, `seq_pages`, `table_row`; gets a page table every step

    @staticmethod
    def group_key(request) -> Optional[object]:
        """Requests with equal keys share one store; None: every entry gets a store of its own."""
        return None

    def view(self, entry: int):
        """What the mixer of schedule entry `entry` is handed each step."""
        raise NotImplementedError

    def open(self, slot: int) -> None:            # a slot starts a new sequence
        pass

    def release(self, slot: int) -> None:         # the sequence is over (or starts again)
        pass

    def pages_needed(self, slot: int, new_len: int) -> int:
        return 0

    def reserve(self, slot: int, new_len: int) -> None:
        pass

    def trim(self, slot: int, length: int) -> None:   # after a step's commit
        pass

    def can_shorten(self, slot: int, length: int) -> bool:
        """Can the sequence be cut back to its first `length` tokens without running them again?"""
        return True

    def shorten(self, slot: int, length: int) -> None:
        pass

    def check(self, is_open) -> None:             # bookkeeping invariants, for tests
        pass


class PagedStore(CacheStore):
    """Page bookkeeping for per-token storage: a free list of pages and, per slot, the pages that hold
    its positions.  A subclass allocates its tensors (indexed ``[layer_in_store][page]...``) and
    implements `view`; an optional `window` gives pages back once every position in them has left it."""

    paged = True

    def __init__(self, request, entries: List[int], n_pages: int, page_size: int, window: Optional[int] = None):
        self.request = request
        self.entries = list(entries)          # schedule entries that own a layer of this store
        self.page_size = page_size
        self.n_pages = n_pages
        self.window = window
        self.pages = FreeList(n_pages, "page")
        self.seq_pages: Dict[int, List[int]] = {}   # slot -> page id per page index (-1 once given back)
        self.index = -1                        # position among the cache's paged stores (set by the cache):
        #                                        a step's page table of this store is ctx.page_tables[index]

    def check(self, is_open) -> None:
        self.pages.check()
        held = [p for pl in self.seq_pages.values() for p in pl if p >= 0]
        if len(held) != len(set(held)):
            raise CacheError("a page is held by two sequences")
        if len(held) != self.pages.held_count:
            raise CacheError(f"{self.pages.held_count} pages are held but sequences list {len(held)}")
        for s in self.seq_pages:
            if not is_open(s):
                raise CacheError(f"pages are listed for slot {s}, which is not open")

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
        w = self.window
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
        w = self.window
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



@register_cache_store(KVRequest)
class KVGroup(PagedStore):
    """Storage of the layers that share one `KVRequest`: pools ``k, v [layer][page][kv_head][page_size][head_dim]``."""

    @staticmethod
    def group_key(request: KVRequest):
        return request

    def __init__(self, request: KVRequest, entries: List[int], n_pages: int, page_size: int,
                 dtype: torch.dtype, device, max_slots: int = 0):
        super().__init__(request, entries, n_pages, page_size, window=request.window)
        shape = (len(entries), n_pages, request.num_kv_heads, page_size, request.head_dim)
        # zero-filled once: a page that is handed out again holds old finite numbers, never NaN patterns
        self.k = torch.zeros(shape, dtype=dtype, device=device)
        self.v = torch.zeros(shape, dtype=dtype, device=device)

    def view(self, entry: int) -> "KVView":
        li = self.entries.index(entry)
        return KVView(group=self.index, k=self.k[li], v=self.v[li], page_size=self.page_size, request=self.request)


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


@register_cache_store(StateRequest)
class StateStore(CacheStore):
    """A fixed-size state per sequence for one layer: ``[max_slots, *shape]``, zeroed when a slot is
    opened.  All tokens are folded into it, so a sequence cannot be cut back without running it again."""

    def __init__(self, request: StateRequest, entries: List[int], n_pages: int, page_size: int,
                 dtype: torch.dtype, device, max_slots: int = 0):
        self.request = request
        self.entries = list(entries)
        self.state = torch.zeros((max_slots,) + tuple(request.shape), dtype=request.dtype, device=device)
        self._view = StateView(state=self.state, request=request)

    def view(self, entry: int) -> StateView:
        return self._view

    def open(self, slot: int) -> None:
        self.state[slot].zero_()

    def can_shorten(self, slot: int, length: int) -> bool:
        return False


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

        self.stores: List[CacheStore] = []        # every store, paged or not
        self.groups: List[PagedStore] = []        # the paged ones, in the order of their page tables
        self._views: Dict[int, object] = {}
        shared: Dict[Tuple[type, object], List[int]] = {}
        own: List[Tuple[type, object, List[int]]] = []
        for i, (rq, src) in enumerate(zip(requests, cache_of)):
            if src is not None:
                continue
            if rq is None:
                self._views[i] = None
                continue
            store_cls = STORES.get(type(rq))
            if store_cls is None:
                raise CacheError(f"schedule entry {i}: no store is registered for cache requests of type "
                                 f"{type(rq).__name__} (registered: {sorted(c.__name__ for c in STORES)})")
            key = store_cls.group_key(rq)
            if key is None:
                own.append((store_cls, rq, [i]))
            else:
                shared.setdefault((store_cls, key), []).append(i)
        built = [(cls, requests[entries[0]], entries) for (cls, _), entries in shared.items()] + own
        for store_cls, rq, entries in sorted(built, key=lambda b: b[2][0]):
            st = store_cls(rq, entries, n_pages=self.n_pages, page_size=page_size, dtype=dtype,
                           device=self.device, max_slots=self.max_slots)
            self.stores.append(st)
            if st.paged:
                st.index = len(self.groups)
                self.groups.append(st)
            for e in entries:
                self._views[e] = st.view(e)
        # fixed-size states by schedule entry (kept for callers that look at them directly)
        self.states: Dict[int, torch.Tensor] = {e: st.state for st in self.stores if isinstance(st, StateStore)
                                                for e in st.entries}
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
        for st in self.stores:
            st.open(s)
        return s

    def close(self, slot: int) -> None:
        """Give back a sequence's slot and pages.  Nothing is cleared: reads are bounded by lengths."""
        if not self.slots.is_held(slot):
            raise CacheError(f"slot {slot} is not open")
        for st in self.stores:
            st.release(slot)
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
        if not all(st.can_shorten(slot, length) for st in self.stores):
            return False
        for st in self.stores:
            st.shorten(slot, length)
        self.lengths[slot] = length
        return True

    def restart(self, slot: int) -> None:
        """An open slot as `open` hands it out: length 0, no pages, state zeroed."""
        if not self.slots.is_held(slot):
            raise CacheError(f"slot {slot} is not open")
        for st in self.stores:
            st.release(slot)
            st.open(slot)
        self.lengths[slot] = 0

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

    def pages_short(self, slots: Sequence[int], counts: Sequence[int]) -> int:
        """How many pages the fullest group lacks for `counts[i]` new tokens of `slots[i]` (<= 0: it fits)."""
        short = -self.n_pages
        for g in self.groups:
            need = sum(g.pages_needed(s, self.lengths[s] + n) for s, n in zip(slots, counts))
            short = max(short, need - g.pages.free_count)
        return short if self.groups else 0

    def unplan(self, slots: Sequence[int]) -> None:
        """Undo `plan` for a step that did not run to its commit: pages beyond what each sequence's
        committed length needs go back."""
        for g in self.groups:
            for s in slots:
                g.shorten(s, self.lengths[s])

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
        for st in self.stores:
            st.check(self.slots.is_held)
