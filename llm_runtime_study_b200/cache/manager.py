"""The cache manager: pages of keys and values per group of layers, a block
table per request, and slots for per-request state of fixed size.

What the reference has (mini_llm/cache/paged/cache.py:257-352): one pool for all
layers, one block table per request filled for the request's whole lifetime at
admission, a host-side logical length committed before the forward pass and
rolled back on failure (mini_llm/cache/lengths.py:8-43, mini_llm/model/base.py:
169-175, 188-190).  What is added here: *groups* of layers with different needs
(all keys, or a window of them) that own pages of their own; pages taken when a
sequence grows into them and given back when it ends or its window has passed
them; and slots for fixed-size state.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Sequence

import torch

from ..errors import KVCacheError
from ..parts.base import FixedState, PagedKV
from .pages import PageAllocator
from .slots import SlotTable


@dataclass(frozen=True)
class PageGroup:
    """Layers (indices into the model's layer list) whose mixers need the same
    kind of paged memory; they share page ids: page ``p`` addresses the same
    positions in every layer of the group (mini_llm/cache/paged/store.py:13-14)."""

    requirement: PagedKV
    layers: tuple[int, ...]


@dataclass(frozen=True)
class StateArray:
    layer: int
    requirement: FixedState


@dataclass(frozen=True)
class CacheLayout:
    """What a model needs of the cache: derived from its mixers, not from its name."""

    groups: tuple[PageGroup, ...]
    states: tuple[StateArray, ...]

    @classmethod
    def from_requirements(cls, requirements: Sequence[PagedKV | FixedState | None]) -> "CacheLayout":
        """``requirements[i]`` is what layer ``i``'s mixer asks for (``None`` for
        a layer that owns no cache)."""

        by_need: dict[PagedKV, list[int]] = {}
        states = []
        for layer, need in enumerate(requirements):
            if isinstance(need, PagedKV):
                by_need.setdefault(need, []).append(layer)
            elif isinstance(need, FixedState):
                states.append(StateArray(layer, need))
            elif need is not None:
                raise KVCacheError(f"layer {layer} asks for an unknown kind of cache: {need!r}")
        groups = tuple(PageGroup(need, tuple(layers)) for need, layers in by_need.items())
        return cls(groups, tuple(states))


@dataclass(frozen=True)
class LayerCache:
    """What a mixer is handed for its layer."""

    group: int | None = None            # page group index
    keys: torch.Tensor | None = None    # [pages, kv_heads, page_size, head_dim]
    values: torch.Tensor | None = None
    page_size: int = 0
    state: torch.Tensor | None = None   # [slots, *shape] for fixed-size state


@dataclass
class RequestCache:
    """A request's hold on the cache: a slot, a logical length, and one block
    table (list of page ids, ``-1`` where a page has been given back) per group."""

    slot: int
    tables: list[list[int]]
    length: int = 0
    released: bool = False
    id: int = field(default=0)


@dataclass(frozen=True)
class CacheAllocation:
    capacity: int
    num_bytes: int


class CacheManager:
    """Owns the device pools, the page allocators, the request slots.

    ``max_tokens`` sizes every group's pool (``ceil(max_tokens / page_size)``
    pages, plus what rounding each of ``max_requests`` sequences up to whole
    pages may cost is the caller's business: give the rounded figure).
    """

    def __init__(
        self, layout: CacheLayout, *, max_tokens: int, page_size: int, max_requests: int,
        dtype: torch.dtype, device: torch.device | str, max_seq_len: int | None = None,
    ) -> None:
        if max_tokens <= 0 or page_size <= 0 or max_requests <= 0:
            raise KVCacheError("max_tokens, page_size and max_requests must be positive")
        self.layout = layout
        self.page_size = page_size
        self.max_requests = max_requests
        self.capacity = max_tokens
        self.max_seq_len = max_seq_len or max_tokens
        self.device = torch.device(device)
        self.dtype = dtype
        self.num_pages = -(-max_tokens // page_size)
        self.pools: list[torch.Tensor] = []
        self.allocators: list[PageAllocator] = []
        for group in layout.groups:
            need = group.requirement
            # [layer in group][K|V][page][kv head][slot in page][head_dim]; zero-filled so
            # that nothing a kernel may touch under a mask is ever a NaN pattern.
            self.pools.append(torch.zeros(
                (len(group.layers), 2, self.num_pages, need.num_kv_heads, page_size, need.head_dim),
                dtype=dtype, device=self.device,
            ))
            self.allocators.append(PageAllocator(self.num_pages))
        # Fixed-size state: one row per request slot and one more that belongs to nobody, for the rows that
        # pad a batch up to the size of its captured graph (what a mixer writes there is never read).
        self.padding_slot = max_requests
        self.state_arrays: dict[int, torch.Tensor] = {
            s.layer: torch.zeros((max_requests + 1, *s.requirement.shape), dtype=s.requirement.dtype, device=self.device)
            for s in layout.states
        }
        self.slots = SlotTable(max_requests, self.device)
        self._layer_group = {layer: (g, i) for g, group in enumerate(layout.groups) for i, layer in enumerate(group.layers)}
        self._free_slots = list(range(max_requests - 1, -1, -1))
        self._active: dict[int, RequestCache] = {}
        self._next_id = 0
        self.last_allocation: CacheAllocation | None = None

    # -------------------------------------------------------------- views
    def layer_cache(self, layer: int) -> LayerCache:
        """The cache view of a layer that owns one."""

        if layer in self._layer_group:
            g, i = self._layer_group[layer]
            pool = self.pools[g]
            return LayerCache(group=g, keys=pool[i, 0], values=pool[i, 1], page_size=self.page_size)
        if layer in self.state_arrays:
            return LayerCache(state=self.state_arrays[layer])
        return LayerCache()

    @property
    def num_bytes(self) -> int:
        return sum(p.numel() * p.element_size() for p in self.pools) + sum(
            s.numel() * s.element_size() for s in self.state_arrays.values()
        )

    def bytes_per_token(self) -> int:
        return sum(
            len(g.layers) * 2 * g.requirement.num_kv_heads * g.requirement.head_dim
            for g in self.layout.groups
        ) * torch.empty((), dtype=self.dtype).element_size()

    # ----------------------------------------------------------- counters
    @property
    def free_pages(self) -> int:
        return min((a.num_free for a in self.allocators), default=self.num_pages)

    @property
    def used_pages(self) -> int:
        return max((a.num_held for a in self.allocators), default=0)

    @property
    def used_tokens(self) -> int:
        return sum(r.length for r in self._active.values())

    @property
    def active_sequences(self) -> int:
        return len(self._active)

    @property
    def free_slots(self) -> int:
        return len(self._free_slots)

    # ---------------------------------------------------------- lifecycle
    def admit(self) -> RequestCache:
        """Take a slot (its fixed-size state zeroed) and an empty block table."""

        if not self._free_slots:
            raise KVCacheError(f"all {self.max_requests} request slots are taken")
        slot = self._free_slots.pop()
        for array in self.state_arrays.values():
            array[slot].zero_()
        request = RequestCache(slot=slot, tables=[[] for _ in self.layout.groups], id=self._next_id)
        self._next_id += 1
        self._active[request.id] = request
        return request

    def _check_live(self, request: RequestCache) -> None:
        if request.released or request.id not in self._active:
            raise KVCacheError("the request's cache has been released")

    def pages_needed(self, request: RequestCache, new_length: int) -> int:
        """Pages each group would have to take for the request to hold
        ``new_length`` tokens (the largest need over the groups)."""

        need_total = -(-new_length // self.page_size)
        return max((max(0, need_total - len(t)) for t in request.tables), default=0)

    def pages_held(self, request: RequestCache) -> int:
        """Pages' worth of positions the request's block tables cover (the same in every
        group: groups grow together; a page that a window has given back still counts)."""

        return min((len(t) for t in request.tables), default=0)

    def can_grow(self, request: RequestCache, new_length: int) -> bool:
        if new_length > self.max_seq_len:
            return False
        need_total = -(-new_length // self.page_size)
        return all(
            max(0, need_total - len(t)) <= a.num_free for t, a in zip(request.tables, self.allocators)
        )

    def can_admit(self, tokens: int) -> bool:
        """A free slot and pages for ``tokens`` tokens in every group."""

        need = -(-tokens // self.page_size)
        return bool(self._free_slots) and all(need <= a.num_free for a in self.allocators)

    def grow(self, request: RequestCache, new_length: int) -> None:
        """Take the pages needed to hold ``new_length`` tokens, in every group or
        in none.  The logical length is not changed (see ``commit``)."""

        self._check_live(request)
        if new_length > self.max_seq_len:
            raise KVCacheError(
                f"sequence of {new_length} tokens exceeds the cache's limit of {self.max_seq_len}"
            )
        if not self.can_grow(request, new_length):
            need = self.pages_needed(request, new_length)
            raise KVCacheError(
                f"KV page pool exhausted: need {need} pages but only {self.free_pages} are free"
            )
        need_total = -(-new_length // self.page_size)
        for table, allocator in zip(request.tables, self.allocators):
            table.extend(allocator.allocate(max(0, need_total - len(table))))
        held = max((len(t) for t in request.tables), default=0) * self.page_size
        self.last_allocation = CacheAllocation(held, held * self.bytes_per_token())

    def commit(self, request: RequestCache, new_length: int) -> None:
        """Set the logical length after a step (the reference commits before the
        forward pass and rolls back on failure; here the step commits on success,
        which is the same contract seen from outside).  Pages that a window has
        passed are given back."""

        self._check_live(request)
        capacity = min((len(t) for t in request.tables), default=new_length // self.page_size + 1) * self.page_size
        if request.tables and new_length > capacity:
            raise KVCacheError(f"length {new_length} exceeds the {capacity} tokens of pages held")
        request.length = new_length
        for g, group in enumerate(self.layout.groups):
            window = group.requirement.window
            if window is None:
                continue
            # the next query sits at position new_length and reads keys > new_length - window
            dead_tokens = new_length - window + 1
            table = request.tables[g]
            for index in range(min(len(table), max(0, dead_tokens // self.page_size))):
                if table[index] >= 0:
                    self.allocators[g].free([table[index]])
                    table[index] = -1

    def rollback(self, request: RequestCache, length: int) -> None:
        self._check_live(request)
        if length > request.length:
            raise KVCacheError("rollback cannot lengthen a sequence")
        request.length = length

    def release(self, request: RequestCache) -> None:
        """Give back pages and slot.  Idempotent (mini_llm/cache/paged/cache.py:346-352)."""

        if request.released:
            return
        request.released = True
        for table, allocator in zip(request.tables, self.allocators):
            allocator.free([p for p in table if p >= 0])
            table.clear()
        self._active.pop(request.id, None)
        self._free_slots.append(request.slot)
        self.slots.clear(request.slot)
        request.length = 0

    def check(self) -> None:
        """No page lost, held twice or freed twice; held pages are exactly those
        in live block tables."""

        for g, allocator in enumerate(self.allocators):
            allocator.check()
            in_tables = [p for r in self._active.values() for p in r.tables[g] if p >= 0]
            if len(in_tables) != len(set(in_tables)):
                raise KVCacheError(f"group {g}: a page is in two block tables")
            if set(in_tables) != allocator._held:
                raise KVCacheError(f"group {g}: held pages differ from the pages in block tables")
        slots = [r.slot for r in self._active.values()]
        if len(slots) != len(set(slots)) or set(slots) & set(self._free_slots):
            raise KVCacheError("a request slot is held twice")
        if len(slots) + len(self._free_slots) != self.max_requests:
            raise KVCacheError("a request slot was lost")
