"""The cache manager: pages of keys and values per group of layers, a block
table per request, and slots for per-request state of fixed size.

What the reference has (mini_llm/cache/paged/cache.py:257-352): one pool for all
layers, one block table per request filled for the request's whole lifetime at
admission, a host-side logical length committed before the forward pass and
rolled back on failure (mini_llm/cache/lengths.py:8-43, mini_llm/model/base.py:
169-175, 188-190).  What is added here: *groups* of layers with different needs
(all keys, or a window of them; keys and values, or whatever tensors per token a
mixer declares; a page size of their own) that own pages of their own; pages taken
when a sequence grows into them and given back when it ends or its window has
passed them; and slots for fixed-size state.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Sequence

import torch

from ..errors import KVCacheError
from ..parts.base import FixedState, PagedTensors
from .pages import PageAllocator
from .slots import SlotTable


@dataclass(frozen=True)
class PageGroup:
    """Layers (indices into the model's layer list) whose mixers need the same
    kind of paged memory; they share page ids: page ``p`` addresses the same
    positions in every layer of the group (mini_llm/cache/paged/store.py:13-14)."""

    requirement: PagedTensors
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
    def from_requirements(cls, requirements: Sequence[PagedTensors | FixedState | None]) -> "CacheLayout":
        """``requirements[i]`` is what layer ``i``'s mixer asks for (``None`` for
        a layer that owns no cache)."""

        by_need: dict[PagedTensors, list[int]] = {}
        states = []
        for layer, need in enumerate(requirements):
            if isinstance(need, PagedTensors):
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
    tensors: dict = field(default_factory=dict)   # name -> this layer's pages of that tensor, [pages, ...]
    page_size: int = 0
    state: torch.Tensor | None = None   # [slots, *shape] for fixed-size state

    @property
    def keys(self) -> torch.Tensor | None:      # [pages, kv_heads, page_size, head_dim]
        return self.tensors.get("keys")

    @property
    def values(self) -> torch.Tensor | None:
        return self.tensors.get("values")


def pool_shape(per_token: tuple[int, ...], pages: int, page_size: int) -> tuple[int, ...]:
    """Pages of a tensor whose shape per token is ``per_token``: the page axis goes behind the first
    per-token axis (heads), so that one (page, head) tile is contiguous; a vector per token is simply
    ``[pages, page_size, width]``."""

    if len(per_token) >= 2:
        return (pages, per_token[0], page_size, *per_token[1:])
    return (pages, page_size, *per_token)


class GroupPool:
    """The pages of one group of layers: its own page size, page count, tensors and allocator."""

    def __init__(self, group: PageGroup, *, page_size: int, num_pages: int, dtype: torch.dtype, device: torch.device) -> None:
        self.group, self.page_size, self.num_pages = group, page_size, num_pages
        self.window = group.requirement.window
        # [layer in group][page]...; zero-filled so that nothing a kernel may touch under a mask is ever a NaN pattern
        self.tensors = {
            name: torch.zeros((len(group.layers), *pool_shape(tuple(shape), num_pages, page_size)), dtype=dtype, device=device)
            for name, shape in group.requirement.tensors
        }
        self.allocator = PageAllocator(num_pages)
        elements = sum(int(torch.tensor(shape).prod()) for _, shape in group.requirement.tensors)
        self.bytes_per_token = len(group.layers) * elements * torch.empty((), dtype=dtype).element_size()

    def pages_for(self, tokens: int) -> int:
        return -(-tokens // self.page_size)

    @property
    def num_bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self.tensors.values())


class PageBudget:
    """A planner's copy of the free pages of every group: what fits, and what is left after taking it."""

    def __init__(self, manager: "CacheManager") -> None:
        self._pools = manager.groups
        self.free = [pool.allocator.num_free for pool in manager.groups]

    def _need(self, held: Sequence[int], new_length: int) -> list[int]:
        return [max(0, pool.pages_for(new_length) - h) for pool, h in zip(self._pools, held)]

    def fits(self, held: Sequence[int], new_length: int) -> bool:
        """``held``: pages' worth of positions each group's block table of the request covers already."""

        return all(n <= f for n, f in zip(self._need(held, new_length), self.free))

    def take(self, held: Sequence[int], new_length: int) -> bool:
        need = self._need(held, new_length)
        if any(n > f for n, f in zip(need, self.free)):
            return False
        self.free = [f - n for f, n in zip(self.free, need)]
        return True

    def room(self, held: Sequence[int]) -> int:
        """The longest sequence the request could hold with what is free now (tokens)."""

        return min(((h + f) * pool.page_size for pool, h, f in zip(self._pools, held, self.free)), default=1 << 60)

    def short_by(self, held: Sequence[int], new_length: int) -> tuple[int, int]:
        """(pages needed, pages free) of the group that is shortest of pages, for messages."""

        pairs = list(zip(self._need(held, new_length), self.free))
        return max(pairs, key=lambda nf: nf[0] - nf[1], default=(0, 0))


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

    ``max_tokens`` sizes the pool of every group that keeps whole sequences
    (``ceil(max_tokens / page_size)`` pages; what rounding each of ``max_requests``
    sequences up to whole pages may cost is the caller's business: give the rounded
    figure).  A group with a window keeps, per request, the window and what one step may
    add (``max_step_tokens`` for all requests together), so its pool is sized for that.
    ``page_size`` is the default for groups that name none of their own.
    """

    def __init__(
        self, layout: CacheLayout, *, max_tokens: int, page_size: int, max_requests: int,
        dtype: torch.dtype, device: torch.device | str, max_seq_len: int | None = None,
        max_step_tokens: int | None = None,
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
        self.groups: list[GroupPool] = []
        for group in layout.groups:
            size = group.requirement.page_size or page_size
            pages = -(-max_tokens // size)
            window = group.requirement.window
            if window is not None and max_step_tokens is not None:
                # per request: the window, a page at either end, the page being filled; for all together: one step's tokens
                pages = min(pages, max_requests * (-(-window // size) + 3) + -(-max_step_tokens // size))
            self.groups.append(GroupPool(group, page_size=size, num_pages=pages, dtype=dtype, device=self.device))
        self.num_pages = min((pool.num_pages for pool in self.groups), default=-(-max_tokens // page_size))
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

    @property
    def allocators(self) -> list[PageAllocator]:
        return [pool.allocator for pool in self.groups]

    @property
    def pools(self) -> list[torch.Tensor]:
        """Every pool tensor (for accounting)."""

        return [t for pool in self.groups for t in pool.tensors.values()]

    # -------------------------------------------------------------- views
    def layer_cache(self, layer: int) -> LayerCache:
        """The cache view of a layer that owns one."""

        if layer in self._layer_group:
            g, i = self._layer_group[layer]
            pool = self.groups[g]
            return LayerCache(group=g, tensors={name: t[i] for name, t in pool.tensors.items()}, page_size=pool.page_size)
        if layer in self.state_arrays:
            return LayerCache(state=self.state_arrays[layer])
        return LayerCache()

    @property
    def num_bytes(self) -> int:
        return sum(pool.num_bytes for pool in self.groups) + sum(
            s.numel() * s.element_size() for s in self.state_arrays.values()
        )

    def bytes_per_token(self) -> int:
        return sum(pool.bytes_per_token for pool in self.groups)

    @property
    def max_request_tokens(self) -> int:
        """The longest sequence a single request could ever hold: the smallest pool among the groups that keep
        whole sequences (a group with a window never holds more than its window of any request)."""

        whole = [pool.num_pages * pool.page_size for pool in self.groups if pool.window is None]
        return min(whole, default=self.max_seq_len)

    # ----------------------------------------------------------- counters
    @property
    def free_pages(self) -> int:
        """Free pages of the group that has fewest."""

        return min((pool.allocator.num_free for pool in self.groups), default=self.num_pages)

    @property
    def all_free(self) -> bool:
        return all(pool.allocator.num_free == pool.num_pages for pool in self.groups)

    @property
    def used_pages(self) -> int:
        return max((pool.allocator.num_held for pool in self.groups), default=0)

    @property
    def used_tokens(self) -> int:
        return sum(r.length for r in self._active.values())

    @property
    def active_sequences(self) -> int:
        return len(self._active)

    @property
    def free_slots(self) -> int:
        return len(self._free_slots)

    def budget(self) -> PageBudget:
        return PageBudget(self)

    @staticmethod
    def held(request: RequestCache | None) -> list[int]:
        """Pages' worth of positions each group's block table of the request covers (a page that a window has
        given back still counts: its positions need no page again)."""

        return [len(t) for t in request.tables] if request is not None else []

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

    def _held(self, request: RequestCache | None) -> list[int]:
        return [len(t) for t in request.tables] if request is not None else [0] * len(self.groups)

    def pages_needed(self, request: RequestCache | None, new_length: int) -> int:
        """Pages the neediest group would have to take for the request to hold ``new_length`` tokens."""

        return max((max(0, pool.pages_for(new_length) - h) for pool, h in zip(self.groups, self._held(request))), default=0)

    def pages_held(self, request: RequestCache) -> int:
        """Pages' worth of positions the request's shortest block table covers."""

        return min((len(t) for t in request.tables), default=0)

    def can_grow(self, request: RequestCache, new_length: int) -> bool:
        if new_length > self.max_seq_len:
            return False
        return self.budget().fits(self._held(request), new_length)

    def can_admit(self, tokens: int) -> bool:
        """A free slot and pages for ``tokens`` tokens in every group."""

        return bool(self._free_slots) and self.budget().fits(self._held(None), tokens)

    def grow(self, request: RequestCache, new_length: int) -> None:
        """Take the pages needed to hold ``new_length`` tokens, in every group or
        in none.  The logical length is not changed (see ``commit``)."""

        self._check_live(request)
        if new_length > self.max_seq_len:
            raise KVCacheError(
                f"sequence of {new_length} tokens exceeds the cache's limit of {self.max_seq_len}"
            )
        budget = self.budget()
        if not budget.fits(self._held(request), new_length):
            need, free = budget.short_by(self._held(request), new_length)
            raise KVCacheError(f"KV page pool exhausted: need {need} pages but only {free} are free")
        for table, pool in zip(request.tables, self.groups):
            table.extend(pool.allocator.allocate(max(0, pool.pages_for(new_length) - len(table))))
        held = min((len(t) * pool.page_size for t, pool in zip(request.tables, self.groups)), default=0)
        self.last_allocation = CacheAllocation(held, held * self.bytes_per_token())

    def commit(self, request: RequestCache, new_length: int) -> None:
        """Set the logical length after a step (the reference commits before the
        forward pass and rolls back on failure; here the step commits on success,
        which is the same contract seen from outside).  Pages that a window has
        passed are given back."""

        self._check_live(request)
        capacity = min((len(t) * pool.page_size for t, pool in zip(request.tables, self.groups)), default=new_length)
        if request.tables and new_length > capacity:
            raise KVCacheError(f"length {new_length} exceeds the {capacity} tokens of pages held")
        request.length = new_length
        for table, pool in zip(request.tables, self.groups):
            if pool.window is None:
                continue
            # the next query sits at position new_length and reads keys > new_length - window
            dead_tokens = new_length - pool.window + 1
            for index in range(min(len(table), max(0, dead_tokens // pool.page_size))):
                if table[index] >= 0:
                    pool.allocator.free([table[index]])
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
        for table, pool in zip(request.tables, self.groups):
            pool.allocator.free([p for p in table if p >= 0])
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
