"""The cache manager: keys and values in pages with a block table per request, and slots
for per-request state of fixed size.

The reference keeps one pool ``[layers, blocks, block_size, kv_dim]`` for keys and one for
values, in which one page id addresses that page in every layer
(model/src/qwen3_kv_cache.cpp:14-44, kernels/src/paged_attention_cuda.cu:63-65); its
``BlockManager`` hands out the lowest free id first, takes all pages of a prompt at
admission, one more when decoding crosses a page edge, and gives everything back when a
request finishes or is preempted (engine/src/block_manager.cpp:66-182).  It has one kind
of layer, so one group.

Here caches with the same need form a *group*: "every key" or "the last W keys".  A group
has its own pool of page ids and its own block table per request; inside a group one page
id addresses that page in every cache of the group.  A windowed group gives pages back as
soon as the window has passed them, while the request lives.  Each request also owns a
*slot* (its row in every block table); mixers that declare a fixed-size state get
``state[slot]``, zeroed at admission.  Qwen3 dense declares none.

Host bookkeeping is plain Python and is tested without a GPU (``device=None`` allocates
no tensors).
"""
from __future__ import annotations

import heapq
from dataclasses import dataclass
from typing import Dict, Hashable, List, Optional, Tuple

import numpy as np
import torch

from ..parts.spec import CacheSpec, StateSpec


class CacheError(RuntimeError):
    pass


class OutOfPages(CacheError):
    pass


class OutOfSlots(CacheError):
    pass


class PagePool:
    """Page ids 0..n-1; the lowest free id is handed out first."""

    def __init__(self, num_pages: int):
        if num_pages <= 0:
            raise CacheError("a page pool needs at least one page")
        self.num_pages = num_pages
        self._free = list(range(num_pages))
        heapq.heapify(self._free)
        self._held = [False] * num_pages

    @property
    def free_count(self) -> int:
        return len(self._free)

    def alloc(self) -> int:
        if not self._free:
            raise OutOfPages("no free page")
        page = heapq.heappop(self._free)
        self._held[page] = True
        return page

    def free(self, page: int) -> None:
        if not 0 <= page < self.num_pages or not self._held[page]:
            raise CacheError(f"page {page} is freed but not held")
        self._held[page] = False
        heapq.heappush(self._free, page)

    def audit(self) -> None:
        free = sorted(self._free)
        if len(set(free)) != len(free):
            raise CacheError("a page is on the free list twice")
        held = {p for p, h in enumerate(self._held) if h}
        if held & set(free) or len(held) + len(free) != self.num_pages:
            raise CacheError("pages lost or both held and free")


@dataclass
class LayerCacheView:
    """What one visit of a mixer sees of the cache."""
    kv: Optional[torch.Tensor]            # [pages, 2, kv_heads, page_size, head_dim]
    block_table: Optional[torch.Tensor]   # [slots, max_pages] int32, -1 where no page
    page_size: int
    writes: bool
    state: Optional[torch.Tensor]         # [slots, *state shape]
    window: Optional[int] = None


class _Group:
    def __init__(self, window: Optional[int], page_size: int, num_pages: int, max_slots: int,
                 max_pages_per_seq: int):
        self.window = window
        self.page_size = page_size
        self.pool = PagePool(num_pages)
        self.table = np.full((max_slots, max_pages_per_seq), -1, dtype=np.int32)
        self.end_page = [0] * max_slots       # pages [first_page, end_page) of a slot are held
        self.first_page = [0] * max_slots
        self.cache_ids: List[int] = []
        self.dirty = True
        self.device_table: Optional[torch.Tensor] = None
        self._staging: Optional[torch.Tensor] = None
        self._copied: Optional[torch.cuda.Event] = None

    def dead_before(self, computed: int) -> int:
        """First page index that a query at position >= computed can still read."""
        if self.window is None:
            return 0
        first_key = max(0, computed - self.window + 1)
        return first_key // self.page_size


class CacheManager:
    def __init__(self, needs: Dict[int, Tuple[Optional[CacheSpec], Optional[StateSpec]]],
                 page_size: int, num_pages, max_slots: int, max_seq_len: int,
                 dtype: torch.dtype = torch.bfloat16, device=None):
        """``needs``: per cache id what its mixer asks for (``Model.cache_needs()``).
        ``num_pages``: pages of every group, or a dict ``{window or None: pages}``."""
        if page_size <= 0 or max_slots <= 0 or max_seq_len <= 0:
            raise CacheError("page_size, max_slots and max_seq_len must be positive")
        self.page_size, self.max_slots, self.max_seq_len = page_size, max_slots, max_seq_len
        self.max_pages_per_seq = -(-max_seq_len // page_size)
        self.dtype, self.device = dtype, device
        self.groups: Dict[Optional[int], _Group] = {}
        self._cache_group: Dict[int, _Group] = {}
        self._specs = dict(needs)
        for cache_id in sorted(needs):
            spec, _ = needs[cache_id]
            if spec is None:
                continue
            key = spec.window
            if key not in self.groups:
                n = num_pages[key] if isinstance(num_pages, dict) else num_pages
                self.groups[key] = _Group(key, page_size, int(n), max_slots, self.max_pages_per_seq)
            self.groups[key].cache_ids.append(cache_id)
            self._cache_group[cache_id] = self.groups[key]
        self._free_slots = list(range(max_slots))
        heapq.heapify(self._free_slots)
        self._slot_of: Dict[Hashable, int] = {}
        self._request_of: Dict[int, Hashable] = {}
        self._reserved = [0] * max_slots       # tokens covered by pages
        self._computed = [0] * max_slots       # tokens whose keys and values are in the cache
        self.kv: Dict[int, torch.Tensor] = {}
        self.state: Dict[int, torch.Tensor] = {}
        if device is not None:
            self._allocate_device()

    # ------------------------------------------------------------------ device memory
    def _allocate_device(self) -> None:
        for cache_id, (spec, state) in self._specs.items():
            if spec is not None:
                g = self._cache_group[cache_id]
                self.kv[cache_id] = torch.zeros(
                    (g.pool.num_pages, 2, spec.kv_heads, self.page_size, spec.head_dim),
                    dtype=self.dtype, device=self.device)
            if state is not None:
                self.state[cache_id] = torch.zeros((self.max_slots, *state.shape),
                                                   dtype=getattr(torch, state.dtype), device=self.device)
        for g in self.groups.values():
            g.device_table = torch.full(g.table.shape, -1, dtype=torch.int32, device=self.device)
            if torch.device(self.device).type == "cuda":
                g._staging = torch.empty(g.table.shape, dtype=torch.int32).pin_memory()

    @staticmethod
    def bytes_per_page(needs, page_size: int, dtype: torch.dtype) -> Dict[Optional[int], int]:
        """Bytes one page id costs in each group (all caches of the group together)."""
        size = torch.empty((), dtype=dtype).element_size()
        out: Dict[Optional[int], int] = {}
        for spec, _ in needs.values():
            if spec is not None:
                out[spec.window] = out.get(spec.window, 0) + 2 * spec.kv_heads * page_size * spec.head_dim * size
        return out

    def sync(self) -> None:
        """Bring the device copies of the block tables up to date (current stream)."""
        for g in self.groups.values():
            if not g.dirty or g.device_table is None:
                continue
            host = torch.from_numpy(g.table)
            if g._staging is not None:
                if g._copied is not None:
                    g._copied.synchronize()
                g._staging.copy_(host)
                g.device_table.copy_(g._staging, non_blocking=True)
                g._copied = torch.cuda.Event()
                g._copied.record()
            else:
                g.device_table.copy_(host)
            g.dirty = False

    def view(self, cache_id: int, writes: bool = True) -> LayerCacheView:
        g = self._cache_group.get(cache_id)
        return LayerCacheView(
            kv=self.kv.get(cache_id), block_table=None if g is None else g.device_table,
            page_size=self.page_size, writes=writes, state=self.state.get(cache_id),
            window=None if g is None else g.window)

    # ------------------------------------------------------------------ requests
    @property
    def free_slots(self) -> int:
        return len(self._free_slots)

    def free_pages(self) -> Dict[Optional[int], int]:
        return {k: g.pool.free_count for k, g in self.groups.items()}

    def capacity_pages(self) -> Dict[Optional[int], int]:
        return {k: g.pool.num_pages for k, g in self.groups.items()}

    def slot_of(self, request: Hashable) -> int:
        return self._slot_of[request]

    def has(self, request: Hashable) -> bool:
        return request in self._slot_of

    def computed(self, request: Hashable) -> int:
        return self._computed[self._slot_of[request]]

    def admit(self, request: Hashable) -> int:
        """Give a request its slot (row of the block tables, index of its state)."""
        if request in self._slot_of:
            raise CacheError(f"request {request!r} is already admitted")
        if not self._free_slots:
            raise OutOfSlots("every request slot is taken")
        slot = heapq.heappop(self._free_slots)
        self._slot_of[request] = slot
        self._request_of[slot] = request
        self._reserved[slot] = self._computed[slot] = 0
        for g in self.groups.values():
            g.first_page[slot] = g.end_page[slot] = 0
        for s in self.state.values():
            s[slot].zero_()
        return slot

    def pages_needed(self, request: Hashable, new_len: int) -> Dict[Optional[int], int]:
        """Pages each group must still hand out so that tokens [0, new_len) are covered."""
        slot = self._slot_of[request]
        want_end = -(-new_len // self.page_size)
        return {k: max(0, want_end - max(g.end_page[slot], g.first_page[slot]))
                for k, g in self.groups.items()}

    def can_reserve(self, request: Hashable, new_len: int) -> bool:
        if new_len > self.max_seq_len:
            return False
        need = self.pages_needed(request, new_len)
        return all(self.groups[k].pool.free_count >= n for k, n in need.items())

    def reserve(self, request: Hashable, new_len: int) -> None:
        """Cover tokens [0, new_len) with pages in every group, or change nothing."""
        if new_len > self.max_seq_len:
            raise CacheError(f"{new_len} tokens exceed the maximum sequence length {self.max_seq_len}")
        if not self.can_reserve(request, new_len):
            raise OutOfPages(f"request {request!r} needs {self.pages_needed(request, new_len)} "
                             f"more pages, free are {self.free_pages()}")
        slot = self._slot_of[request]
        want_end = -(-new_len // self.page_size)
        for g in self.groups.values():
            start = max(g.end_page[slot], g.first_page[slot])
            for p in range(start, want_end):
                g.table[slot, p] = g.pool.alloc()
                g.dirty = True
            g.end_page[slot] = max(g.end_page[slot], want_end)
        self._reserved[slot] = max(self._reserved[slot], new_len)

    def commit(self, request: Hashable, computed_len: int) -> None:
        """Tokens [0, computed_len) are now in the cache.  Windowed groups give back the
        pages that no later query can read."""
        slot = self._slot_of[request]
        if computed_len > self._reserved[slot]:
            raise CacheError("more tokens computed than pages were reserved for")
        self._computed[slot] = computed_len
        for g in self.groups.values():
            dead = min(g.dead_before(computed_len), g.end_page[slot])
            for p in range(g.first_page[slot], dead):
                g.pool.free(int(g.table[slot, p]))
                g.table[slot, p] = -1
                g.dirty = True
            g.first_page[slot] = max(g.first_page[slot], dead)

    def release(self, request: Hashable) -> None:
        """The request has ended (or is preempted): all it holds is given back."""
        slot = self._slot_of.pop(request)
        del self._request_of[slot]
        for g in self.groups.values():
            for p in range(g.end_page[slot] - 1, g.first_page[slot] - 1, -1):
                g.pool.free(int(g.table[slot, p]))
                g.table[slot, p] = -1
                g.dirty = True
            g.first_page[slot] = g.end_page[slot] = 0
        self._reserved[slot] = self._computed[slot] = 0
        heapq.heappush(self._free_slots, slot)

    def pages_of(self, request: Hashable) -> Dict[Optional[int], List[int]]:
        slot = self._slot_of[request]
        return {k: [int(x) for x in g.table[slot, g.first_page[slot]:g.end_page[slot]]]
                for k, g in self.groups.items()}

    def audit(self) -> None:
        """No page lost, held twice or freed twice; tables agree with the pools."""
        for g in self.groups.values():
            g.pool.audit()
            seen = set()
            for slot in range(self.max_slots):
                live = slot in self._request_of
                row = g.table[slot]
                held = [int(x) for x in row if x >= 0]
                if not live and held:
                    raise CacheError(f"free slot {slot} still lists pages")
                inside = [int(x) for x in row[g.first_page[slot]:g.end_page[slot]]]
                if live and (sorted(held) != sorted(inside) or any(x < 0 for x in inside)):
                    raise CacheError(f"slot {slot}: table and page range disagree")
                for p in held:
                    if p in seen:
                        raise CacheError(f"page {p} is held twice")
                    if not g.pool._held[p]:
                        raise CacheError(f"page {p} is in a table but free")
                    seen.add(p)
            if len(seen) != g.pool.num_pages - g.pool.free_count:
                raise CacheError("a page is held by nobody")
        if len(self._free_slots) + len(self._slot_of) != self.max_slots:
            raise CacheError("a slot is lost")
