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

The reference's block manager also keeps a *prefix cache* (engine/src/block_manager.cpp:
24-64, 97-125, 184-224): every full page gets a hash chained over the pages before it; a
new prompt walks its full pages (all but the last token's), and where a page with the same
chain and the same tokens still exists it is shared instead of computed again, whether
another request still holds it or it was freed and not yet handed out again.  Pages are
counted by their users and freed by the last.  ``prefix_cache=True`` does the same here,
for models whose caches all keep every key and that have no per-request state (a window
gives pages back, and a state cannot skip tokens): ``admit(request, tokens)`` shares what
it finds and reports it through ``computed()``, ``commit(..., tokens)`` hashes the pages
a step has completed.

Host bookkeeping is plain Python and is tested without a GPU (``device=None`` allocates
no tensors).
"""
from __future__ import annotations

import hashlib
import heapq
from collections import deque
from dataclasses import dataclass
from typing import Deque, Dict, Hashable, List, Optional, Sequence, Tuple

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
    """Page ids 0..n-1; the lowest free id is handed out first.  Pages freed with
    ``cached=True`` (they still hold what the prefix cache knows them by) are handed out
    only when no other is left, the one freed longest ago first.  ``take`` claims one given
    free page (the prefix cache revives pages this way); its entry then is stale and is
    skipped when it comes up."""

    def __init__(self, num_pages: int):
        if num_pages <= 0:
            raise CacheError("a page pool needs at least one page")
        self.num_pages = num_pages
        self._stamp = [0] * num_pages          # of the page's latest entry
        self._free = [(p, 0) for p in range(num_pages)]      # heap of (page, stamp)
        heapq.heapify(self._free)
        self._cached: Deque[Tuple[int, int]] = deque()       # (page, stamp), oldest first
        self._held = [False] * num_pages
        self._free_count = num_pages

    @property
    def free_count(self) -> int:
        return self._free_count

    def is_free(self, page: int) -> bool:
        return 0 <= page < self.num_pages and not self._held[page]

    def _valid(self, entry: Tuple[int, int]) -> bool:
        page, stamp = entry
        return not self._held[page] and self._stamp[page] == stamp

    def alloc(self) -> int:
        if self._free_count == 0:
            raise OutOfPages("no free page")
        while self._free:
            entry = heapq.heappop(self._free)
            if self._valid(entry):
                break
        else:
            while True:
                entry = self._cached.popleft()
                if self._valid(entry):
                    break
        page = entry[0]
        self._held[page] = True
        self._free_count -= 1
        return page

    def take(self, page: int) -> None:
        if not self.is_free(page):
            raise CacheError(f"page {page} is taken but not free")
        self._held[page] = True
        self._free_count -= 1

    def free(self, page: int, cached: bool = False) -> None:
        if not 0 <= page < self.num_pages or not self._held[page]:
            raise CacheError(f"page {page} is freed but not held")
        self._held[page] = False
        self._free_count += 1
        self._stamp[page] += 1
        if cached:
            self._cached.append((page, self._stamp[page]))
        else:
            heapq.heappush(self._free, (page, self._stamp[page]))

    def audit(self) -> None:
        listed = [e[0] for e in list(self._free) + list(self._cached) if self._valid(e)]
        if len(set(listed)) != len(listed):
            raise CacheError("a page is on the free lists twice")
        if set(listed) != {p for p in range(self.num_pages) if not self._held[p]}:
            raise CacheError("pages lost or both held and free")
        if len(listed) != self._free_count:
            raise CacheError("the count of free pages is wrong")


@dataclass
class LayerCacheView:
    """What one visit of a mixer sees of the cache."""
    kv: Optional[torch.Tensor]            # planes of one shape: [pages, planes, heads, page_size, width]; else None
    block_table: Optional[torch.Tensor]   # [slots, max_pages] int32, -1 where no page
    page_size: int
    writes: bool
    state: Optional[torch.Tensor]         # [slots, *state shape]
    window: Optional[int] = None
    planes: Tuple[torch.Tensor, ...] = ()  # per plane a view [pages, heads, page_size, width] of the cache's pages


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
        self.users = [0] * num_pages          # requests that list the page
        # prefix cache: a page's chained hash and tokens while it holds what they say
        self.hash_of: List[Optional[bytes]] = [None] * num_pages
        self.tokens_of: List[Optional[Tuple[int, ...]]] = [None] * num_pages
        self.by_hash: Dict[bytes, int] = {}

    def take_new(self) -> int:
        """A fresh page for one user; what it held before is forgotten."""
        page = self.pool.alloc()
        self.forget(page)
        self.users[page] = 1
        return page

    def drop(self, page: int) -> None:
        """One user less; the last one frees the page (it keeps its hash until handed out again)."""
        if self.users[page] <= 0:
            raise CacheError(f"page {page} is given back but has no user")
        self.users[page] -= 1
        if self.users[page] == 0:
            self.pool.free(page, cached=self.hash_of[page] is not None)

    def forget(self, page: int) -> None:
        h = self.hash_of[page]
        if h is not None and self.by_hash.get(h) == page:
            del self.by_hash[h]
        self.hash_of[page] = self.tokens_of[page] = None

    def dead_before(self, computed: int) -> int:
        """First page index that a query at position >= computed can still read."""
        if self.window is None:
            return 0
        first_key = max(0, computed - self.window + 1)
        return first_key // self.page_size


class CacheManager:
    def __init__(self, needs: Dict[int, Tuple[Optional[CacheSpec], Optional[StateSpec]]],
                 page_size: int, num_pages, max_slots: int, max_seq_len: int,
                 dtype: torch.dtype = torch.bfloat16, device=None, prefix_cache: bool = False):
        """``needs``: per cache id what its mixer asks for (``Model.cache_needs()``).
        ``num_pages``: pages of every group, or a dict ``{window or None: pages}``.
        ``prefix_cache``: share full pages between requests whose tokens agree up to them
        (only if every cache keeps all keys and no mixer has a state; else it stays off)."""
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
        self._windowed = [g for g in self.groups.values() if g.window is not None]
        self._one_group = next(iter(self.groups.values())) if len(self.groups) == 1 else None
        self.prefix_active = bool(prefix_cache) and set(self.groups) == {None} \
            and all(state is None for _, state in needs.values())
        self._tokens: List[Optional[List[int]]] = [None] * max_slots   # of the request, while they are known
        self._hashed = [0] * max_slots         # pages of the slot that carry a hash
        self._chain: List[bytes] = [b""] * max_slots                   # hash of the last of them
        self.prefix_hit_pages = 0
        self.prefix_lookups = 0
        self.pages: Dict[int, torch.Tensor] = {}                       # per cache [pages, elements of a page]
        self.planes: Dict[int, Tuple[torch.Tensor, ...]] = {}
        self.kv: Dict[int, torch.Tensor] = {}                          # the same memory, where all planes have one shape
        self.state: Dict[int, torch.Tensor] = {}
        if device is not None:
            self._allocate_device()

    # ------------------------------------------------------------------ device memory
    def _allocate_device(self) -> None:
        for cache_id, (spec, state) in self._specs.items():
            if spec is not None:
                # a page holds its planes one after the other, each [heads, page_size, width]: the tokens
                # of one head of one plane are one contiguous block
                g = self._cache_group[cache_id]
                flat = torch.zeros((g.pool.num_pages, self.page_size * spec.elements_per_token),
                                   dtype=self.dtype, device=self.device)
                views, at = [], 0
                for heads, width in spec.planes:
                    n = heads * self.page_size * width
                    views.append(flat[:, at:at + n].unflatten(1, (heads, self.page_size, width)))
                    at += n
                self.pages[cache_id], self.planes[cache_id] = flat, tuple(views)
                if spec.uniform:
                    heads, width = spec.planes[0]
                    self.kv[cache_id] = flat.view(g.pool.num_pages, len(spec.planes), heads, self.page_size, width)
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
                out[spec.window] = out.get(spec.window, 0) + spec.elements_per_token * page_size * size
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
            window=None if g is None else g.window, planes=self.planes.get(cache_id, ()))

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

    def admit(self, request: Hashable, tokens: Optional[Sequence[int]] = None) -> int:
        """Give a request its slot (row of the block tables, index of its state).  With the
        prefix cache on and the request's ``tokens`` given, full pages whose chain of hashes
        and tokens are already in the cache are shared (never the page of the last token: at
        least one token is computed); ``computed(request)`` then says how many tokens that
        covers, and the request's first step starts there."""
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
        self._tokens[slot], self._hashed[slot], self._chain[slot] = None, 0, b""
        if self.prefix_active and tokens is not None:
            self._tokens[slot] = []
            self._share_prefix(slot, [int(t) for t in tokens])
        return slot

    @staticmethod
    def _page_hash(previous: bytes, tokens: Sequence[int]) -> bytes:
        """Chained over the pages before (the reference chains FNV-1a the same way,
        engine/src/block_manager.cpp:24-40); a hit is only trusted if the tokens agree too."""
        return hashlib.blake2b(previous + np.asarray(tokens, dtype=np.int64).tobytes(), digest_size=16).digest()

    def _share_prefix(self, slot: int, tokens: List[int]) -> None:
        g, ps = self.groups[None], self.page_size
        chain, hits = b"", 0
        while (hits + 1) * ps <= min(len(tokens) - 1, self.max_seq_len):
            page_tokens = tuple(tokens[hits * ps:(hits + 1) * ps])
            h = self._page_hash(chain, page_tokens)
            self.prefix_lookups += 1
            page = g.by_hash.get(h)
            if page is None or g.tokens_of[page] != page_tokens:
                break
            if g.users[page] == 0:
                g.pool.take(page)              # freed, but not handed out again since
            g.users[page] += 1
            g.table[slot, hits] = page
            g.dirty = True
            chain, hits = h, hits + 1
        self.prefix_hit_pages += hits
        g.end_page[slot] = hits
        self._reserved[slot] = self._computed[slot] = hits * ps
        self._tokens[slot] = tokens[:hits * ps]
        self._hashed[slot], self._chain[slot] = hits, chain

    def _covered(self, slot: int) -> int:
        """Tokens [0, n) that the slot's pages cover in every group."""
        if self._one_group is not None:
            return self._one_group.end_page[slot] * self.page_size
        return min(g.end_page[slot] for g in self.groups.values()) * self.page_size if self.groups else 0

    def try_reserve(self, request: Hashable, new_len: int) -> bool:
        """``reserve`` if it can be done, else nothing and False (one look-up for the common case
        of a decode step whose page is there already)."""
        slot = self._slot_of[request]
        if new_len <= self._covered(slot) and new_len <= self.max_seq_len:
            if new_len > self._reserved[slot]:
                self._reserved[slot] = new_len
            return True
        if not self.can_reserve(request, new_len):
            return False
        self.reserve(request, new_len)
        return True

    def pages_needed(self, request: Hashable, new_len: int) -> Dict[Optional[int], int]:
        """Pages each group must still hand out so that tokens [0, new_len) are covered."""
        slot = self._slot_of[request]
        want_end = -(-new_len // self.page_size)
        return {k: max(0, want_end - max(g.end_page[slot], g.first_page[slot]))
                for k, g in self.groups.items()}

    def can_reserve(self, request: Hashable, new_len: int) -> bool:
        if new_len <= self._covered(self._slot_of[request]):
            return new_len <= self.max_seq_len   # the pages are there already (most decode steps)
        if new_len > self.max_seq_len:
            return False
        need = self.pages_needed(request, new_len)
        return all(self.groups[k].pool.free_count >= n for k, n in need.items())

    def reserve(self, request: Hashable, new_len: int) -> None:
        """Cover tokens [0, new_len) with pages in every group, or change nothing."""
        slot = self._slot_of[request]
        if new_len <= self._covered(slot) and new_len <= self.max_seq_len:
            if new_len > self._reserved[slot]:
                self._reserved[slot] = new_len
            return
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
                g.table[slot, p] = g.take_new()
                g.dirty = True
            g.end_page[slot] = max(g.end_page[slot], want_end)
        self._reserved[slot] = max(self._reserved[slot], new_len)

    def commit(self, request: Hashable, computed_len: int, tokens: Optional[Sequence[int]] = None) -> None:
        """Tokens [0, computed_len) are now in the cache.  Windowed groups give back the
        pages that no later query can read.  ``tokens``: the ones this step added, for the
        prefix cache (a request whose tokens are not told stops being hashed); a negative one
        stands for a token that is computed but not known on the host yet: its page waits for
        ``fill_token`` before it gets a hash."""
        slot = self._slot_of[request]
        if computed_len > self._reserved[slot]:
            raise CacheError("more tokens computed than pages were reserved for")
        before = self._computed[slot]
        self._computed[slot] = computed_len
        for g in self._windowed:
            dead = min(g.dead_before(computed_len), g.end_page[slot])
            for p in range(g.first_page[slot], dead):
                g.drop(int(g.table[slot, p]))
                g.table[slot, p] = -1
                g.dirty = True
            g.first_page[slot] = max(g.first_page[slot], dead)
        if self.prefix_active and self._tokens[slot] is not None:
            if tokens is None or len(tokens) != computed_len - before:
                self._tokens[slot] = None
            else:
                self._tokens[slot].extend(int(t) for t in tokens)
                self._hash_full_pages(slot)

    def _hash_full_pages(self, slot: int) -> None:
        g, ps, known = self.groups[None], self.page_size, self._tokens[slot]
        while (self._hashed[slot] + 1) * ps <= len(known):
            i = self._hashed[slot]
            page_tokens = tuple(known[i * ps:(i + 1) * ps])
            if min(page_tokens) < 0:           # a token of this page is still to be told
                break
            h = self._page_hash(self._chain[slot], page_tokens)
            page = int(g.table[slot, i])
            if h not in g.by_hash:             # the first page with this content stands for it
                g.forget(page)
                g.hash_of[page], g.tokens_of[page] = h, page_tokens
                g.by_hash[h] = page
            self._hashed[slot], self._chain[slot] = i + 1, h

    def fill_token(self, request: Hashable, position: int, token: int) -> None:
        """The token at ``position`` of the request, committed as unknown, is ``token``."""
        slot = self._slot_of.get(request)
        if slot is None or not self.prefix_active:
            return
        known = self._tokens[slot]
        if known is not None and position < len(known) and known[position] < 0:
            known[position] = int(token)
            self._hash_full_pages(slot)

    def release(self, request: Hashable) -> None:
        """The request has ended (or is preempted): all it holds is given back."""
        slot = self._slot_of.pop(request)
        del self._request_of[slot]
        for g in self.groups.values():
            for p in range(g.end_page[slot] - 1, g.first_page[slot] - 1, -1):
                g.drop(int(g.table[slot, p]))
                g.table[slot, p] = -1
                g.dirty = True
            g.first_page[slot] = g.end_page[slot] = 0
        self._reserved[slot] = self._computed[slot] = 0
        self._tokens[slot], self._hashed[slot], self._chain[slot] = None, 0, b""
        heapq.heappush(self._free_slots, slot)

    def pages_of(self, request: Hashable) -> Dict[Optional[int], List[int]]:
        slot = self._slot_of[request]
        return {k: [int(x) for x in g.table[slot, g.first_page[slot]:g.end_page[slot]]]
                for k, g in self.groups.items()}

    def audit(self) -> None:
        """No page lost, held twice or freed twice; tables agree with the pools."""
        for g in self.groups.values():
            g.pool.audit()
            seen: Dict[int, int] = {}
            for slot in range(self.max_slots):
                live = slot in self._request_of
                row = g.table[slot]
                held = [int(x) for x in row if x >= 0]
                if not live and held:
                    raise CacheError(f"free slot {slot} still lists pages")
                inside = [int(x) for x in row[g.first_page[slot]:g.end_page[slot]]]
                if live and (sorted(held) != sorted(inside) or any(x < 0 for x in inside)):
                    raise CacheError(f"slot {slot}: table and page range disagree")
                if len(set(held)) != len(held):
                    raise CacheError(f"slot {slot} lists a page twice")
                for p in held:
                    if p in seen and not self.prefix_active:
                        raise CacheError(f"page {p} is held twice")
                    if not g.pool._held[p]:
                        raise CacheError(f"page {p} is in a table but free")
                    seen[p] = seen.get(p, 0) + 1
            if len(seen) != g.pool.num_pages - g.pool.free_count:
                raise CacheError("a page is held by nobody")
            for p in range(g.pool.num_pages):
                if g.users[p] != seen.get(p, 0):
                    raise CacheError(f"page {p} counts {g.users[p]} users but {seen.get(p, 0)} tables list it")
            for h, p in g.by_hash.items():
                if g.hash_of[p] != h or g.tokens_of[p] is None:
                    raise CacheError(f"the prefix cache points at page {p}, which does not carry that hash")
        if len(self._free_slots) + len(self._slot_of) != self.max_slots:
            raise CacheError("a slot is lost")
