"""The cache manager: pages of keys and values with a block table per request, in groups, and
slots of fixed-size state per request.

Layer calls whose mixers have the same need (same key/value heads and head size, same window)
form a *group*: the group has one pool of pages, and one page id addresses that page in every
layer call of the group (the reference has a single such group: the same page id indexes every
layer's k_cache/v_cache, tokasaurus/model/kv_cache.py:27-54, tokasaurus/model/llama.py:675-691).
A request holds one block table per group.  Pages are handed out as the request's tokens need
them (tokasaurus/manager/allocator.py:254-296 ``allocate_up_to_length``), given back when the
request ends (tokasaurus/manager/types.py:324-338 ``deallocate``) or, in a group whose mixer sees
only a window of keys, as soon as the window has moved past them.  Device layout of a group:
``[layer call, k|v, page, kv head, slot in page, head_dim]``.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Mapping

import numpy as np
import torch

from tokasaurus_b200.cache.pages import NoSpaceError, PageAllocator
from tokasaurus_b200.cache.slots import StateSlotAllocator
from tokasaurus_b200.parts.base import PagedCacheNeed, StateNeed

_DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16, "int32": torch.int32}


@dataclass
class CacheGroup:
    index: int
    need: PagedCacheNeed
    entries: list[int]
    allocator: PageAllocator
    storage: torch.Tensor | None = None  # [len(entries), 2, pages, kv heads, page_size, head_dim]

    def bytes_per_token(self, element_size: int) -> int:
        return 2 * len(self.entries) * self.need.n_kv_heads * self.need.head_dim * element_size


@dataclass
class PagedLayerCache:
    group: int
    k: torch.Tensor | None
    v: torch.Tensor | None
    page_size: int
    writable: bool = True


@dataclass
class StateLayerCache:
    state: torch.Tensor | None  # [slots, *shape]
    writable: bool = True


@dataclass
class RequestCache:
    request: object
    slot: int
    tables: list[list[int]]  # per group; -1 where a page was given back behind a window
    released: list[int] = field(default_factory=list)  # per group: leading pages already given back
    arrays: dict[int, np.ndarray] = field(default_factory=dict)  # per group: tables[g] as int32, made on demand

    def live_pages(self, g: int) -> list[int]:
        return [p for p in self.tables[g] if p >= 0]

    def table_array(self, g: int) -> np.ndarray:
        """``tables[g]`` as an int32 array.  A step of many requests at long contexts brings thousands of page
        ids; turning Python lists into an array every step costs more than everything else the host does for
        the step, so the array is kept and made anew only when the table has grown (or lost pages behind a
        window, which drops it)."""
        a = self.arrays.get(g)
        if a is None or a.shape[0] != len(self.tables[g]):
            a = np.asarray(self.tables[g], dtype=np.int32)
            self.arrays[g] = a
        return a


class CacheManager:
    def __init__(self, needs: Mapping[int, PagedCacheNeed | StateNeed | None], page_size: int, num_pages: int,
                 max_requests: int, dtype: torch.dtype = torch.bfloat16, device: torch.device | str | None = None,
                 max_step_tokens: int | None = None):
        """``needs``: {cache entry: need of the mixer using it} (``DecoderModel.cache_entries``).
        ``device=None`` keeps the books only (no device memory), for tests of the accounting.

        ``num_pages`` is a count of tokens a request may hold, in pages: every group whose mixers see all keys
        gets a pool of that many pages (a token needs an entry in each of them), so the memory is the sum over the
        groups of ``num_pages`` times the group's bytes a page (``device_bytes_by_group``).  A windowed group needs
        less: with ``max_step_tokens`` given (the most tokens one request brings in a step) its pool is capped at
        what ``max_requests`` requests can hold at once: a window, a step's tokens and the one token of a step
        launched ahead each, and a page for where the window starts inside a page."""
        if page_size <= 0:
            raise ValueError("page_size must be positive")
        self.page_size = page_size
        self.num_pages = num_pages
        self.max_step_tokens = max_step_tokens
        self.dtype = dtype
        self.device = torch.device(device) if device is not None else None
        self.groups: list[CacheGroup] = []
        self._entry_group: dict[int, tuple[int, int]] = {}  # entry -> (group, index within group)
        self._state: dict[int, torch.Tensor | None] = {}
        self._state_need: dict[int, StateNeed] = {}
        by_need: dict[PagedCacheNeed, CacheGroup] = {}
        for entry in sorted(needs):
            need = needs[entry]
            if isinstance(need, PagedCacheNeed):
                g = by_need.get(need)
                if g is None:
                    pool = num_pages
                    if need.window and max_step_tokens is not None:
                        pool = min(num_pages, max_requests * (self.pages_for(need.window + max_step_tokens + 1) + 1))
                    g = CacheGroup(len(self.groups), need, [], PageAllocator(pool))
                    by_need[need] = g
                    self.groups.append(g)
                self._entry_group[entry] = (g.index, len(g.entries))
                g.entries.append(entry)
            elif isinstance(need, StateNeed):
                self._state_need[entry] = need
            elif need is not None:
                raise TypeError(f"cache entry {entry}: unknown need {need!r}")
        self.slots = StateSlotAllocator(max_requests)
        self.requests: dict[object, RequestCache] = {}
        self.last_token: torch.Tensor | None = None
        if self.device is not None:
            for g in self.groups:
                n = g.need
                g.storage = torch.zeros((len(g.entries), 2, g.allocator.num_pages, n.n_kv_heads, page_size, n.head_dim),
                                        dtype=dtype, device=self.device)
            for entry, need in self._state_need.items():
                self._state[entry] = torch.zeros((max_requests, *need.shape), dtype=_DTYPES[need.dtype],
                                                 device=self.device)
            self.last_token = torch.zeros((max_requests,), dtype=torch.int32, device=self.device)

    # ------------------------------------------------------------------ sizes
    def pages_for(self, n_tokens: int) -> int:
        return (n_tokens + self.page_size - 1) // self.page_size

    def device_bytes(self) -> int:
        return sum(self.device_bytes_by_group())

    def device_bytes_by_group(self) -> list[int]:
        """Bytes of key/value storage of each cache group (0 where the manager keeps books only)."""
        return [g.storage.numel() * g.storage.element_size() if g.storage is not None else 0 for g in self.groups]

    def num_free_pages(self) -> list[int]:
        return [g.allocator.num_free for g in self.groups]

    # ------------------------------------------------------------------ requests
    def admit(self, request: object) -> RequestCache:
        if request in self.requests:
            raise ValueError(f"request {request!r} is already admitted")
        slot = self.slots.allocate(request)
        rc = RequestCache(request, slot, [[] for _ in self.groups], [0 for _ in self.groups])
        self.requests[request] = rc
        for st in self._state.values():
            if st is not None:
                st[slot].zero_()
        return rc

    def pages_missing(self, request: object, n_tokens: int, windowed_tokens: int | None = None) -> list[int]:
        """Per group: pages to add so that positions [0, n_tokens) have a page; in groups with a window,
        positions [0, min(n_tokens, windowed_tokens)) if ``windowed_tokens`` is given."""
        rc = self.requests[request]
        need = self.pages_for(n_tokens)
        need_w = need if windowed_tokens is None else self.pages_for(min(n_tokens, windowed_tokens))
        return [max(0, (need_w if g.need.window else need) - len(rc.tables[g.index])) for g in self.groups]

    def can_hold(self, request: object, n_tokens: int, windowed_tokens: int | None = None) -> bool:
        return all(m <= g.allocator.num_free
                   for m, g in zip(self.pages_missing(request, n_tokens, windowed_tokens), self.groups))

    def ensure_capacity(self, request: object, n_tokens: int, windowed_tokens: int | None = None) -> None:
        """Give the request pages for positions [0, n_tokens) in every group, or raise ``NoSpaceError`` and change
        nothing.  A group with a window only needs pages for the tokens that have gone, or are about to go,
        through the model: ``windowed_tokens`` (at most ``n_tokens``) says how far such groups are filled, so that
        a long prompt takes pages there portion by portion while the pages behind the window come back."""
        rc = self.requests[request]
        if windowed_tokens is None:
            need = (n_tokens + self.page_size - 1) // self.page_size
            if all(len(t) >= need for t in rc.tables):
                return  # the common case of a decode step: the token's page is there already
        missing = self.pages_missing(request, n_tokens, windowed_tokens)
        for m, g in zip(missing, self.groups):
            if m > g.allocator.num_free:
                raise NoSpaceError(
                    f"request {request!r} needs {m} more pages in cache group {g.index}, "
                    f"{g.allocator.num_free} of {g.allocator.num_pages} are free"
                )
        for m, g in zip(missing, self.groups):
            if m:
                rc.tables[g.index].extend(g.allocator.allocate(m, request))

    def release_behind_window(self, request: object, n_processed: int) -> int:
        """After ``n_processed`` tokens of the request have gone through the model, give back the
        pages of windowed groups that no later token can see.  Returns how many pages came back."""
        rc = self.requests[request]
        count = 0
        for g in self.groups:
            w = g.need.window
            if not w:
                continue
            # the next query sits at position >= n_processed and sees keys > position - w
            first_visible = max(0, n_processed - w + 1)
            full_pages_behind = min(first_visible // self.page_size, len(rc.tables[g.index]))
            lo = rc.released[g.index]
            if full_pages_behind > lo:
                pages = rc.tables[g.index][lo:full_pages_behind]
                g.allocator.release(pages, request)
                for i in range(lo, full_pages_behind):
                    rc.tables[g.index][i] = -1
                rc.arrays.pop(g.index, None)
                rc.released[g.index] = full_pages_behind
                count += len(pages)
        return count

    def free(self, request: object) -> None:
        rc = self.requests.pop(request)
        for g in self.groups:
            g.allocator.release(rc.live_pages(g.index), request)
        self.slots.release(rc.slot, request)

    def table(self, request: object, group: int) -> list[int]:
        return self.requests[request].tables[group]

    def slot(self, request: object) -> int:
        return self.requests[request].slot

    # ------------------------------------------------------------------ device views
    def layer_cache(self, entry: int, writable: bool = True):
        if entry in self._entry_group:
            g, i = self._entry_group[entry]
            st = self.groups[g].storage
            return PagedLayerCache(g, st[i, 0] if st is not None else None, st[i, 1] if st is not None else None,
                                   self.page_size, writable)
        if entry in self._state_need:
            return StateLayerCache(self._state.get(entry), writable)
        return None

    def group_of(self, entry: int) -> int | None:
        ge = self._entry_group.get(entry)
        return ge[0] if ge else None

    # ------------------------------------------------------------------ invariants
    def check(self) -> None:
        """No page lost, held twice or freed twice; every table entry is owned by its request."""
        self.slots.check()
        for g in self.groups:
            g.allocator.check()
            held: dict[int, object] = {}
            for req, rc in self.requests.items():
                for p in rc.live_pages(g.index):
                    if p in held:
                        raise AssertionError(f"group {g.index}: page {p} is held by {held[p]!r} and {req!r}")
                    held[p] = req
                    if g.allocator.owner_of(p) != req:
                        raise AssertionError(f"group {g.index}: page {p} in {req!r}'s table is owned by "
                                             f"{g.allocator.owner_of(p)!r}")
            if len(held) + g.allocator.num_free != g.allocator.num_pages:
                raise AssertionError(f"group {g.index}: {len(held)} held + {g.allocator.num_free} free != "
                                     f"{g.allocator.num_pages} pages")
        slots = [rc.slot for rc in self.requests.values()]
        if len(set(slots)) != len(slots):
            raise AssertionError("two requests share a state slot")
