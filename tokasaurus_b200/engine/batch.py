"""One step's input: a batch of (request, its next tokens), turned into device arrays.

The reference ships a step as Python lists (``ModelInput``, tokasaurus/model/types.py:343-384,
built by ``seqs_to_input``, tokasaurus/manager/input_building.py:151-320) and turns them into
several tensors that are copied one by one (tokasaurus/model/utils.py:113-202,227-264).  Here
all integer arrays of a step are packed into one pinned buffer and reach the device in one copy;
the views below are slices of that device buffer.

Per token: id (or -1: "the token this request sampled last", read on the device from the slot
table as in tokasaurus/model/basic_worker.py:101-114), position, and the row of its request in the
batch.  Per request: state slot, first token row, number of tokens, key/value length after this
step.  Per cache group: the block tables in CSR form (``indptr`` over requests, ``page_ids``), as in
tokasaurus/model/types.py:41-56,122-147.  ``logit_rows``: token rows whose logits are wanted.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Sequence

import numpy as np
import torch


_TORCH_OF = {"float32": torch.float32, "int64": torch.int64, "uint64": torch.int64, "uint32": torch.int32}


@dataclass
class StepEntry:
    request: object
    tokens: Sequence[int] | None  # None: one token, the one this request sampled last (kept on the device)
    start: int  # position of the first of these tokens within the request
    want: Sequence[int] = ()  # indices into ``tokens`` whose logits are wanted

    @property
    def n_tokens(self) -> int:
        return 1 if self.tokens is None else len(self.tokens)


@dataclass
class GroupTables:
    indptr: torch.Tensor  # int32 [S + 1]
    page_ids: torch.Tensor  # int32 [sum of pages]


@dataclass
class HostBatch:
    """The same step as plain numpy arrays, for planners and for mixers that loop over requests."""

    token_ids: np.ndarray
    positions: np.ndarray
    token_seq: np.ndarray
    seq_slot: np.ndarray
    seq_q_start: np.ndarray
    seq_q_len: np.ndarray
    seq_kv_len: np.ndarray
    logit_rows: np.ndarray
    table_indptr: list[np.ndarray]
    table_pages: list[np.ndarray]
    requests: list[object] = field(default_factory=list)


class StepContext:
    """Everything a part may look at while it runs one step."""

    def __init__(self, host: HostBatch, cache_manager, device: torch.device, stager: "Stager",
                 extra: dict[str, np.ndarray] | None = None, plans: dict | None = None):
        self.host = host
        self.cache_manager = cache_manager
        self.device = device
        self.n_tokens = int(host.token_ids.shape[0])
        self.n_seqs = int(host.seq_slot.shape[0])
        self.all_rows_wanted = (
            host.logit_rows.shape[0] == self.n_tokens
            and bool(np.array_equal(host.logit_rows, np.arange(self.n_tokens, dtype=np.int32)))
        )
        arrays = [host.token_ids, host.positions, host.token_seq, host.seq_slot, host.seq_q_start, host.seq_q_len,
                  host.seq_kv_len, host.logit_rows]
        n_groups = len(host.table_indptr)
        extra = extra or {}
        plans = plans or {}
        flat = [(key, name, arr) for key, d in plans.items() for name, arr in d.items()]
        # The page ids go last: a step graph stages them at the capacity of the page pool, and only the part in
        # use (the last entry of the row pointers) is copied.
        everything = arrays + list(host.table_indptr) + list(extra.values()) + [a for _, _, a in flat] + list(host.table_pages)
        used_of_last = int(host.table_indptr[-1][-1]) if n_groups else None
        views = stager.upload(everything, used_of_last)
        at = len(arrays)
        indptrs = views[at:at + n_groups]
        at += n_groups
        self.extra = dict(zip(extra.keys(), views[at:at + len(extra)]))
        at += len(extra)
        self.plans: dict = {}
        self.plan_caps: dict | None = None
        self.host_plans = plans
        for (key, name, _), v in zip(flat, views[at:at + len(flat)]):
            self.plans.setdefault(key, {})[name] = v
        at += len(flat)
        (self.token_ids, self.positions, self.token_seq, self.seq_slot, self.seq_q_start, self.seq_q_len,
         self.seq_kv_len, self.logit_rows) = views[:8]
        self.tables = [GroupTables(indptrs[g], views[at + g]) for g in range(n_groups)]
        self.last_token = cache_manager.last_token
        self.status = stager.status

    def layer_cache(self, entry: int, writable: bool = True):
        return self.cache_manager.layer_cache(entry, writable)


class Stager:
    """Pinned host buffers and their device twin; ``upload`` packs int32 arrays into a host buffer and
    copies once.  Segments start on 16-byte boundaries.  ``host_buffers``: how many pinned buffers take turns, so
    that as many uploads can be in the stream at a time without the host waiting for the oldest to be over (the
    device twin is one: copies into it are ordered by the stream behind the kernels that read it)."""

    def __init__(self, device: torch.device, capacity_ints: int = 1 << 16, host_buffers: int = 1):
        self.device = device
        self.status = torch.zeros((1,), dtype=torch.int32, device=device)
        self.host_buffers = max(1, int(host_buffers))
        self._alloc(capacity_ints)

    def _alloc(self, n: int) -> None:
        self.capacity = n
        pin = self.device.type == "cuda"
        self._hosts = [torch.empty((n,), dtype=torch.int32, pin_memory=pin) for _ in range(self.host_buffers)]
        self._hosts_np = [h.numpy() for h in self._hosts]
        self.dev = torch.empty((n,), dtype=torch.int32, device=self.device)
        self.bytes_last_upload = 0
        self._copied = [torch.cuda.Event() if pin else None for _ in range(self.host_buffers)]
        self._pending = [False] * self.host_buffers
        self._turn = 0

    def upload(self, arrays: Sequence[np.ndarray], used_of_last: int | None = None) -> list[torch.Tensor]:
        """Pack the arrays and copy them to the device in one copy; returns their device views.  ``used_of_last``:
        only this many leading elements of the LAST array hold anything (the rest is padding that nothing reads),
        so the copy ends there."""
        offs = []
        total = 0
        kinds = [a.dtype for a in arrays]
        arrays = [a if a.dtype == np.int32 else np.ascontiguousarray(a).view(np.int32) for a in arrays]
        for a, k in zip(arrays, kinds):
            if k.itemsize not in (4, 8):
                raise TypeError("step arrays have 4- or 8-byte elements")
            offs.append(total)
            total += (a.shape[0] + 3) & ~3
        total = max(total, 4)
        if total > self.capacity:
            # wait for copies in flight from the old pinned buffer before dropping it
            if self.device.type == "cuda":
                torch.cuda.current_stream(self.device).synchronize()
            self._alloc(max(total, 2 * self.capacity))
        turn = self._turn
        self._turn = (turn + 1) % self.host_buffers
        host, host_np = self._hosts[turn], self._hosts_np[turn]
        if self._pending[turn]:
            self._copied[turn].synchronize()  # the last copy out of this pinned buffer must be over before it is rewritten
            self._pending[turn] = False
        n_copy = total
        if used_of_last is not None and arrays:
            n_copy = max(4, offs[-1] + min(int(used_of_last), arrays[-1].shape[0]))
        for a, o in zip(arrays, offs):
            n = min(a.shape[0], n_copy - o)
            if n > 0:
                host_np[o:o + n] = a[:n]
        total_bytes = n_copy
        self.dev[:n_copy].copy_(host[:n_copy], non_blocking=True)
        if self._copied[turn] is not None:
            self._copied[turn].record()
            self._pending[turn] = True
        self.bytes_last_upload = total_bytes * 4
        out = []
        for a, o, k in zip(arrays, offs, kinds):
            v = self.dev[o:o + a.shape[0]]
            out.append(v if k == np.int32 else v.view(_TORCH_OF[k.name]))
        return out


def build_host_batch(entries: Sequence[StepEntry], cache_manager) -> HostBatch:
    """Lay the entries out as one batch.  Every request must already hold pages for the positions
    it brings (``CacheManager.ensure_capacity``)."""
    if all(e.tokens is None and len(e.want) == 1 and e.want[0] == 0 for e in entries):
        return _decode_host_batch(entries, cache_manager)
    return _general_host_batch(entries, cache_manager)


def _general_host_batch(entries: Sequence[StepEntry], cache_manager) -> HostBatch:
    seen = set()
    tok: list[int] = []
    pos: list[int] = []
    tseq: list[int] = []
    rows: list[int] = []
    slot, q_start, q_len, kv_len = [], [], [], []
    ps = cache_manager.page_size
    n_groups = len(cache_manager.groups)
    indptr = [[0] for _ in range(n_groups)]
    pages: list[list[np.ndarray]] = [[] for _ in range(n_groups)]  # per group: each request's page ids
    for s, e in enumerate(entries):
        if e.request in seen:
            raise ValueError(f"request {e.request!r} appears twice in one step")
        seen.add(e.request)
        n = e.n_tokens
        if n <= 0:
            raise ValueError(f"request {e.request!r} brings no tokens")
        rc = cache_manager.requests[e.request]
        end = e.start + n
        for g in range(n_groups):
            table = rc.table_array(g)
            need = (end + ps - 1) // ps
            if table.shape[0] < need:
                raise ValueError(f"request {e.request!r} holds {table.shape[0]} pages of group {g}, needs {need}")
            pages[g].append(table[:need])
            indptr[g].append(indptr[g][-1] + need)
        base = len(tok)
        tok.extend([-1] if e.tokens is None else [int(t) for t in e.tokens])
        pos.extend(range(e.start, end))
        tseq.extend([s] * n)
        for w in e.want:
            if not 0 <= w < n:
                raise ValueError(f"request {e.request!r}: wanted place {w} is outside its {n} tokens")
            rows.append(base + w)
        slot.append(rc.slot)
        q_start.append(base)
        q_len.append(n)
        kv_len.append(end)
    i32 = lambda x: np.asarray(x, dtype=np.int32)  # noqa: E731
    return HostBatch(i32(tok), i32(pos), i32(tseq), i32(slot), i32(q_start), i32(q_len), i32(kv_len), i32(rows),
                     [i32(x) for x in indptr],
                     [np.concatenate(x) if x else np.zeros((0,), dtype=np.int32) for x in pages],
                     [e.request for e in entries])


def _decode_host_batch(entries: Sequence[StepEntry], cache_manager) -> HostBatch:
    """``build_host_batch`` for a step in which every request brings the one token it sampled last and wants its
    logits (a decode step): the same arrays, made whole instead of request by request, which is what the host has
    time for when hundreds of requests decode."""
    S = len(entries)
    ps = cache_manager.page_size
    requests = cache_manager.requests
    ids = [e.request for e in entries]
    if len(set(ids)) != S:
        seen = set()
        for r in ids:
            if r in seen:
                raise ValueError(f"request {r!r} appears twice in one step")
            seen.add(r)
    rcs = [requests[r] for r in ids]
    start = np.fromiter((e.start for e in entries), dtype=np.int32, count=S)
    ar = np.arange(S, dtype=np.int32)
    need = (start + ps) // ps  # pages for positions [0, start + 1)
    need_list = need.tolist()
    indptrs, pages = [], []
    for g in range(len(cache_manager.groups)):
        tables = [rc.table_array(g) for rc in rcs]
        for r, t, n in zip(ids, tables, need_list):
            if t.shape[0] < n:
                raise ValueError(f"request {r!r} holds {t.shape[0]} pages of group {g}, needs {n}")
        indptr = np.zeros(S + 1, dtype=np.int32)
        np.cumsum(need, out=indptr[1:])
        indptrs.append(indptr)
        pages.append(np.concatenate([t[:n] for t, n in zip(tables, need_list)]) if S else np.zeros((0,), dtype=np.int32))
    slot = np.fromiter((rc.slot for rc in rcs), dtype=np.int32, count=S)
    return HostBatch(np.full(S, -1, dtype=np.int32), start, ar, slot, ar.copy(), np.ones(S, dtype=np.int32), start + 1,
                     ar.copy(), indptrs, pages, ids)
