"""CUDA graphs for steps in which every request brings one token.

The reference records graphs for decode-only batches of 16, 32, ... 128 requests, pads a batch up
to the next recorded size and sends padded rows to a spare page (tokasaurus/model/utils.py:512-720,
:839-882; sizes from ``cudagraph_step``/``cudagraph_max_size``, tokasaurus/common_types.py:119-122).
Here a graph holds the whole step, model and sampler, for one padded batch size; it is recorded the
first time that size comes up.  The block tables are staged at the capacity of the whole page pool
and the attention work list at the most items the planner can make for that batch size, so neither
the contexts' lengths nor their growth ever ask for another graph.  All graphs share one memory
pool (they never run at the same time).  Every array of the step lives at a fixed place of the
graph's own staging buffer, so a replay is: fill the pinned copy, one copy to the device, one graph
launch.  Padded rows carry request row -1: the kernels skip them, nothing is written for them, no
spare page is needed.
"""

from __future__ import annotations

import numpy as np
import torch

from tokasaurus_b200.engine.batch import HostBatch, Stager, StepContext, StepEntry, build_host_batch


def _pow2_at_least(n: int, floor: int) -> int:
    c = floor
    while c < n:
        c *= 2
    return c


# padded token counts of steps that bring prompt portions (a step is padded up to the next of these)
TOKEN_BUCKETS = (16, 32, 48, 64, 96, 128, 192, 256, 384, 512, 768, 1024, 1536, 2048, 3072, 4096, 6144, 8192)


def _pad(a: np.ndarray, n: int, fill: int = 0) -> np.ndarray:
    out = np.full((n,), fill, dtype=a.dtype)
    out[: a.shape[0]] = a
    return out


class DecodeGraphs:
    def __init__(self, runner, sampler, max_size: int, step: int, max_tokens: int = 0,
                 max_pages_per_request: int | None = None, host_buffers: int = 2):
        """``max_pages_per_request``: the reference's ``cudagraph_max_kv_indices_per_seq`` (common_types.py:117):
        a step with a request that holds more pages than this runs without a graph.  (The reference sizes its
        graphs' block tables by it; here they are sized by the pool, so the option only keeps its meaning.)
        ``host_buffers``: pinned buffers a graph's inputs take turns in, one for each step that can be in the stream
        at a time."""
        self.host_buffers = host_buffers
        self.max_pages_per_request = max_pages_per_request
        self.runner = runner
        self.sampler = sampler
        self.max_size = max_size
        self.max_tokens = max_tokens  # steps with prompt portions of up to this many tokens run as graphs too (0: none)
        self.sizes = sorted({s for s in (1, 2, 4, 8) if s <= max_size} | set(range(step, max_size + 1, step)))
        self.graphs: dict[tuple, dict] = {}
        self.launches_per_replay = 0
        self.pool = None  # memory pool shared by all graphs

    def _tables_fit(self, entries) -> bool:
        limit = self.max_pages_per_request
        if limit is None:
            return True
        pages_for = self.runner.cache.pages_for
        return all(pages_for(e.start + e.n_tokens) <= limit for e in entries)

    def _page_caps(self, host: HostBatch) -> list[int]:
        """Length to which each cache group's block tables are padded (part of a graph's key).  The capacity of
        the pool, which the tables of a group that sees all keys never outgrow; a windowed group's tables also
        list the pages given back (as -1) and can grow past its pool: then the next power of two, so that a graph
        is recorded anew at doublings only."""
        caps = []
        for g, pg in zip(self.runner.cache.groups, host.table_pages):
            pool = max(g.allocator.num_pages, 1)
            caps.append(pool if pg.shape[0] <= pool else _pow2_at_least(pg.shape[0], pool))
        return caps

    def usable(self, entries) -> bool:
        return (bool(self.sizes) and len(entries) <= self.sizes[-1] and self.runner.model.graph_safe
                and all(e.n_tokens == 1 and list(e.want) == [0] for e in entries) and self._tables_fit(entries))

    def usable_general(self, entries) -> bool:
        """A step with prompt portions that is small enough for a graph of its padded shape: what it costs on
        the host to launch its kernels one by one is then more than the GPU needs for them."""
        if not self.sizes or self.max_tokens <= 0 or not self.runner.model.graph_safe:
            return False
        return (len(entries) <= self.sizes[-1] and sum(e.n_tokens for e in entries) <= min(self.max_tokens, TOKEN_BUCKETS[-1])
                and all(len(e.want) <= 1 for e in entries) and self._tables_fit(entries))

    def prepare_general(self, entries: list[StepEntry], extra: dict[str, np.ndarray]) -> dict | None:
        """``prepare`` for a step with prompt portions: tokens padded to a bucket (padding tokens carry request
        row -1), requests and wanted rows to a batch size, every work list to its bound for that shape.  None if
        a work list is longer than its bound (the step then runs without a graph)."""
        runner = self.runner
        host = build_host_batch(entries, runner.cache)
        T, S, R = host.token_ids.shape[0], len(entries), host.logit_rows.shape[0]
        tp = next(b for b in TOKEN_BUCKETS if b >= T)
        sp = next(s for s in self.sizes if s >= S)
        page_caps = self._page_caps(host)
        planners = runner.model.planners()
        raw = {key: m.plan(host) for key, m in planners.items()}
        caps = {}
        for key, p in raw.items():
            if not hasattr(planners[key], "plan_capacity_general"):
                return None
            c = planners[key].plan_capacity_general(tp, sp, sp, p["counts"])
            n = p["counts"]
            if int(n[0]) > c["items"] or int(n[1]) > c["dec"] or int(n[2]) > c["tiles"] or int(n[3]) > c["row_items"] \
                    or int(n[4]) > c["rows"]:
                return None
            caps[key] = c
        key = ("general", tp, sp, tuple(page_caps),
               tuple(sorted((str(k), tuple(sorted(c.items())), int(raw[k]["counts"][5]), int(raw[k]["counts"][6]),
                             int(raw[k]["counts"][7]))
                            for k, c in caps.items())))
        plans = {k: planners[k].pad_plan(p, caps[k]) for k, p in raw.items()}
        last = [int(ip[-1]) for ip in host.table_indptr]
        padded = HostBatch(
            _pad(host.token_ids, tp), _pad(host.positions, tp), _pad(host.token_seq, tp, -1), _pad(host.seq_slot, sp),
            _pad(host.seq_q_start, sp), _pad(host.seq_q_len, sp), _pad(host.seq_kv_len, sp), _pad(host.logit_rows, sp),
            [_pad(ip, sp + 1, l) for ip, l in zip(host.table_indptr, last)],
            [_pad(pg, cap) for pg, cap in zip(host.table_pages, page_caps)], host.requests)
        ex = dict(temperature=_pad(extra["temperature"], sp), stream_key=_pad(extra["stream_key"], sp),
                  sample_pos=_pad(extra["sample_pos"], sp), row_slot=_pad(extra["row_slot"], sp, -1))
        return dict(key=key, bp=sp, padded=padded, plans=plans, caps=caps, ex=ex,
                    signature=[(e.request, e.start) for e in entries])

    def _padded(self, host: HostBatch, bp: int, page_caps: list[int]) -> HostBatch:
        last = [int(ip[-1]) for ip in host.table_indptr]
        return HostBatch(
            _pad(host.token_ids, bp), _pad(host.positions, bp), _pad(host.token_seq, bp, -1), _pad(host.seq_slot, bp),
            _pad(host.seq_q_start, bp), _pad(host.seq_q_len, bp), _pad(host.seq_kv_len, bp),
            np.arange(bp, dtype=np.int32),
            [_pad(ip, bp + 1, l) for ip, l in zip(host.table_indptr, last)],
            [_pad(pg, cap) for pg, cap in zip(host.table_pages, page_caps)], host.requests)

    def prepare(self, entries: list[StepEntry], extra: dict[str, np.ndarray]) -> dict:
        """All host work of a step that needs no result of the step before it: the batch arrays padded to
        the graph's sizes, the work plans, the sampling arrays.  The engine calls this for the NEXT step
        while the GPU is still busy with the current one."""
        runner = self.runner
        B = len(entries)
        bp = next(s for s in self.sizes if s >= B)
        host = build_host_batch(entries, runner.cache)
        page_caps = self._page_caps(host)
        planners = runner.model.planners()
        raw = {key: m.plan(host) for key, m in planners.items()}
        caps = {}
        for key, p in raw.items():
            bound = planners[key].plan_capacity(bp) if hasattr(planners[key], "plan_capacity") else None
            items = int(p["counts"][0])
            # the planner's own bound for this batch size; a plan beyond it (there should be none) gets a graph of its own
            cap = bound["items"] if bound is not None and items <= bound["items"] else _pow2_at_least(items, 8)
            caps[key] = dict(items=cap, dec=bp, tiles=0)
        # the kernels a graph holds are chosen at recording: whatever of a plan decides between variants is in the key
        key = (bp, tuple(page_caps), tuple(sorted((str(k), c["items"], int(raw[k]["counts"][5])) for k, c in caps.items())))
        plans = {k: planners[k].pad_plan(p, caps[k]) for k, p in raw.items()}
        ex = dict(temperature=_pad(extra["temperature"], bp), stream_key=_pad(extra["stream_key"], bp),
                  sample_pos=_pad(extra["sample_pos"], bp), row_slot=_pad(extra["row_slot"], bp, -1))
        return dict(key=key, bp=bp, padded=self._padded(host, bp, page_caps), plans=plans, caps=caps, ex=ex,
                    signature=[(e.request, e.start) for e in entries])

    def launch(self, prep: dict) -> int:
        """Copy a prepared step to the device and replay (or first record) its graph; returns the padded
        batch size (the sampler's results for the real rows are the first rows of each part)."""
        from tokasaurus_b200.kernels import ops

        runner = self.runner
        slot = self.graphs.get(prep["key"])
        if slot is None:
            slot = dict(stager=Stager(runner.rt.device, 1 << 12, self.host_buffers), graph=None)
            slot["stager"].status = runner.stager.status
            self.graphs[prep["key"]] = slot
        ctx = StepContext(prep["padded"], runner.cache, runner.rt.device, slot["stager"], prep["ex"], prep["plans"])
        ctx.plan_caps = prep["caps"]
        runner.last_upload_bytes = slot["stager"].bytes_last_upload
        runner.last_context = ctx
        if slot["graph"] is None:
            self._record(slot, ctx, prep["bp"])
        slot["graph"].replay()
        ops.LAUNCHES += slot["launches"]
        return prep["bp"]

    def run(self, entries: list[StepEntry], extra: dict[str, np.ndarray]) -> int:
        """Prepare and launch one decode step for ``entries``, sampling included."""
        return self.launch(self.prepare(entries, extra))

    def _record(self, slot: dict, ctx: StepContext, bp: int) -> None:
        from tokasaurus_b200.kernels import ops

        runner, sampler = self.runner, self.sampler
        if bp > sampler.max_rows:
            raise ValueError(f"graph batch {bp} exceeds the sampler's {sampler.max_rows} rows")
        last = runner.cache.last_token

        def body():
            logits = runner.model.forward(ctx)
            e = ctx.extra
            sampler.sample(logits, e["temperature"], e["stream_key"], e["sample_pos"], e["row_slot"], last)
            return logits

        # One eager run first (library handles, kernel modules); it must not move the requests on,
        # so the last-token table is put back afterwards.  Writes to the cache are the same ones the
        # replay makes again.
        saved = last.clone()
        torch.cuda.synchronize()
        body()
        last.copy_(saved)
        torch.cuda.synchronize()
        before = ops.LAUNCHES
        g = torch.cuda.CUDAGraph()
        if self.pool is None:
            self.pool = torch.cuda.graph_pool_handle()
        with torch.cuda.graph(g, pool=self.pool):
            slot["logits"] = body()
        slot["launches"] = ops.LAUNCHES - before
        ops.LAUNCHES = before
        slot["graph"] = g
        slot["ctx"] = ctx  # keeps the views alive
