"""Grouped-query attention over the paged cache.

Follows tokasaurus/model/llama.py:218-287: q, k, v projections without bias (:235-237), views by
head (:239-241), rotary encoding of q and k (:243-256), append of k and v to the cache and
causal attention over it with scale 1/sqrt(head_dim) (tokasaurus/model/attention_utils.py:108-175),
restriction to the wanted rows (llama.py:273-278), output projection (:280).  The three
projection matrices are stacked into one so that one matrix product makes q|k|v.

When every request of a step has a single split (short contexts) the split-key kernel writes the final
result itself; otherwise a second small kernel merges the splits (measured faster on B200 than letting the
last block of each request merge them inside the attention kernel, which the kernel can also do).

Kernels: in float32 one FP32 kernel serves every token.  In bfloat16 the requests of a step are
split as the reference splits them into a prefill and a decode call
(attention_utils.py:129-151): requests that bring one token go to the split-key tensor-core
kernel, longer portions to the tiled tensor-core kernel; the host plans the work items of both
(the reference's ``plan`` calls, llama.py:698-764).
"""

from __future__ import annotations

import numpy as np
import torch

from tokasaurus_b200.kernels import ops
from tokasaurus_b200.parts.base import Mixer, PagedCacheNeed, PositionEncoding, QkvStage, WeightSpec

MIN_SPLIT_KEYS = 128  # no work item of the split-key kernel is cut finer than this
QUERY_TILE = 64  # queries per block of the tiled mma.sync kernel
QUERY_TILE_TC = 128  # queries per block of the tcgen05 kernel
def decode_block_slots(head_dim: int, limits=None) -> int:
    """Blocks of the split-key kernel that the GPU holds at once: what of an SM's shared memory the kernel's
    stages take (two tiles of 64 rows a stage, rows of head_dim * 2 bytes, padded by 16 where the head size is
    no multiple of 64; three stages, two when three pass 110 KiB), at most four blocks an SM (128 threads of up to
    124 registers each).  ``limits``: the
    device's SM count and shared memory (``kernels.device.DeviceLimits``; None: planning without a device)."""
    if limits is None:
        from tokasaurus_b200.kernels.device import NO_DEVICE as limits
    stage = 2 * 64 * (head_dim * 2 + (0 if head_dim % 64 == 0 else 16))
    stages = 3 if 3 * stage <= 110 * 1024 else 2
    return limits.sm_count * max(1, min(4, limits.shared_memory_per_sm // (stages * stage + 2048)))


DECODE_BLOCK_SLOTS = decode_block_slots(64)  # the default of the planning functions below


def split_keys_evenly(span: np.ndarray, blocks_per_item: int, slots: int = DECODE_BLOCK_SLOTS
                      ) -> tuple[np.ndarray, np.ndarray]:
    """How many work items each single-token request gets and how many keys each item holds (a multiple of
    64, the kernel's tile): requests are cut evenly, in proportion to their keys, so that the step's items fill
    one wave of blocks.  A request shorter than an item's share stays whole (such items may take the count over
    the wave; they are short).  Measured on B200 (8 kv heads, contexts of 2,048): a wave that is at least 0.7
    full beats any finer cut into a second wave (batches 8 and 16: 0.86 of a wave), but a wave less than 0.7
    full loses to 1.15 waves of items half the size (batch 32), and requests that cannot be cut to fit
    (batch 64: 1.15 waves of whole requests) are best left whole."""
    max_items = max(1, slots // max(1, blocks_per_item))
    if span.shape[0] == 0:
        return np.zeros((0,), dtype=np.int64), np.zeros((0,), dtype=np.int64)
    total = int(span.sum())

    def cut(budget: int):
        target = max(MIN_SPLIT_KEYS, -(-total // budget))
        n = np.maximum(1, span // target)
        size = -(-(-(-span // n)) // 64) * 64
        return np.maximum(1, -(-span // size)), size

    n, size = cut(max_items)
    if int(n.sum()) < 0.7 * max_items:
        n2, size2 = cut(max_items + max_items // 4)
        if int(n2.sum()) > int(n.sum()):
            return n2, size2
    return n, size


def plan_attention(host, window: int | None, capacity: dict | None = None, blocks_per_item: int = 8,
                   query_tile: int = QUERY_TILE, slots: int = DECODE_BLOCK_SLOTS,
                   head_blocks: int = 0) -> dict[str, np.ndarray]:
    """Work items for one step: (request row, first key, keys) triples for requests with one token,
    (request row, first query) pairs for ``query_tile``-query tiles of longer portions.  ``blocks_per_item``:
    blocks the split-key kernel launches per item (kv heads x head tiles).  ``head_blocks``: how many query tiles
    a step may have for the portions' kernel to give every query head a block of its own (0: never)."""
    q_len = np.asarray(host.seq_q_len, dtype=np.int64)
    kv_len = np.asarray(host.seq_kv_len, dtype=np.int64)
    dec_seqs = np.nonzero(q_len == 1)[0]
    span = kv_len[dec_seqs]
    if window:
        span = np.minimum(span, window)
    n_splits, split_size = split_keys_evenly(span, blocks_per_item, slots)
    dec_start = np.concatenate([[0], np.cumsum(n_splits)])
    n_items = int(dec_start[-1])
    item_seq = np.repeat(dec_seqs, n_splits)
    item_size = np.repeat(split_size, n_splits)
    item_first = (np.arange(n_items) - np.repeat(dec_start[:-1], n_splits)) * item_size
    items = np.stack([item_seq, item_first, item_size], axis=1).reshape(-1)
    item_entry = np.repeat(np.arange(dec_seqs.shape[0]), n_splits)  # index of each item's request in dec_seqs
    pre_seqs = np.nonzero(q_len > 1)[0]
    n_tiles_seq = -(-q_len[pre_seqs] // query_tile)
    tile_start = np.concatenate([[0], np.cumsum(n_tiles_seq)])
    n_tiles = int(tile_start[-1])
    tile_seq = np.repeat(pre_seqs, n_tiles_seq)
    tile_q0 = (np.arange(n_tiles) - np.repeat(tile_start[:-1], n_tiles_seq)) * query_tile
    # tiles that see the most keys first: the long ones must not be left for the end of the launch
    reach = kv_len[tile_seq] - q_len[tile_seq] + tile_q0
    order = np.argsort(-reach, kind="stable")
    tiles = np.stack([tile_seq[order], tile_q0[order]], axis=1).reshape(-1)
    cap = capacity or {}
    # wanted rows, when they are only some of the step's rows: each is one query over the keys up to its
    # own position, which is what the split-key kernel computes for a request that brings one token
    extra = {}
    n_row_items = n_rows = 0
    rows = getattr(host, "logit_rows", None)
    if rows is not None and capacity is None and 0 < rows.shape[0] and not (
            rows.shape[0] == host.token_ids.shape[0] and np.array_equal(rows, np.arange(rows.shape[0]))):
        rows = np.asarray(rows, dtype=np.int64)
        r_kv = np.asarray(host.positions, dtype=np.int64)[rows] + 1
        r_span = np.minimum(r_kv, window) if window else r_kv
        r_splits, r_size = split_keys_evenly(r_span, blocks_per_item, slots)
        r_start = np.concatenate([[0], np.cumsum(r_splits)])
        n_row_items, n_rows = int(r_start[-1]), int(rows.shape[0])
        r_item = np.repeat(np.arange(n_rows), r_splits)
        r_isize = np.repeat(r_size, r_splits)
        r_first = (np.arange(n_row_items) - np.repeat(r_start[:-1], r_splits)) * r_isize
        i32 = lambda a: np.ascontiguousarray(a, dtype=np.int32)  # noqa: E731
        extra = dict(row_items=i32(np.stack([r_item, r_first, r_isize], axis=1).reshape(-1)), row_item_start=i32(r_start),
                     row_item_entry=i32(r_item),
                     row_token=i32(rows), row_kv_len=i32(r_kv),
                     row_index=i32(np.arange(n_rows)))
        # where each row's request starts in the page-id list of each cache group (a windowed group's tables can be
        # shorter than those of a group that sees all keys while a prompt is on its way)
        for g, indptr in enumerate(host.table_indptr):
            extra[f"row_indptr_g{g}"] = i32(np.asarray(indptr)[np.asarray(host.token_seq)[rows]])
    # counts[5], counts[6]: some work item of the requests that decode (of the wanted rows) is longer than three
    # tiles of 64 keys; the split-key kernel then runs in the variant that fetches whole tiles by TMA
    long_items = int(n_items > 0 and int(item_size.max()) > 3 * 64)
    long_row_items = int(n_row_items > 0 and int(r_isize.max()) > 3 * 64)
    # counts[7]: so few query tiles that blocks of two heads would leave SMs idle: one head a block
    few_tiles = int(0 < n_tiles <= head_blocks)
    counts = np.asarray([n_items, dec_seqs.shape[0], n_tiles, n_row_items, n_rows, long_items, long_row_items,
                         few_tiles], dtype=np.int32)

    def padded(x, n):
        a = np.zeros(max(n, x.shape[0], 1), dtype=np.int32)
        a[: x.shape[0]] = x
        return a

    return dict(counts=counts, items=padded(items, 3 * cap.get("items", 0)),
                item_entry=padded(item_entry, cap.get("items", 0)),
                dec_seqs=padded(dec_seqs, cap.get("dec", 0)), dec_item_start=padded(dec_start, cap.get("dec", 0) + 1),
                tiles=padded(tiles, 2 * cap.get("tiles", 0)), **extra)


class PagedAttention(Mixer):
    graph_safe = True

    def __init__(self, width: int, n_heads: int, n_kv_heads: int, head_dim: int, position: PositionEncoding,
                 q_name: str, k_name: str, v_name: str, o_name: str, window: int | None = None,
                 softmax_scale: float | None = None, qkv_stage: QkvStage | None = None):
        """``qkv_stage``: an element-wise stage between the projections and the position encoding (biases, per-head
        norms; ``parts.base.QkvStage``).  Llama has none."""
        if n_heads % n_kv_heads:
            raise ValueError(f"n_heads={n_heads} is not a multiple of n_kv_heads={n_kv_heads}")
        ops.check_head_dim(head_dim)
        self.width = width
        self.n_heads = n_heads
        self.n_kv_heads = n_kv_heads
        self.head_dim = head_dim
        self.position = position
        self.window = window
        self.scale = float(softmax_scale) if softmax_scale is not None else ops.softmax_scale(head_dim)
        self.names = (q_name, k_name, v_name, o_name)
        self.qkv_stage = qkv_stage
        self.qkv_bias: torch.Tensor | None = None   # float32 [(heads + 2 kv heads) * head_dim]
        self.qk_norm: torch.Tensor | None = None    # float32 [2, head_dim]
        self.norm_eps = float(qkv_stage.norm_eps) if qkv_stage is not None else 0.0
        self.w_qkv: torch.Tensor | None = None
        self.w_o: torch.Tensor | None = None
        self.inv_freq: torch.Tensor | None = None
        self.dtype: torch.dtype | None = None
        self.block_slots = decode_block_slots(head_dim)  # bind() asks the device
        self.sm_count = 0

    # --- declarations ---
    def weight_specs(self):
        q, k, v, o = self.names
        hd = self.head_dim
        specs = [
            WeightSpec(q, (self.n_heads * hd, self.width)),
            WeightSpec(k, (self.n_kv_heads * hd, self.width)),
            WeightSpec(v, (self.n_kv_heads * hd, self.width)),
            WeightSpec(o, (self.width, self.n_heads * hd)),
        ]
        st = self.qkv_stage
        if st is not None and st.bias_names is not None:
            for name, heads in zip(st.bias_names, (self.n_heads, self.n_kv_heads, self.n_kv_heads)):
                specs.append(WeightSpec(name, (heads * hd,), role="vector"))
        if st is not None and st.qk_norm_names is not None:
            specs += [WeightSpec(name, (hd,), role="vector") for name in st.qk_norm_names]
        return tuple(specs)

    def cache_need(self):
        return PagedCacheNeed(self.n_kv_heads, self.head_dim, self.window)

    def bind(self, weights, rt) -> None:
        q, k, v, o = self.names
        self.w_qkv = torch.cat([weights[q], weights[k], weights[v]], dim=0).contiguous()
        self.w_o = weights[o].contiguous()
        st = self.qkv_stage
        if st is not None and st.bias_names is not None:
            self.qkv_bias = torch.cat([weights[n].float() for n in st.bias_names]).contiguous()
        if st is not None and st.qk_norm_names is not None:
            self.qk_norm = torch.stack([weights[n].float() for n in st.qk_norm_names]).contiguous()
        inv = self.position.inv_freq() if self.position.kind == "rotary" else None
        self.inv_freq = inv.to(rt.device) if inv is not None else None
        self.dtype = rt.dtype
        self.block_slots = decode_block_slots(self.head_dim, getattr(rt, "limits", None))
        from tokasaurus_b200.kernels.device import NO_DEVICE

        self.sm_count = (getattr(rt, "limits", None) or NO_DEVICE).sm_count

    def plan_key(self):
        if self.dtype != torch.bfloat16:
            return None
        return ("paged_attention", self.window, self._blocks_per_item(), self._query_tile(), self.head_dim)

    def _query_tile(self) -> int:
        return QUERY_TILE_TC if ops.can_use_attn_prefill_tc(self.head_dim) else QUERY_TILE

    def _blocks_per_item(self) -> int:
        return self.n_kv_heads * ((self.n_heads // self.n_kv_heads + 15) // 16)

    def plan(self, host, capacity=None):
        return plan_attention(host, self.window, capacity, self._blocks_per_item(), self._query_tile(),
                              self.block_slots, self.sm_count // self.n_heads)

    def plan_capacity(self, n_requests: int) -> dict:
        """The most work items ``plan`` can make for a step of ``n_requests`` single-token requests, whatever
        their contexts: each request gets at most (its keys // the item size) items, at least one."""
        wave = max(1, self.block_slots // max(1, self._blocks_per_item()))
        return dict(items=n_requests + wave + wave // 4 + 1, dec=n_requests, tiles=0)

    def plan_capacity_general(self, n_tokens: int, n_requests: int, n_rows: int, counts) -> dict:
        """Capacities of every work list for a step of up to ``n_tokens`` tokens in ``n_requests`` requests with
        ``n_rows`` wanted rows; a list the step does not use at all (``counts`` are the plan's own) gets 0, so that
        its kernel is not launched."""
        wave = max(1, self.block_slots // max(1, self._blocks_per_item()))
        spare = wave + wave // 4 + 1
        has_dec, has_tiles, has_rows = int(counts[1]) > 0, int(counts[2]) > 0, int(counts[4]) > 0
        return dict(items=(n_requests + spare) if has_dec else 0, dec=n_requests if has_dec else 0,
                    tiles=(n_tokens // self._query_tile() + n_requests) if has_tiles else 0,
                    row_items=(n_rows + spare) if has_rows else 0, rows=n_rows if has_rows else 0)

    def pad_plan(self, plan: dict, capacity: dict) -> dict:
        """The same plan with its arrays at the fixed sizes of a CUDA graph."""
        def padded(x, n):
            a = np.zeros(max(n, x.shape[0], 1), dtype=np.int32)
            a[: x.shape[0]] = x
            return a

        out = dict(plan)
        out["items"] = padded(plan["items"], 3 * capacity.get("items", 0))
        out["item_entry"] = padded(plan["item_entry"], capacity.get("items", 0))
        out["dec_seqs"] = padded(plan["dec_seqs"], capacity.get("dec", 0))
        out["dec_item_start"] = padded(plan["dec_item_start"], capacity.get("dec", 0) + 1)
        out["tiles"] = padded(plan["tiles"], 2 * capacity.get("tiles", 0))
        if "row_items" in plan:
            ri, rows = capacity.get("row_items", 0), capacity.get("rows", 0)
            out["row_items"] = padded(plan["row_items"], 3 * ri)
            out["row_item_entry"] = padded(plan["row_item_entry"], ri)
            out["row_item_start"] = padded(plan["row_item_start"], rows + 1)
            for name in plan:
                if name in ("row_token", "row_kv_len", "row_index") or name.startswith("row_indptr_g"):
                    out[name] = padded(plan[name], rows)
        return out

    # --- one step ---
    def forward(self, ctx, h, cache, out_rows=None):
        T = h.shape[0]
        hd, nh, nkv = self.head_dim, self.n_heads, self.n_kv_heads
        tables = ctx.tables[cache.group]
        rot = self.position.rotary_dim if self.position.kind == "rotary" else 0
        small = (ops.can_use_few_rows(h, self.w_qkv, ops.ATTN_FEW_ROWS_MAX) and (nh * hd) % 8 == 0
                 and (self.w_qkv.shape[0] + max(rot, 2)) * 4 <= 160 * 1024)
        few = lambda a, w: ops.linear_few_rows(a, w, ctx.status)  # noqa: E731
        if small:
            # few rows: K-split products whose float32 slices the next kernel adds
            parts = few(h, self.w_qkv)
            plan = ctx.plans.get(self.plan_key())
            counts = ctx.host_plans[self.plan_key()]["counts"] if plan is not None else None
            if plan is not None and out_rows is None and int(counts[2]) == 0 and int(counts[1]) > 0 and rot % 4 == 0:
                # every request brings one token: the attention kernel adds the slices, rotates, writes the cache
                attn = torch.empty((T, nh * hd), dtype=h.dtype, device=h.device)
                caps = ctx.plan_caps.get(self.plan_key()) if ctx.plan_caps else None
                c = plan["counts"]
                ops.attn_decode_rope_mma(parts, cache.k, cache.v, ctx.seq_q_start, ctx.seq_kv_len, tables.indptr,
                                         tables.page_ids, plan["items"], c[0:1], caps["items"] if caps else int(counts[0]),
                                         plan["dec_seqs"], plan["dec_item_start"], c[1:2],
                                         caps["dec"] if caps else int(counts[1]), attn, nh, nkv, hd, cache.page_size,
                                         self.scale, self.window, self.inv_freq, rot, cache.writable,
                                         ctx.status, item_entry=plan["item_entry"], tma=bool(counts[5]),
                                         bias=self.qkv_bias, qk_norm=self.qk_norm, norm_eps=self.norm_eps)
                return few(attn, self.w_o)
            qkv = torch.empty((T, nh * hd), dtype=h.dtype, device=h.device)  # q only; k and v go straight to the cache
            ops.rope_kv_write_partials(parts, qkv, ctx.positions, ctx.token_seq, tables.indptr, tables.page_ids,
                                       self.inv_freq, cache.k, cache.v, nh, nkv, hd, rot, cache.page_size,
                                       cache.writable, ctx.status, bias=self.qkv_bias, qk_norm=self.qk_norm, norm_eps=self.norm_eps)
            project = few
        else:
            qkv = ops.linear(h, self.w_qkv)
            ops.rope_kv_write(qkv, ctx.positions, ctx.token_seq, tables.indptr, tables.page_ids, self.inv_freq,
                              cache.k, cache.v, nh, nkv, hd, rot, cache.page_size, cache.writable, ctx.status,
                              bias=self.qkv_bias, qk_norm=self.qk_norm, norm_eps=self.norm_eps)
            project = ops.linear
        plan = ctx.plans.get(self.plan_key()) if h.dtype == torch.bfloat16 else None
        if plan is not None and out_rows is not None and out_rows is ctx.logit_rows and "row_items" in plan:
            # only some rows are wanted (the last block of a step): one split-key query per wanted row
            counts = ctx.host_plans[self.plan_key()]["counts"]
            caps = ctx.plan_caps.get(self.plan_key()) if ctx.plan_caps else None
            n_items = caps["row_items"] if caps else int(counts[3])
            n_rows = caps["rows"] if caps else int(counts[4])
            attn = torch.empty((n_rows, nh * hd), dtype=h.dtype, device=h.device)
            c = plan["counts"]
            ops.attn_decode_mma(qkv, cache.k, cache.v, plan["row_token"], plan["row_kv_len"],
                                plan[f"row_indptr_g{cache.group}"],
                                tables.page_ids, plan["row_items"], c[3:4], n_items, plan["row_index"],
                                plan["row_item_start"], c[4:5], n_rows, attn, nh, nkv, hd, cache.page_size,
                                self.scale, self.window, out_row_of=plan["row_index"],
                                item_entry=plan["row_item_entry"], tma=bool(counts[6]), status=ctx.status)
            return project(attn, self.w_o)
        if plan is None or out_rows is not None:
            # float32, or only some rows are wanted: the FP32-pipe kernel, one warp per (row, head)
            n_rows = T if out_rows is None else out_rows.numel()
            attn = torch.empty((n_rows, nh * hd), dtype=h.dtype, device=h.device)
            ops.attn_paged(qkv, qkv.shape[1], attn, cache.k, cache.v, ctx.token_seq, ctx.positions, tables.indptr,
                           tables.page_ids, out_rows, n_rows, nh, nkv, hd, cache.page_size, self.scale, self.window,
                           ctx.status)
            return project(attn, self.w_o)
        attn = torch.empty((T, nh * hd), dtype=h.dtype, device=h.device)
        caps = ctx.plan_caps.get(self.plan_key()) if ctx.plan_caps else None
        counts = ctx.host_plans[self.plan_key()]["counts"]
        items_cap = caps["items"] if caps else int(counts[0])
        dec_cap = caps["dec"] if caps else int(counts[1])
        tiles_cap = caps["tiles"] if caps else int(counts[2])
        c = plan["counts"]
        if dec_cap:
            ops.attn_decode_mma(qkv, cache.k, cache.v, ctx.seq_q_start, ctx.seq_kv_len, tables.indptr, tables.page_ids,
                                plan["items"], c[0:1], items_cap, plan["dec_seqs"], plan["dec_item_start"], c[1:2],
                                dec_cap, attn, nh, nkv, hd, cache.page_size, self.scale, self.window,
                                item_entry=plan["item_entry"], tma=bool(counts[5]), status=ctx.status)
        if tiles_cap and self._query_tile() == QUERY_TILE_TC:
            ops.attn_prefill_tc(qkv, attn, cache.k, cache.v, ctx.seq_q_start, ctx.seq_q_len, ctx.seq_kv_len,
                                tables.indptr, tables.page_ids, plan["tiles"], c[2:3], tiles_cap, nh, nkv, hd,
                                cache.page_size, self.scale, self.window, ctx.status, single_heads=bool(counts[7]))
        elif tiles_cap:
            ops.attn_prefill_mma(qkv, attn, cache.k, cache.v, ctx.seq_q_start, ctx.seq_q_len, ctx.seq_kv_len,
                                 tables.indptr, tables.page_ids, plan["tiles"], c[2:3], tiles_cap, nh, nkv, hd,
                                 cache.page_size, self.scale, self.window, ctx.status)
        return project(attn, self.w_o)
