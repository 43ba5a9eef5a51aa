"""Grouped-query attention over the paged cache.

Follows tokasaurus/model/llama.py:218-287: q, k, v projections without bias (:235-237), views by
head (:239-241), rotary encoding of q and k (:243-256), append of k and v to the cache and
causal attention over it with scale 1/sqrt(head_dim) (tokasaurus/model/attention_utils.py:108-175),
restriction to the wanted rows (llama.py:273-278), output projection (:280).  The three
projection matrices are stacked into one so that one matrix product makes q|k|v.
"""

from __future__ import annotations

import torch

from tokasaurus_b200.kernels import ops
from tokasaurus_b200.parts.base import Mixer, PagedCacheNeed, PositionEncoding, WeightSpec


class PagedAttention(Mixer):
    def __init__(self, width: int, n_heads: int, n_kv_heads: int, head_dim: int, position: PositionEncoding,
                 q_name: str, k_name: str, v_name: str, o_name: str, window: int | None = None,
                 softmax_scale: float | None = None):
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
        self.w_qkv: torch.Tensor | None = None
        self.w_o: torch.Tensor | None = None
        self.inv_freq: torch.Tensor | None = None

    # --- declarations ---
    def weight_specs(self):
        q, k, v, o = self.names
        hd = self.head_dim
        return (
            WeightSpec(q, (self.n_heads * hd, self.width)),
            WeightSpec(k, (self.n_kv_heads * hd, self.width)),
            WeightSpec(v, (self.n_kv_heads * hd, self.width)),
            WeightSpec(o, (self.width, self.n_heads * hd)),
        )

    def cache_need(self):
        return PagedCacheNeed(self.n_kv_heads, self.head_dim, self.window)

    def bind(self, weights, rt) -> None:
        q, k, v, o = self.names
        self.w_qkv = torch.cat([weights[q], weights[k], weights[v]], dim=0).contiguous()
        self.w_o = weights[o].contiguous()
        inv = self.position.inv_freq() if self.position.kind == "rotary" else None
        self.inv_freq = inv.to(rt.device) if inv is not None else None

    # --- one step ---
    def forward(self, ctx, h: torch.Tensor, cache, out_rows=None) -> torch.Tensor:
        T = h.shape[0]
        hd, nh, nkv = self.head_dim, self.n_heads, self.n_kv_heads
        qkv = ops.linear(h, self.w_qkv)
        tables = ctx.tables[cache.group]
        rot = self.position.rotary_dim if self.position.kind == "rotary" else 0
        ops.rope_kv_write(qkv, ctx.positions, ctx.token_seq, tables.indptr, tables.page_ids, self.inv_freq,
                          cache.k, cache.v, nh, nkv, hd, rot, cache.page_size, cache.writable, ctx.status)
        n_rows = T if out_rows is None else out_rows.numel()
        attn = torch.empty((n_rows, nh * hd), dtype=h.dtype, device=h.device)
        ops.attn_paged(qkv, qkv.shape[1], attn, cache.k, cache.v, ctx.token_seq, ctx.positions, tables.indptr,
                       tables.page_ids, out_rows, n_rows, nh, nkv, hd, cache.page_size, self.scale, self.window)
        return ops.linear(attn, self.w_o)
