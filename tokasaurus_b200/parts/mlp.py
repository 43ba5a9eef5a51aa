"""SiLU-gated feed-forward: ``down(silu(gate(h)) * up(h))`` without biases
(tokasaurus/model/llama.py:319-339; :329-332 are the three products and the activation).  The
gate and up matrices are stacked so that one matrix product makes gate|up."""

from __future__ import annotations

import torch

from tokasaurus_b200.kernels import ops
from tokasaurus_b200.parts.base import FeedForward, WeightSpec


class GatedMLP(FeedForward):
    def __init__(self, width: int, inner: int, gate_name: str, up_name: str, down_name: str):
        self.width = width
        self.inner = inner
        self.names = (gate_name, up_name, down_name)
        self.interleave = 0
        self.w_gate_up: torch.Tensor | None = None
        self.w_down: torch.Tensor | None = None

    def weight_specs(self):
        g, u, d = self.names
        return (
            WeightSpec(g, (self.inner, self.width)),
            WeightSpec(u, (self.inner, self.width)),
            WeightSpec(d, (self.width, self.inner)),
        )

    def bind(self, weights, rt) -> None:
        g, u, d = self.names
        # bfloat16: gate and up rows interleaved in groups of 8, the layout whose product the small-batch
        # kernel can turn into silu(gate) * up in its epilogue
        self.interleave = 8 if (rt.dtype == torch.bfloat16 and self.inner % 8 == 0) else 0
        if self.interleave:
            self.w_gate_up = ops.interleave_gate_up(weights[g], weights[u])
        else:
            self.w_gate_up = torch.cat([weights[g], weights[u]], dim=0).contiguous()
        self.w_down = weights[d].contiguous()

    def forward(self, ctx, h):
        """Returns the update [rows, width] in h's dtype, or as float32 slices [slices, rows, width]
        that the next norm adds (few rows, bfloat16)."""
        status = ctx.status if ctx is not None else None
        if self.interleave and ops.can_use_few_rows(h, self.w_gate_up) and self.w_gate_up.shape[0] % 16 == 0:
            act = ops.linear_few_rows_gated(h, self.w_gate_up, status)
            return ops.linear_few_rows(act, self.w_down, status)
        if self.interleave and h.shape[0] >= ops.TCGEN05_M_MIN and ops.can_use_tcgen05(h, self.w_gate_up):
            # many rows: the tcgen05 product with the SiLU gate in its epilogue (no activation pass over memory)
            act = ops.gemm_tcgen05(h, self.w_gate_up,
                                   status if status is not None else torch.zeros(1, dtype=torch.int32, device=h.device),
                                   gated=True)
        else:
            gu = ops.linear(h, self.w_gate_up)
            act = torch.empty((h.shape[0], self.inner), dtype=h.dtype, device=h.device)
            ops.silu_mul(gu, act, self.interleave)
        if ops.can_use_few_rows(act, self.w_down):
            return ops.linear_few_rows(act, self.w_down, status)
        return ops.linear(act, self.w_down)
