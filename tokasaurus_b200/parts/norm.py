"""RMS norm: ``y = weight * x / sqrt(mean(x^2) + eps)`` with the statistics in float32
(tokasaurus/model/llama.py:44-51).  The kernel also folds in the residual add that precedes the
norm (llama.py:284 and :336 add, the next block's :230 / :325 normalises)."""

from __future__ import annotations

import torch

from tokasaurus_b200.kernels import ops
from tokasaurus_b200.parts.base import Norm, ResidualStream, WeightSpec


class RMSNorm(Norm):
    def __init__(self, width: int, eps: float, weight_name: str):
        self.width = width
        self.eps = float(eps)
        self.weight_name = weight_name
        self.weight: torch.Tensor | None = None
        self.out_dtype: torch.dtype | None = None

    def weight_specs(self):
        return (WeightSpec(self.weight_name, (self.width,), role="vector"),)

    def bind(self, weights, rt) -> None:
        self.weight = weights[self.weight_name]
        self.out_dtype = rt.dtype

    def _run(self, x: torch.Tensor, delta=None) -> torch.Tensor:
        out = torch.empty(x.shape, dtype=self.out_dtype, device=x.device)
        ops.add_rmsnorm(x, delta, self.weight, self.eps, out)
        return out

    def forward(self, ctx, stream: ResidualStream):
        out = self._run(stream.x, stream.delta)
        stream.delta = None
        return out
