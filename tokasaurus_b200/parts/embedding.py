"""Token embedding (row gather, tokasaurus/model/llama.py:507-518) and output head (final norm
and vocabulary projection to float32 logits, llama.py:441-467)."""

from __future__ import annotations

import torch

from tokasaurus_b200.kernels import ops
from tokasaurus_b200.parts.base import Norm, Part, ResidualStream, WeightSpec


class TokenEmbedding(Part):
    def __init__(self, vocab: int, width: int, weight_name: str):
        self.vocab = vocab
        self.width = width
        self.weight_name = weight_name
        self.table: torch.Tensor | None = None

    def weight_specs(self):
        return (WeightSpec(self.weight_name, (self.vocab, self.width)),)

    def bind(self, weights, rt) -> None:
        self.table = weights[self.weight_name]

    def forward(self, ctx) -> ResidualStream:
        x = torch.empty((ctx.n_tokens, self.width), dtype=torch.float32, device=self.table.device)
        ops.embed_gather(self.table, ctx.token_ids, ctx.token_seq, ctx.seq_slot, ctx.last_token, x, ctx.status)
        return ResidualStream(x)


class OutputHead(Part):
    """``weight_name`` may be the embedding's tensor (tied weights): the loader hands the same
    storage to both parts."""

    def __init__(self, vocab: int, width: int, norm: Norm, weight_name: str):
        self.vocab = vocab
        self.width = width
        self.norm = norm
        self.weight_name = weight_name
        self.weight: torch.Tensor | None = None

    def weight_specs(self):
        return tuple(self.norm.weight_specs()) + (WeightSpec(self.weight_name, (self.vocab, self.width)),)

    def bind(self, weights, rt) -> None:
        self.norm.bind(weights, rt)
        self.weight = weights[self.weight_name]

    def forward(self, ctx, stream: ResidualStream) -> torch.Tensor:
        h = self.norm.forward(ctx, stream)
        return ops.linear(h, self.weight, out_dtype=torch.float32)
