"""Arrangement of a mixer and a feed-forward in one block: pre-norm with residual sums,
``x = x + mixer(norm1(x)); x = x + ffn(norm2(x))`` (tokasaurus/model/llama.py:342-359 with the
norms at :230 and :325 and the sums at :284 and :336).  The sums are carried in the float32
residual stream and are folded into the norm kernel that follows them."""

from __future__ import annotations

import torch

from tokasaurus_b200.kernels import ops
from tokasaurus_b200.parts.base import FeedForward, Mixer, Norm, Part, ResidualStream


class PreNormBlock(Part):
    def __init__(self, mixer_norm: Norm, mixer: Mixer, ffn_norm: Norm, ffn: FeedForward):
        self.mixer_norm = mixer_norm
        self.mixer = mixer
        self.ffn_norm = ffn_norm
        self.ffn = ffn

    def parts(self):
        return (self.mixer_norm, self.mixer, self.ffn_norm, self.ffn)

    def weight_specs(self):
        return tuple(s for p in self.parts() for s in p.weight_specs())

    def bind(self, weights, rt) -> None:
        for p in self.parts():
            p.bind(weights, rt)

    def forward(self, ctx, stream: ResidualStream, cache, out_rows=None) -> ResidualStream:
        """``out_rows`` (int32 device tensor or None): only these rows are needed after the mixer
        (the last block of a step: tokasaurus/model/llama.py:273-278); the stream that comes back
        then has len(out_rows) rows."""
        h = self.mixer_norm.forward(ctx, stream)
        if out_rows is not None:
            x = torch.empty((out_rows.numel(), stream.x.shape[1]), dtype=stream.x.dtype, device=stream.x.device)
            ops.gather_rows(stream.x, out_rows, x)
            stream = ResidualStream(x)
        stream.delta = self.mixer.forward(ctx, h, cache, out_rows)
        h = self.ffn_norm.forward(ctx, stream)
        stream.delta = self.ffn.forward(ctx, h)
        return stream
