"""Rotary position encoding: the per-pair inverse frequencies, plain or llama3-scaled.

The reference takes its cos/sin tables from ``LlamaRotaryEmbedding`` for every position up to
max_position_embeddings and keeps them in float32 (tokasaurus/model/llama.py:559-570), then
gathers rows by position (llama.py:576-578) and applies ``apply_rotary_pos_emb`` (llama.py:243-256).
Those tables equal ``cos(pos * inv_freq)``, ``sin(pos * inv_freq)`` with the inverse frequencies
below, so this engine keeps only ``inv_freq`` (head_dim/2 floats) and forms the angle in the
kernel, in float32, as the same product.

    inv_freq_j = theta ** (-2j / rotary_dim),  j in [0, rotary_dim/2)
    llama3:  wavelen = 2*pi / inv_freq
             wavelen > orig/low_freq_factor   ->  inv_freq / factor
             wavelen < orig/high_freq_factor  ->  inv_freq
             otherwise  smooth = (orig/wavelen - low) / (high - low);
                        (1 - smooth) * inv_freq / factor + smooth * inv_freq
"""

from __future__ import annotations

import math

import torch

from tokasaurus_b200.parts.base import PositionEncoding


class NoPositionEncoding(PositionEncoding):
    kind = "none"
    rotary_dim = 0

    def inv_freq(self) -> None:
        return None


class RotaryEncoding(PositionEncoding):
    kind = "rotary"

    def __init__(self, rotary_dim: int, theta: float, scaling_type: str = "default", factor: float = 1.0,
                 low_freq_factor: float = 1.0, high_freq_factor: float = 4.0,
                 original_max_position_embeddings: int = 8192):
        if rotary_dim <= 0 or rotary_dim % 2:
            raise ValueError(f"rotary_dim must be a positive even number, got {rotary_dim}")
        if scaling_type not in ("default", "llama3"):
            raise ValueError(f"unknown rotary scaling {scaling_type!r}")
        self.rotary_dim = rotary_dim
        self.theta = float(theta)
        self.scaling_type = scaling_type
        self.factor = float(factor)
        self.low_freq_factor = float(low_freq_factor)
        self.high_freq_factor = float(high_freq_factor)
        self.original_max_position_embeddings = int(original_max_position_embeddings)

    def inv_freq(self) -> torch.Tensor:
        """float32 [rotary_dim / 2], on the CPU."""
        d = self.rotary_dim
        inv = 1.0 / (self.theta ** (torch.arange(0, d, 2, dtype=torch.int64).to(torch.float32) / d))
        if self.scaling_type == "default":
            return inv
        orig = self.original_max_position_embeddings
        low_wavelen = orig / self.low_freq_factor
        high_wavelen = orig / self.high_freq_factor
        wavelen = 2 * math.pi / inv
        scaled = torch.where(wavelen > low_wavelen, inv / self.factor, inv)
        smooth = (orig / wavelen - self.low_freq_factor) / (self.high_freq_factor - self.low_freq_factor)
        mid = (1 - smooth) * scaled / self.factor + smooth * scaled
        is_mid = ~(wavelen < high_wavelen) & ~(wavelen > low_wavelen)
        return torch.where(is_mid, mid, scaled).to(torch.float32)
