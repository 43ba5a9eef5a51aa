"""A decoder as data: embedding, blocks, the order in which the blocks run, head.

``run_order`` is a list of ``LayerCall``.  Each call names the block to run and the cache entry
it uses; by default call i runs block i on cache entry i (tokasaurus/model/llama.py:580-581 is
the reference's plain loop over layers).  A block may be named in several calls (shared
weights), and a call may read the cache entry that another call writes (``write_cache=False``).
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Sequence

import torch

from tokasaurus_b200.parts.base import Part, WeightSpec


@dataclass(frozen=True)
class LayerCall:
    block: int
    cache: int | None = None  # cache entry; None: an entry of this call's own
    write_cache: bool = True


class DecoderModel(Part):
    def __init__(self, embedding, blocks: Sequence, head, run_order: Sequence[LayerCall] | None = None,
                 ignored_weight_patterns: Sequence[str] = ()):
        """``ignored_weight_patterns``: names (shell patterns) of tensors that checkpoints of this architecture may
        carry although no part reads them; the loader passes over them with a warning instead of refusing the
        folder, as it does for any other tensor nobody asked for."""
        self.ignored_weight_patterns = tuple(ignored_weight_patterns)
        self.embedding = embedding
        self.blocks = list(blocks)
        self.head = head
        order = list(run_order) if run_order is not None else [LayerCall(i) for i in range(len(self.blocks))]
        # give every call without an explicit cache entry one of its own
        used = {c.cache for c in order if c.cache is not None}
        fresh = (i for i in range(len(order) + len(used) + 1) if i not in used)
        self.run_order = [c if c.cache is not None else LayerCall(c.block, next(fresh), c.write_cache) for c in order]
        for c in self.run_order:
            if not 0 <= c.block < len(self.blocks):
                raise ValueError(f"run order names block {c.block}, but there are {len(self.blocks)} blocks")
        writers = {c.cache for c in self.run_order if c.write_cache}
        for c in self.run_order:
            if not c.write_cache and c.cache not in writers:
                raise ValueError(f"a layer call reads cache entry {c.cache} that no call writes")

    @property
    def vocab(self) -> int:
        return self.head.vocab

    def weight_specs(self):
        specs: dict[str, WeightSpec] = {}
        for part in [self.embedding, *self.blocks, self.head]:
            for s in part.weight_specs():
                if s.name in specs and specs[s.name].shape != s.shape:
                    raise ValueError(f"tensor {s.name} is wanted with shapes {specs[s.name].shape} and {s.shape}")
                specs.setdefault(s.name, s)
        return tuple(specs.values())

    def bind(self, weights, rt) -> None:
        for part in [self.embedding, *self.blocks, self.head]:
            part.bind(weights, rt)

    @property
    def graph_safe(self) -> bool:
        return all(getattr(m, "graph_safe", False) for m in self.mixers())

    def planners(self) -> dict:
        """{plan key: one mixer that makes that plan}."""
        out = {}
        for m in self.mixers():
            key = m.plan_key() if hasattr(m, "plan_key") else None
            if key is not None and key not in out:
                out[key] = m
        return out

    def mixers(self):
        return [b.mixer for b in self.blocks]

    def cache_entries(self):
        """{cache entry: the need of the mixer that uses it}."""
        needs = {}
        for c in self.run_order:
            need = self.blocks[c.block].mixer.cache_need()
            if c.cache in needs and needs[c.cache] != need:
                raise ValueError(f"cache entry {c.cache} is shared by mixers with different needs")
            needs[c.cache] = need
        return needs

    def forward(self, ctx) -> torch.Tensor:
        """Run this step's tokens; return float32 logits [len(ctx.logit_rows), vocab]."""
        stream = self.embedding.forward(ctx)
        last = len(self.run_order) - 1
        rows = None if ctx.all_rows_wanted else ctx.logit_rows
        for i, call in enumerate(self.run_order):
            cache = ctx.layer_cache(call.cache, call.write_cache)
            stream = self.blocks[call.block].forward(ctx, stream, cache, rows if i == last else None)
        return self.head.forward(ctx, stream)
