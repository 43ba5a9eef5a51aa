"""Interfaces of the parts a model is put together from.

A model is an embedding, a list of blocks, a run order over those blocks, a final norm and
an output head.  A block arranges a *mixer* (the part that lets tokens see earlier tokens:
attention here), a *feed-forward*, *norms*, and the mixer's *position encoding*.  Each part
receives its sizes and constants as constructor arguments and declares

* the tensors it wants from the weight files (``weight_specs``),
* what it needs from the cache manager (``cache_need``: pages of per-token keys and
  values, or a fixed-size state per request, or nothing),
* how it runs one step's tokens (``forward``).

No part looks at a model configuration or knows which model it is in.  The reference has the
same pieces as ``nn.Module`` classes bound to ``LlamaConfig`` (tokasaurus/model/llama.py:35-53
RMSNorm, :96-287 LlamaAttention, :290-339 LlamaMLP, :342-359 LlamaBlock).
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import TYPE_CHECKING, Mapping, Sequence

if TYPE_CHECKING:  # pragma: no cover
    import torch
    from tokasaurus_b200.engine.batch import StepContext
    from tokasaurus_b200.engine.runtime import Runtime


@dataclass(frozen=True)
class WeightSpec:
    """One tensor a part reads from the weight files, by its name there."""

    name: str
    shape: tuple[int, ...]
    # "matrix": cast to the engine's dtype.  "vector": small per-channel tensor used in
    # 32-bit arithmetic (norm weights); always held as float32.  "table": integer table,
    # held as int32.
    role: str = "matrix"
    # A tensor stored as float32 in the file stays float32 whatever the engine's dtype.
    keep_32bit: bool = False


@dataclass(frozen=True)
class PagedCacheNeed:
    """Per-token keys and values kept in pages.  ``window``: only the last ``window`` keys
    (the query's own included) are ever read, so pages behind it can be given back."""

    n_kv_heads: int
    head_dim: int
    window: int | None = None


@dataclass(frozen=True)
class StateNeed:
    """A fixed-size state per live request (a recurrent mixer's carry, for instance), kept
    in the slot that the cache manager gives the request.  Zeroed when a slot is handed out."""

    shape: tuple[int, ...]
    dtype: str = "float32"


@dataclass(frozen=True)
class QkvStage:
    """An element-wise stage between "q|k|v ready" and the position encoding of an attention mixer, for
    architectures whose projections carry a bias or whose heads are normalised.  The attention kernels honour it
    on every path, the fused decode path included: a mixer that needs one of these gives up no fast path.

    ``bias_names``: tensors (q bias [heads*head_dim], k bias and v bias [kv heads*head_dim]) added to the
    projections.  ``qk_norm_names``: tensors [head_dim] by which every q head / every k head is scaled after an
    RMS norm over the head size (statistics in 32-bit, ``norm_eps``)."""

    bias_names: tuple[str, str, str] | None = None
    qk_norm_names: tuple[str, str] | None = None
    norm_eps: float = 1e-6


class Part:
    def weight_specs(self) -> Sequence[WeightSpec]:
        return ()

    def bind(self, weights: Mapping[str, "torch.Tensor"], rt: "Runtime") -> None:
        """Take the loaded tensors (keys are the names of ``weight_specs``), already on the
        device and in the dtype their role asks for."""


class Norm(Part):
    def forward(self, ctx: "StepContext", stream: "ResidualStream"):
        """Fold the stream's pending update into it and return the normalised rows [T, width]
        in the engine's dtype."""
        raise NotImplementedError


class PositionEncoding:
    """How positions enter a mixer.  ``kind`` is "none" or "rotary"."""

    kind: str = "none"


class Mixer(Part):
    # True if ``forward`` only launches work on the current stream and reads nothing of the step on
    # the host that could change between two steps of the same shape: such a step can be replayed
    # from a CUDA graph.
    graph_safe = False

    def cache_need(self) -> PagedCacheNeed | StateNeed | None:
        return None

    def plan_key(self):
        """A hashable key if this mixer wants a host-side work plan for each step, else None.  Mixers
        with equal keys share one plan."""
        return None

    def plan(self, host, capacity=None):
        """The plan for one step: ``{name: int32 numpy array}``, made from the step's host arrays.  The
        arrays travel to the device with the batch and are found at ``ctx.plans[key][name]`` (host copy:
        ``ctx.host_plans[key]``).  ``capacity`` (a dict or None) gives fixed array sizes when the step
        is captured in a CUDA graph."""
        return {}

    def pad_plan(self, plan: dict, capacity: dict) -> dict:
        """A plan made without capacities, brought to the fixed array sizes ``capacity`` asks for."""
        return plan

    def forward(self, ctx: "StepContext", h: "torch.Tensor", cache, out_rows=None) -> "torch.Tensor":
        """``h`` [T, width]: normalised input rows of this step's tokens.  ``cache``: what the
        cache manager holds for this layer call (``PagedLayerCache`` or ``StateLayerCache`` or
        None).  ``out_rows``: int32 device tensor of the rows whose output is needed (None:
        all).  The cache must be updated for every token whatever ``out_rows`` says.
        Returns [T or len(out_rows), width]."""
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, ctx: "StepContext", h: "torch.Tensor") -> "torch.Tensor":
        raise NotImplementedError


class ResidualStream:
    """The running sum of a token's representation, held in float32, plus one pending
    update in the engine's dtype that the next norm adds before it normalises (so the add
    costs no extra pass over memory)."""

    __slots__ = ("x", "delta")

    def __init__(self, x: "torch.Tensor", delta: "torch.Tensor | None" = None):
        self.x = x
        self.delta = delta
