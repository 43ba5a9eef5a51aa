"""What a caller may ask of sampling, and what comes back.

The reference's request carries ``SamplingParams(temperature, top_p)``, ``max_num_tokens``,
``stop``, ``n``, ``ignore_eos`` and ``topk_logprobs`` (tokasaurus/server/types.py:136-152); ``top_p``
must be 1.0 (tokasaurus/model/types.py:318) and a temperature of 0 means greedy
(tokasaurus/model/types.py:302-312).  Stop *strings* need a tokenizer, which this engine does not
have: ``stop_token_ids`` stands in.  ``seed`` exists in the reference's API but is never read
there; here it selects the random stream of the request.
"""

from __future__ import annotations

from dataclasses import dataclass, field


@dataclass
class SamplingParams:
    temperature: float = 0.0
    top_p: float = 1.0
    seed: int | None = None

    def validate(self) -> None:
        if self.top_p != 1.0:
            raise ValueError("top_p must be 1.0: nucleus sampling is not offered (nor by the reference's model code)")
        if not self.temperature >= 0.0:
            raise ValueError("temperature must be >= 0 (0 is greedy)")


@dataclass
class Request:
    id: str
    input_ids: list[int]
    max_num_tokens: int
    sampling_params: SamplingParams = field(default_factory=SamplingParams)
    ignore_eos: bool = False
    stop_token_ids: tuple[int, ...] = ()
    topk_logprobs: int | None = None


@dataclass
class RequestOutput:
    id: str
    completion_ids: list[int] = field(default_factory=list)
    logprobs: list[float] = field(default_factory=list)
    topk_ids: list[list[int]] = field(default_factory=list)
    topk_logprobs: list[list[float]] = field(default_factory=list)
    finish_reason: str | None = None  # "length" or "stop" (tokasaurus/manager/manager.py:224-231)
    num_preemptions: int = 0


_MASK = (1 << 64) - 1


def _splitmix64(x: int) -> int:
    x = (x + 0x9E3779B97F4A7C15) & _MASK
    z = x
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _MASK
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _MASK
    return z ^ (z >> 31)


def stream_key(seed: int, request_index: int) -> int:
    """64-bit key of a request's random stream, as a signed int64 for transport."""
    k = _splitmix64((seed & _MASK) ^ _splitmix64(request_index & _MASK))
    return k - (1 << 64) if k >= (1 << 63) else k
