"""Turns the logits of a step into next tokens on the device.

The reference computes ``softmax(logits / temperature)``, draws with FlashInfer's
``sampling_from_probs`` from ``torch.rand``, takes ``argmax`` for greedy rows and the log of the
chosen probability (tokasaurus/model/llama.py:377-423).  Here one kernel does greedy argmax or a
Gumbel-max draw (the same distribution), the chosen token's log-probability under
softmax(logits / temperature), and the write of the token into the per-slot last-token table
(tokasaurus/model/basic_worker.py:125-137); an optional second kernel gives top-k log-probabilities.
"""

from __future__ import annotations

import torch

from tokasaurus_b200.kernels import ops


class Sampler:
    def __init__(self, device: torch.device, max_rows: int, want_logprobs: bool = True, landing_places: int = 2):
        self.device = device
        self.landing_places = max(2, int(landing_places))
        self.want_logprobs = want_logprobs
        self.bytes_last_read = 0
        self._alloc(max_rows)

    def _alloc(self, n: int) -> None:
        self.max_rows = n
        self.out = torch.zeros((2 * n,), dtype=torch.int32, device=self.device)
        cuda = self.device.type == "cuda"
        # several landing places on the host, so that the results of the steps in flight can be on their way while
        # the step before them is still being read; the last word of each holds the device's status flag
        self.host = [torch.zeros((2 * n + 1,), dtype=torch.int32, pin_memory=cuda) for _ in range(self.landing_places)]
        self.events = [torch.cuda.Event() if cuda else None for _ in range(self.landing_places)]

    def sample(self, logits: torch.Tensor, temperature: torch.Tensor, stream_key: torch.Tensor,
               sample_pos: torch.Tensor, row_slot: torch.Tensor, last_token: torch.Tensor) -> None:
        """Fill ``self.out``: ids in [0, R), log-probabilities (float bits) in [R, 2R)."""
        R = logits.shape[0]
        if R > self.max_rows:
            raise ValueError(f"{R} rows to sample, the sampler was made for {self.max_rows}")
        ids = self.out[:R]
        lp = self.out[R:2 * R].view(torch.float32) if self.want_logprobs else None
        ops.sample(logits, temperature, stream_key, sample_pos, row_slot, ids, lp, last_token)

    def start_read(self, R: int, slot: int = 0, status: torch.Tensor | None = None) -> None:
        """Put the copy of the last results (and of the device's status word) to landing place ``slot`` into
        the stream; does not wait."""
        n = 2 * R if self.want_logprobs else R
        host = self.host[slot]
        host[:n].copy_(self.out[:n], non_blocking=True)
        if status is not None:
            host[-1:].copy_(status, non_blocking=True)
        else:
            host[-1] = 0
        if self.events[slot] is not None:
            self.events[slot].record(torch.cuda.current_stream(self.device))
        self.bytes_last_read = 4 * n + (4 if status is not None else 0)

    def finish_read(self, R: int, slot: int = 0) -> tuple[list[int], list[float], int]:
        """Wait for ``start_read`` of ``slot``; ids, log-probabilities and the status word."""
        if self.events[slot] is not None:
            self.events[slot].synchronize()
        host = self.host[slot]
        ids = host[:R].tolist()
        lps = host[R:2 * R].view(torch.float32).tolist() if self.want_logprobs else [0.0] * R
        return ids, lps, int(host[-1])

    def read(self, R: int) -> tuple[list[int], list[float]]:
        """Copy the last results to the host (waits for the step)."""
        self.start_read(R, 0)
        ids, lps, _ = self.finish_read(R, 0)
        return ids, lps

    def topk(self, logits: torch.Tensor, temperature: torch.Tensor, k: int) -> tuple[torch.Tensor, torch.Tensor]:
        R = logits.shape[0]
        idx = torch.empty((R, k), dtype=torch.int32, device=logits.device)
        lp = torch.empty((R, k), dtype=torch.float32, device=logits.device)
        ops.topk_logprobs(logits, temperature, k, idx, lp)
        return idx, lp
