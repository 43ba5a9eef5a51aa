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
    def __init__(self, device: torch.device, max_rows: int, want_logprobs: bool = True):
        self.device = device
        self.want_logprobs = want_logprobs
        self.bytes_last_read = 0
        self._alloc(max_rows)

    def _alloc(self, n: int) -> None:
        self.max_rows = n
        self.out = torch.zeros((2 * n,), dtype=torch.int32, device=self.device)
        self.host = torch.zeros((2 * n,), dtype=torch.int32, pin_memory=self.device.type == "cuda")

    def sample(self, logits: torch.Tensor, temperature: torch.Tensor, stream_key: torch.Tensor,
               sample_pos: torch.Tensor, row_slot: torch.Tensor, last_token: torch.Tensor) -> None:
        """Fill ``self.out``: ids in [0, R), log-probabilities (float bits) in [R, 2R)."""
        R = logits.shape[0]
        if R > self.max_rows:
            raise ValueError(f"{R} rows to sample, the sampler was made for {self.max_rows}")
        ids = self.out[:R]
        lp = self.out[R:2 * R].view(torch.float32) if self.want_logprobs else None
        ops.sample(logits, temperature, stream_key, sample_pos, row_slot, ids, lp, last_token)

    def read(self, R: int) -> tuple[list[int], list[float]]:
        """Copy the last results to the host (waits for the step)."""
        n = 2 * R if self.want_logprobs else R
        self.host[:n].copy_(self.out[:n], non_blocking=True)
        if self.device.type == "cuda":
            torch.cuda.current_stream(self.device).synchronize()
        self.bytes_last_read = 4 * n
        ids = self.host[:R].tolist()
        lps = self.host[R:2 * R].view(torch.float32).tolist() if self.want_logprobs else [0.0] * R
        return ids, lps

    def topk(self, logits: torch.Tensor, temperature: torch.Tensor, k: int) -> tuple[torch.Tensor, torch.Tensor]:
        R = logits.shape[0]
        idx = torch.empty((R, k), dtype=torch.int32, device=logits.device)
        lp = torch.empty((R, k), dtype=torch.float32, device=logits.device)
        ops.topk_logprobs(logits, temperature, k, idx, lp)
        return idx, lp
