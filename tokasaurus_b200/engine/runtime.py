"""What parts need to know about where and how they run."""

from __future__ import annotations

from dataclasses import dataclass

import torch

from tokasaurus_b200.kernels.device import NO_DEVICE, DeviceLimits, device_limits

DTYPES = {"bfloat16": torch.bfloat16, "float32": torch.float32}


@dataclass(frozen=True)
class Runtime:
    device: torch.device
    dtype: torch.dtype  # activations, matrices and cache: bfloat16 (serving) or float32 (true 32-bit path)
    limits: DeviceLimits = NO_DEVICE

    @staticmethod
    def make(device: str | torch.device, dtype: str | torch.dtype) -> "Runtime":
        if isinstance(dtype, str):
            if dtype not in DTYPES:
                raise ValueError(f"dtype {dtype!r}: this engine runs 'bfloat16' or 'float32'")
            dtype = DTYPES[dtype]
        device = torch.device(device)
        return Runtime(device, dtype, device_limits(device))
