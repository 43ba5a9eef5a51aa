"""The one place that asks the device what it is: the SM count and the shared memory of an SM.  Host-side planners
(the attention's work split) size their work by these; the CUDA sources ask the runtime themselves
(``tkb::sm_count()`` in csrc/common.cuh)."""

from __future__ import annotations

from dataclasses import dataclass

import torch


@dataclass(frozen=True)
class DeviceLimits:
    """What host-side planners size their work by.  Asked of the device once (``device_limits``); no other file
    of the package holds such a number."""

    sm_count: int
    shared_memory_per_sm: int  # bytes of shared memory the blocks resident on one SM can hold together


# Planning without a GPU (host-only tests of the planners, which must give the same plans everywhere): the
# figures of the GPU this engine is written for, a B200.
NO_DEVICE = DeviceLimits(sm_count=148, shared_memory_per_sm=227 * 1024)
_limits: dict[tuple, DeviceLimits] = {}


def device_limits(device: torch.device | str) -> DeviceLimits:
    device = torch.device(device)
    if device.type != "cuda" or not torch.cuda.is_available():
        return NO_DEVICE
    key = (device.type, device.index)
    got = _limits.get(key)
    if got is None:
        props = torch.cuda.get_device_properties(device)
        smem = getattr(props, "shared_memory_per_block_optin", None) or (props.shared_memory_per_multiprocessor - 1024)
        got = _limits[key] = DeviceLimits(int(props.multi_processor_count), int(smem))
    return got
