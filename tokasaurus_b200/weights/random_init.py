"""Random weights from a configuration and a seed, and a writer of model folders.

The reference has no such mode (its warm-up runs real checkpoints).  Values are drawn on the
CPU in float32 from one ``torch.Generator``, tensor by tensor in the order of the model's
``weight_specs`` (matrices N(0, std); vectors, i.e. norm weights, ones or U(0.5, 1.5)), then
rounded to the dtype they are stored in, so that anything that reads the folder sees the same
numbers.
"""

from __future__ import annotations

import json
from pathlib import Path
from typing import Any, Iterable

import torch
from safetensors.torch import save_file

from tokasaurus_b200.parts.base import WeightSpec

_STORE = {"bfloat16": torch.bfloat16, "float32": torch.float32}


def random_tensors(specs: Iterable[WeightSpec], seed: int, std: float = 0.02, norm_init: str = "ones",
                   store_dtype: str = "bfloat16", device: torch.device | str = "cpu") -> dict[str, torch.Tensor]:
    """``device``: where the values are drawn and left.  The CPU's generator and a GPU's give different numbers for
    the same seed: a model folder is always written from the CPU's (what reads the folder sees the same numbers on
    any machine), while an engine that only needs some model of the given sizes (the benchmark's billions of
    values) draws them where it will use them."""
    if norm_init not in ("ones", "uniform"):
        raise ValueError("norm_init is 'ones' or 'uniform'")
    dt = _STORE[store_dtype]
    device = torch.device(device)
    g = torch.Generator(device=device)
    g.manual_seed(int(seed))
    out: dict[str, torch.Tensor] = {}
    for s in specs:
        if s.role == "table":
            out[s.name] = torch.randint(0, 2**15, s.shape, generator=g, dtype=torch.int32, device=device)
        elif s.role == "vector":
            if norm_init == "ones":
                t = torch.ones(s.shape, dtype=torch.float32, device=device)
            else:
                t = torch.rand(s.shape, generator=g, dtype=torch.float32, device=device) + 0.5
            out[s.name] = t.to(dt)
        else:
            out[s.name] = torch.randn(s.shape, generator=g, dtype=torch.float32, device=device).mul_(std).to(dt)
    return out


def write_model_folder(folder: str | Path, config_dict: dict[str, Any], seed: int, std: float = 0.02,
                       norm_init: str = "ones", store_dtype: str = "bfloat16") -> Path:
    """Write ``config.json`` and ``model.safetensors`` for the architecture that ``config_dict`` names."""
    from tokasaurus_b200.config.registry import lookup_architecture

    arch = lookup_architecture(config_dict)
    cfg = arch.parse_config(config_dict)
    model = arch.build_model(cfg)
    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    tensors = random_tensors(model.weight_specs(), seed, std, norm_init, store_dtype)
    save_file({k: v.contiguous() for k, v in tensors.items()}, str(folder / "model.safetensors"))
    d = dict(config_dict)
    d.setdefault("architectures", [arch.name])
    d["torch_dtype"] = store_dtype
    with open(folder / "config.json", "w") as f:
        json.dump(d, f, indent=1)
    return folder
