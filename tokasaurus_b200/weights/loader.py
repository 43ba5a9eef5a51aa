"""Read tensors from safetensors files by name.

The reference opens ``model.safetensors``, or the shards that ``model.safetensors.index.json``
maps names to, and takes the wanted names (tokasaurus/model/safetensors_utils.py:29-31,34-97).
A missing name surfaces there as a bare KeyError (tokasaurus/model/llama.py:938) and shapes are
not checked; here all problems of a folder are collected into one error.

dtype policy: "matrix" tensors are kept in the engine's dtype (bfloat16 for serving), except
that a tensor marked ``keep_32bit`` stays float32 if the file stores it so; "vector" tensors
(norm weights) are used in 32-bit arithmetic and are held as float32 (widening loses nothing);
"table" tensors are integer tables and are held as int32.
"""

from __future__ import annotations

import fnmatch
import warnings
import json
from pathlib import Path
from typing import Iterable, Sequence

import torch
from safetensors import safe_open

from tokasaurus_b200.parts.base import WeightSpec


class WeightLoadError(ValueError):
    def __init__(self, folder: str, missing: Sequence[str], unexpected: Sequence[str],
                 wrong_shape: Sequence[tuple[str, tuple, tuple]], other: Sequence[str] = ()):
        self.folder = folder
        self.missing = list(missing)
        self.unexpected = list(unexpected)
        self.wrong_shape = list(wrong_shape)
        self.other = list(other)
        lines = [f"cannot load weights from {folder!r}:"]
        if self.missing:
            lines.append(f"  missing tensors ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected tensors ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        if self.wrong_shape:
            lines.append(f"  wrong shapes ({len(self.wrong_shape)}): " + ", ".join(
                f"{n} is {list(got)}, expected {list(want)}" for n, got, want in self.wrong_shape))
        lines.extend("  " + o for o in self.other)
        super().__init__("\n".join(lines))


def _files_by_name(folder: Path) -> dict[str, Path]:
    single = folder / "model.safetensors"
    index = folder / "model.safetensors.index.json"
    names: dict[str, Path] = {}
    if single.is_file():
        with safe_open(str(single), framework="pt") as f:
            for k in f.keys():
                names[k] = single
        return names
    if index.is_file():
        with open(index) as f:
            weight_map = json.load(f)["weight_map"]
        for k, fname in weight_map.items():
            names[k] = folder / fname
        return names
    raise FileNotFoundError(
        f"model folder {str(folder)!r} holds neither model.safetensors nor model.safetensors.index.json"
    )


def target_dtype(spec: WeightSpec, stored: torch.dtype, engine_dtype: torch.dtype) -> torch.dtype:
    if spec.role == "table":
        return torch.int32
    if spec.role == "vector":
        return torch.float32
    if spec.keep_32bit and stored == torch.float32:
        return torch.float32
    return engine_dtype


def load_weights(folder: str | Path, specs: Iterable[WeightSpec], engine_dtype: torch.dtype,
                 device: torch.device | str, ignore: Sequence[str] = ()) -> dict[str, torch.Tensor]:
    """Return {name: tensor on ``device``} for every spec; raise ``WeightLoadError`` listing all
    missing names, all names in the files that no part asked for (unless they match a pattern of
    ``ignore``), and all shape mismatches."""
    folder = Path(folder)
    specs = list(specs)
    where = _files_by_name(folder)
    wanted = {s.name: s for s in specs}
    missing = [n for n in wanted if n not in where]
    extra = sorted(n for n in where if n not in wanted)
    unexpected = [n for n in extra if not any(fnmatch.fnmatch(n, p) for p in ignore)]
    passed_over = [n for n in extra if n not in unexpected]
    if passed_over:
        warnings.warn(f"{folder}: {len(passed_over)} tensors that this architecture's checkpoints may carry are not "
                      f"used: {', '.join(passed_over[:4])}{', ...' if len(passed_over) > 4 else ''}", stacklevel=2)
    wrong: list[tuple[str, tuple, tuple]] = []
    other: list[str] = []
    by_file: dict[Path, list[str]] = {}
    for n in wanted:
        if n in where:
            by_file.setdefault(where[n], []).append(n)
    out: dict[str, torch.Tensor] = {}
    for path, names in by_file.items():
        if not path.is_file():
            other.append(f"shard file {path.name} named by the index is missing")
            continue
        with safe_open(str(path), framework="pt") as f:
            for n in names:
                shape = tuple(f.get_slice(n).get_shape())
                if shape != tuple(wanted[n].shape):
                    wrong.append((n, shape, tuple(wanted[n].shape)))
                    continue
                if missing or unexpected or wrong or other:
                    continue  # an error is coming: do not spend time reading
                t = f.get_tensor(n)
                spec = wanted[n]
                if spec.role == "table" and t.dtype.is_floating_point:
                    other.append(f"{n} should be an integer table but is stored as {t.dtype}")
                    continue
                if spec.role != "table" and not t.dtype.is_floating_point:
                    other.append(f"{n} should be floating point but is stored as {t.dtype}")
                    continue
                out[n] = t.to(device=device, dtype=target_dtype(spec, t.dtype, engine_dtype)).contiguous()
    if missing or unexpected or wrong or other:
        raise WeightLoadError(str(folder), missing, unexpected, wrong, other)
    return out
