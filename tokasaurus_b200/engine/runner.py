"""The model runner: a model built from a folder, its cache, and the one step function.

``step`` is the only way tokens go through the model: the command line, the Python entry point,
the scheduler, trace replay and the benchmark all call it.  The reference's counterpart is
``ModelRunner.plan``/``run`` around ``LlamaForCausalLM.forward`` (tokasaurus/model/utils.py:723-882,
tokasaurus/model/llama.py:644-667).
"""

from __future__ import annotations

import json
from pathlib import Path
from typing import Any, Sequence

import torch

from tokasaurus_b200.cache.manager import CacheManager
from tokasaurus_b200.config.engine_config import EngineConfig, parse_rope_scaling_override
from tokasaurus_b200.config.model_config import read_config_json, read_eos_token_ids
from tokasaurus_b200.config.registry import lookup_architecture
from tokasaurus_b200.engine.batch import Stager, StepContext, StepEntry, build_host_batch
from tokasaurus_b200.engine.runtime import Runtime
from tokasaurus_b200.kernels import ops
from tokasaurus_b200.parts.base import PagedCacheNeed
from tokasaurus_b200.weights.loader import load_weights, target_dtype
from tokasaurus_b200.weights.random_init import random_tensors


class DeviceStatusError(RuntimeError):
    pass


def require_cuda(device: torch.device) -> None:
    if device.type != "cuda" or not torch.cuda.is_available():
        raise RuntimeError(
            f"tokasaurus_b200 runs on a CUDA device (sm_100a) only; asked for {device}, CUDA available: "
            f"{torch.cuda.is_available()}.  There is no CPU execution path."
        )
    torch.cuda.set_device(device)


class ModelRunner:
    def __init__(self, config: EngineConfig, config_dict: dict[str, Any] | None = None):
        """``config.model`` names a folder with config.json (and model.safetensors unless
        ``config.random_weights`` gives a seed).  ``config_dict`` may stand in for config.json."""
        self.config = config
        self.rt = Runtime.make(config.device, config.dtype)
        require_cuda(self.rt.device)
        if config_dict is None:
            if config.model is None:
                raise ValueError("give model=<folder> or a configuration dictionary")
            config_dict = read_config_json(config.model)
        config_dict = dict(config_dict)
        override = parse_rope_scaling_override(config.rope_scaling)
        if override is not None:
            config_dict["rope_scaling"] = override
        self.config_dict = config_dict
        self.arch = lookup_architecture(config_dict)
        self.model_config = self.arch.parse_config(config_dict)
        self.model = self.arch.build_model(self.model_config)
        self.eos_token_ids = (
            read_eos_token_ids(config.model, config_dict) if config.model else
            tuple([config_dict["eos_token_id"]] if isinstance(config_dict.get("eos_token_id"), int)
                  else config_dict.get("eos_token_id") or ())
        )
        config.finalize(getattr(self.model_config, "max_position_embeddings", None))

        needs = self.model.cache_entries()
        head_dims = sorted({n.head_dim for n in needs.values() if isinstance(n, PagedCacheNeed)})
        ops.prepare(head_dims, self.rt.dtype)

        specs = self.model.weight_specs()
        if config.random_weights is not None:
            host = random_tensors(specs, config.random_weights, device=self.rt.device)
            by_name = {s.name: s for s in specs}
            weights = {
                n: t.to(device=self.rt.device, dtype=target_dtype(by_name[n], t.dtype, self.rt.dtype)).contiguous()
                for n, t in host.items()
            }
        else:
            weights = load_weights(config.model, specs, self.rt.dtype, self.rt.device,
                                   ignore=getattr(self.model, "ignored_weight_patterns", ()))
        self.model.bind(weights, self.rt)
        del weights

        self.cache = CacheManager(needs, config.page_size, config.kv_cache_num_blocks(),
                                  max_requests=config.max_seqs_per_forward, dtype=self.rt.dtype,
                                  device=self.rt.device, max_step_tokens=config.max_tokens_per_forward)
        self.stager = Stager(self.rt.device)
        self.vocab = self.model.vocab
        self.last_upload_bytes = 0

    # ------------------------------------------------------------------
    def step(self, entries: Sequence[StepEntry], extra: dict | None = None) -> torch.Tensor:
        """Run the tokens of ``entries`` as one batch from the cache and return float32 logits
        [wanted places, vocab] on the device, in the order of the entries and of their ``want``.
        Pages for the new positions must have been given to the requests before.  ``extra``: further
        numpy arrays (4- or 8-byte elements) that travel to the device in the same copy; their
        device views are in ``self.last_context.extra``."""
        host = build_host_batch(entries, self.cache)
        plans = {key: mixer.plan(host) for key, mixer in self.model.planners().items()}
        ctx = StepContext(host, self.cache, self.rt.device, self.stager, extra, plans)
        self.last_upload_bytes = self.stager.bytes_last_upload
        self.last_context = ctx
        return self.model.forward(ctx)

    def check_status(self, code: int | None = None) -> None:
        """Raise if a kernel met a token id or a page outside its table since the last check
        (the kernels skip such accesses and set a flag instead of faulting).  ``code``: the status word if
        the caller has read it already (with a step's results); else it is read here, which waits."""
        if code is None:
            code = int(self.stager.status.item())
        if code:
            self.stager.status.zero_()
            what = []
            if code & 1:
                what.append("a token id outside the vocabulary")
            if code & 2:
                what.append("a page id outside the pool")
            if code & 4:
                what.append("a bounded wait in a kernel ran out")
            raise DeviceStatusError("device status " + str(code) + ": " + "; ".join(what))
