"""Trace replay: feed given token ids through the model step by step and write logits.

It samples nothing and owns no model code: it calls ``ModelRunner.step`` with the cache manager
that generation uses.  The reference's nearest tool is tokasaurus/benchmarks/bench_model.py:142-283,
which hand-builds sequences and batches for timing and writes no logits.

Input (standard input), one JSON object a line::

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

For a step in which something is wanted, ``<out>/<step>.f32`` receives the logits at the wanted
places, in the order of the entries and of ``want``, as little-endian float32 [wanted, vocab].
After every step a line ``done <step>`` is printed and flushed.
"""

from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

import numpy as np

from tokasaurus_b200.config.engine_config import EngineConfig
from tokasaurus_b200.engine.batch import StepEntry
from tokasaurus_b200.engine.runner import ModelRunner


class TraceReplayer:
    def __init__(self, model_dir: str, dtype: str, max_tokens: int, page_size: int = 16, device: str = "cuda:0",
                 max_requests: int = 64):
        pool = ((max_tokens + page_size - 1) // page_size) * page_size
        cfg = EngineConfig(model=model_dir, dtype=dtype, page_size=page_size, kv_cache_num_tokens=max(pool, page_size),
                           max_seqs_per_forward=max_requests, device=device, use_cudagraphs=False)
        self.runner = ModelRunner(cfg)
        self.lengths: dict[str, int] = {}

    def run_step(self, record: dict) -> np.ndarray | None:
        cache = self.runner.cache
        entries = []
        for e in record.get("entries", []):
            rid = e["id"]
            tokens = [int(t) for t in e["tokens"]]
            if not tokens:
                continue
            if rid not in self.lengths:
                cache.admit(rid)
                self.lengths[rid] = 0
            start = self.lengths[rid]
            cache.ensure_capacity(rid, start + len(tokens))
            entries.append(StepEntry(rid, tokens, start, [int(w) for w in e.get("want", [])]))
        logits = None
        if entries:
            out = self.runner.step(entries)
            for en in entries:
                self.lengths[en.request] += en.n_tokens
                cache.release_behind_window(en.request, self.lengths[en.request])
            if out.shape[0]:
                logits = out.cpu().numpy()
            self.runner.check_status()
        for rid in record.get("end", []):
            if rid in self.lengths:
                cache.free(rid)
                del self.lengths[rid]
        return logits


def main(argv: list[str] | None = None) -> int:
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True, help="folder for <step>.f32 files")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens that live requests hold at any time (each rounded up to a multiple of 64)")
    ap.add_argument("--page-size", type=int, default=16)
    ap.add_argument("--device", default="cuda:0")
    args = ap.parse_args(argv)
    out_dir = Path(args.out)
    out_dir.mkdir(parents=True, exist_ok=True)
    replayer = TraceReplayer(args.model, args.dtype, args.max_tokens, args.page_size, args.device)
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        record = json.loads(line)
        logits = replayer.run_step(record)
        if logits is not None:
            logits.astype("<f4", copy=False).tofile(out_dir / f"{record['step']}.f32")
        print(f"done {record['step']}", flush=True)
    return 0
