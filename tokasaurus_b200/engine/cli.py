"""The ``toka`` command line: ``toka model=<folder> key=value ...``.

The grammar is the reference's pydra grammar (tokasaurus/entry.py:139-143; ``key=value``,
``key=T``/``key=F``, ``key='(2*1024)'``), and the engine options keep the names of its
``ServerConfig`` (tokasaurus/common_types.py:52-126).  The reference then starts an HTTP server; this
engine has none, so the command takes prompts as token ids (``prompt_ids='[1,2,3]'`` or
``prompts_file=<jsonl>``: one list of ids, or an object with ``input_ids``, a line), generates, and
prints one JSON object a line: ``{"id", "completion_ids", "logprobs", "finish_reason"}``.
"""

from __future__ import annotations

import json
import sys
import time

from tokasaurus_b200.config.engine_config import EngineConfig, OptionError, parse_overrides

RUN_OPTIONS = {
    "prompt_ids": str,
    "prompts_file": str,
    "output_file": str,
    "temperature": float,
    "seed": int,
    "max_num_tokens": int,
    "ignore_eos": bool,
    "topk_logprobs": int,
    "kv_reserve_fraction": float,
    "admission": str,
}


def _read_prompts(opts: dict) -> list[list[int]]:
    prompts: list[list[int]] = []
    if opts.get("prompt_ids"):
        v = json.loads(opts["prompt_ids"])
        prompts.extend(v if v and isinstance(v[0], list) else [v])
    if opts.get("prompts_file"):
        with open(opts["prompts_file"]) as f:
            for line in f:
                line = line.strip()
                if not line:
                    continue
                v = json.loads(line)
                prompts.append(v["input_ids"] if isinstance(v, dict) else v)
    return prompts


def help_text() -> str:
    """The module's description, then every option with its default: the engine's (``EngineConfig``, under the
    reference's names) and those of this command."""
    from dataclasses import fields

    lines = [__doc__.rstrip(), "", "engine options (key=value):"]
    lines += [f"  {f.name}={f.default!r}" for f in fields(EngineConfig)]
    lines += ["", "options of this command:"]
    lines += [f"  {k}=<{t.__name__}>" for k, t in RUN_OPTIONS.items()]
    return "\n".join(lines)


def main(argv: list[str] | None = None) -> int:
    argv = sys.argv[1:] if argv is None else argv
    if not argv or argv[0] in ("-h", "--help"):
        print(help_text())
        return 0
    try:
        cfg, opts = parse_overrides(argv, EngineConfig, RUN_OPTIONS)
    except OptionError as e:
        print(f"toka: {e}", file=sys.stderr)
        return 2
    if cfg.model is None:
        print("toka: model=<folder> is required", file=sys.stderr)
        return 2
    prompts = _read_prompts(opts)
    if not prompts:
        print("toka: give prompt_ids='[...]' or prompts_file=<jsonl>", file=sys.stderr)
        return 2
    import logging

    from tokasaurus_b200.engine.engine import Engine
    from tokasaurus_b200.sampling.params import SamplingParams

    # the engine's statistics lines (level INFO, every stats_report_seconds) go to the standard error stream
    logging.basicConfig(stream=sys.stderr, format="[toka] %(message)s")
    engine = Engine(config=cfg, seed=opts.get("seed") or 0, kv_reserve_fraction=opts.get("kv_reserve_fraction", 1.0),
                    admission=opts.get("admission"))
    sp = SamplingParams(temperature=opts.get("temperature") or 0.0, seed=opts.get("seed"))
    t0 = time.time()
    outs = engine.generate(prompts, sp, max_num_tokens=opts.get("max_num_tokens") or 16,
                           ignore_eos=bool(opts.get("ignore_eos")), topk_logprobs=opts.get("topk_logprobs"))
    dt = time.time() - t0
    sink = open(opts["output_file"], "w") if opts.get("output_file") else sys.stdout
    for o in outs:
        rec = dict(id=o.id, completion_ids=o.completion_ids, logprobs=o.logprobs, finish_reason=o.finish_reason)
        if o.topk_ids:
            rec["topk_ids"] = o.topk_ids
            rec["topk_logprobs"] = o.topk_logprobs
        print(json.dumps(rec), file=sink)
    if sink is not sys.stdout:
        sink.close()
    n = sum(len(o.completion_ids) for o in outs)
    st = engine.scheduler.stats
    print(f"[toka] {len(outs)} requests, {n} tokens in {dt:.2f} s ({n / max(dt, 1e-9):.1f} tok/s); "
          f"steps {st['steps']}, prefill tokens {st['prefill_tokens']}, bumps {st['bumps']}", file=sys.stderr)
    return 0


if __name__ == "__main__":
    sys.exit(main())
