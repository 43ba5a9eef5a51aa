"""Ways of cutting the same requests into steps for trace replay, and the comparison of what
comes back with the plain implementation."""

from __future__ import annotations

import numpy as np
import torch

from plain_llama import PlainLlama


def random_tokens(n: int, vocab: int, seed: int) -> list[int]:
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


def whole(reqs: dict[str, list[int]]):
    """Each request alone and whole: one step, all logits wanted."""
    steps = []
    for i, (rid, toks) in enumerate(reqs.items()):
        steps.append(dict(step=i, entries=[dict(id=rid, tokens=toks, want=list(range(len(toks))))], end=[rid]))
    return steps


def prefix_then_single(reqs: dict[str, list[int]], tail: int = 32):
    """Most of it in one step, the last ``tail`` tokens one by one."""
    steps = []
    n = 0
    for rid, toks in reqs.items():
        cut = max(1, len(toks) - tail)
        steps.append(dict(step=n, entries=[dict(id=rid, tokens=toks[:cut], want=list(range(cut)))], end=[]))
        n += 1
        for j in range(cut, len(toks)):
            steps.append(dict(step=n, entries=[dict(id=rid, tokens=[toks[j]], want=[0])],
                              end=[rid] if j == len(toks) - 1 else []))
            n += 1
        if cut == len(toks):
            steps[-1]["end"] = [rid]
    return steps


PORTIONS = [7, 2, 24, 3, 2, 17, 5, 2, 31, 9, 2, 16, 8, 1, 13]


def changing_portions(reqs: dict[str, list[int]], sizes=PORTIONS):
    steps = []
    n = 0
    for rid, toks in reqs.items():
        at, k = 0, 0
        while at < len(toks):
            m = min(sizes[k % len(sizes)], len(toks) - at)
            k += 1
            steps.append(dict(step=n, entries=[dict(id=rid, tokens=toks[at:at + m], want=list(range(m)))],
                              end=[rid] if at + m == len(toks) else []))
            at += m
            n += 1
    return steps


def mixed(reqs: dict[str, list[int]], max_live: int = 4, prompt_frac: float = 0.6, seed: int = 0,
          sizes=(5, 2, 19, 3, 11, 2, 8)):
    """Up to ``max_live`` requests at a time: each goes through its first part in portions of
    changing size and through the rest one token a step, beside whatever the others are doing;
    now and then a request sits a step out.  A request that ends makes room for the next."""
    rng = np.random.default_rng(seed)
    waiting = list(reqs.items())
    live: dict[str, dict] = {}
    steps = []
    n = 0
    while waiting or live:
        while waiting and len(live) < max_live:
            rid, toks = waiting.pop(0)
            live[rid] = dict(toks=toks, at=0, k=int(rng.integers(0, len(sizes))),
                             prompt=min(len(toks), max(2, int(len(toks) * prompt_frac))))
        entries, end = [], []
        for rid, st in list(live.items()):
            if len(live) > 1 and rng.random() < 0.15:
                continue  # left out of this step, goes on later
            toks, at = st["toks"], st["at"]
            if at < st["prompt"]:
                m = min(sizes[st["k"] % len(sizes)], st["prompt"] - at)
                st["k"] += 1
            else:
                m = 1
            entries.append(dict(id=rid, tokens=toks[at:at + m], want=list(range(m))))
            st["at"] = at + m
            if st["at"] == len(toks):
                end.append(rid)
                del live[rid]
        if entries:
            steps.append(dict(step=n, entries=entries, end=end))
            n += 1
    return steps


def waves_of_decoding(reqs: dict[str, list[int]], wave: int, tail: int = 6, prefill_group: int = 8):
    """Decode steps of many requests: the requests run in waves of ``wave``; within a wave, each request's tokens
    but the last ``tail`` go in as whole prompts, ``prefill_group`` requests a step, then ``tail`` steps follow in
    which EVERY request of the wave brings one token; then the wave ends and the next one takes over its pages."""
    steps = []
    items = list(reqs.items())
    for w in range(0, len(items), wave):
        group = items[w:w + wave]
        for g in range(0, len(group), prefill_group):
            entries = []
            for rid, toks in group[g:g + prefill_group]:
                cut = max(1, len(toks) - tail)
                entries.append(dict(id=rid, tokens=toks[:cut], want=list(range(cut))))
            steps.append(dict(step=len(steps), entries=entries, end=[]))
        for t in range(tail, 0, -1):
            entries = [dict(id=rid, tokens=[toks[len(toks) - t]], want=[0]) for rid, toks in group if len(toks) > t]
            if entries:
                steps.append(dict(step=len(steps), entries=entries, end=[]))
        steps[-1]["end"] = [rid for rid, _ in group]
    return steps


def max_live_tokens(steps, round_to: int = 64) -> int:
    """The --max-tokens a trace needs: the most tokens live requests hold at any time, each
    request's count rounded up to a multiple of ``round_to``."""
    held: dict[str, int] = {}
    peak = 0
    for st in steps:
        for e in st["entries"]:
            held[e["id"]] = held.get(e["id"], 0) + len(e["tokens"])
        peak = max(peak, sum(-(-v // round_to) * round_to for v in held.values()))
        for rid in st["end"]:
            held.pop(rid, None)
    return peak


def collect(steps, outputs) -> dict[str, np.ndarray]:
    """Put the per-step logits back together: {request: [tokens, vocab]} (every place was wanted)."""
    rows: dict[str, list[np.ndarray]] = {}
    for st, out in zip(steps, outputs):
        r = 0
        for e in st["entries"]:
            for _ in e["want"]:
                rows.setdefault(e["id"], []).append(out[r])
                r += 1
        assert out is None and r == 0 or r == out.shape[0]
    return {k: np.stack(v) for k, v in rows.items()}


def plain_logits(model_dir, reqs: dict[str, list[int]], dtype=torch.float64) -> dict[str, np.ndarray]:
    m = PlainLlama(model_dir, dtype)
    return {rid: m.logits(toks).double().numpy() for rid, toks in reqs.items()}


def tolerance(kind: str, plain64: np.ndarray, plain32: np.ndarray | None = None) -> float:
    """float32: four times what 32-bit arithmetic alone costs the plain implementation, at least
    1e-5 of the largest logit.  bfloat16: 3 % of the largest logit (eight-bit mantissas through
    every layer)."""
    top = float(np.abs(plain64).max())
    if kind == "float32":
        spread = float(np.abs(plain32 - plain64).max()) if plain32 is not None else 0.0
        return max(4 * spread, 1e-5 * top)
    return 0.03 * top
