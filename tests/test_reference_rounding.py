"""The reference's bfloat16 arithmetic, stated as roundings (``plain_llama_bf16``), beside the engine's: the engine
keeps the residual stream in float32 and rounds once in its norms, so it must be nearer the float64 yardstick than
the reference's rounding is, and as near the reference's bfloat16 logits as the bfloat16 tolerance allows."""

import numpy as np
import pytest
import torch

import cuttings
from plain_llama import PlainLlama, TINY_WEIGHTS
from plain_llama_bf16 import PlainLlamaReferenceRounding, r, rms_norm


def rms(x) -> float:
    return float(np.sqrt(np.mean(np.square(np.asarray(x, dtype=np.float64)))))


def test_cast_then_weight_is_two_roundings():
    """tokasaurus/model/llama.py:51: the normalised value is cast before it meets the weight.  A normalised value of
    1.0039 times a weight of 1.0078125 rounds differently in the two orders, so the emulation can tell them apart."""
    c = 1.0039
    d = (2.0 - c * c) ** 0.5  # mean square 1: the row is its own normalised value
    x = torch.tensor([[c, d, -c, -d]], dtype=torch.float64)
    w = torch.full((4,), 1.0078125, dtype=torch.float64)  # a bfloat16 number
    two = rms_norm(x, w, 0.0)
    one = r(w * (x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True))))
    assert torch.equal(r(two), two) and torch.equal(r(one), one)
    assert two[0, 0].item() == 1.0078125  # 1.0039 -> 1.0, then times the weight
    assert one[0, 0].item() == 1.015625  # 1.011743 is past the middle between 1.0078125 and 1.015625


@pytest.mark.parametrize("cfg_index", [0, 1])
def test_reference_rounding_stays_near_float64(tiny_model_dirs, cfg_index):
    """The reference's roundings cost a fraction of a percent of the logits' size on the test models, and they are
    not nothing: the emulation differs from the exact arithmetic at most positions."""
    d = tiny_model_dirs[cfg_index]
    toks = cuttings.random_tokens(100, PlainLlama(d).cfg["vocab_size"], 5)
    exact = PlainLlama(d).logits(toks).numpy()
    rounded = PlainLlamaReferenceRounding(d).logits(toks).numpy()
    assert 1e-4 * rms(exact) < rms(rounded - exact) < 2e-2 * rms(exact)
    assert np.abs(rounded - exact).max() <= cuttings.tolerance("bfloat16", exact)


@pytest.mark.gpu
@pytest.mark.parametrize("cfg_index", [0, 1])
def test_engine_bfloat16_beside_the_reference_rounding(tiny_model_dirs, cfg_index):
    from tokasaurus_b200.engine.trace import TraceReplayer

    d = tiny_model_dirs[cfg_index]
    vocab = PlainLlama(d).cfg["vocab_size"]
    reqs = {f"r{i}": cuttings.random_tokens(n, vocab, 40 + i) for i, n in enumerate((100, 160, 37))}
    steps = cuttings.whole(reqs)
    rp = TraceReplayer(str(d), "bfloat16", cuttings.max_live_tokens(steps), page_size=TINY_WEIGHTS[cfg_index]["page_size"])
    got = cuttings.collect(steps, [rp.run_step(st) for st in steps])
    exact_model, rounded_model = PlainLlama(d), PlainLlamaReferenceRounding(d)
    ours, theirs = [], []
    for rid, toks in reqs.items():
        exact = exact_model.logits(toks).numpy()
        rounded = rounded_model.logits(toks).numpy()
        ours.append(got[rid] - exact)
        theirs.append(rounded - exact)
        # as near the reference's bfloat16 logits as the float64 ones
        assert np.abs(got[rid] - rounded).max() <= cuttings.tolerance("bfloat16", exact)
    ours, theirs = np.concatenate(ours), np.concatenate(theirs)
    print(f"config {cfg_index}: rms error of the engine {rms(ours):.3g}, of the reference's rounding {rms(theirs):.3g}")
    # fewer roundings: nearer the exact result, over all logits of all positions
    assert rms(ours) <= rms(theirs)
