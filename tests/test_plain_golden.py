"""The plain implementation against the logits that the reference's own model code gave for the
same tiny random model (tests/golden/make_reference_golden.py made the files)."""

import json
from pathlib import Path

import numpy as np
import pytest
import torch

from plain_llama import PlainLlama

GOLDEN = Path(__file__).resolve().parent / "golden"


@pytest.mark.parametrize("index", [0, 1])
def test_plain_matches_reference_golden(tmp_path, index):
    """index 0: tied head (the reference reads the embedding for the head, tokasaurus/model/llama.py:842-845),
    plain rotary, two kv heads; index 1: a head of its own, llama3 rotary scaling, one kv head."""
    from tokasaurus_b200.weights import write_model_folder

    meta = json.load(open(GOLDEN / f"reference_cfg{index}_meta.json"))
    ref = np.load(GOLDEN / f"reference_cfg{index}_logits.npy")
    assert meta["config"]["tie_word_embeddings"] == (index == 0)
    folder = write_model_folder(tmp_path / "m", meta["config"], seed=meta["seed"], std=meta["std"],
                                norm_init=meta["norm_init"], store_dtype=meta["store_dtype"])
    plain = PlainLlama(folder, torch.float64)
    checksum = float(sum(t.double().sum().item() for t in plain.w.values()))
    assert abs(checksum - meta["weights_checksum"]) < 1e-6, "the seeded weights differ from those of the golden run"
    got = plain.logits(meta["token_ids"]).numpy()
    assert got.shape == ref.shape
    assert np.abs(got - ref).max() < 5e-6 * max(1.0, meta["logits_abs_max"])
    assert np.array_equal(got.argmax(1), ref.argmax(1))


def test_plain_parts():
    from plain_llama import apply_rope, causal_gqa_attention, rms_norm, rope_inv_freq, rope_tables

    x = torch.randn(5, 12, dtype=torch.float64)
    w = torch.rand(12, dtype=torch.float64)
    y = rms_norm(x, w, 1e-5)
    assert torch.allclose(y, w * x / torch.sqrt((x * x).mean(-1, keepdim=True) + 1e-5))
    inv = rope_inv_freq(8, 10000.0, None)
    assert torch.allclose(inv, torch.tensor([1.0, 0.1, 0.01, 0.001]))
    cos, sin = rope_tables(torch.arange(3), inv)
    q = torch.randn(3, 2, 8, dtype=torch.float64)
    r = apply_rope(q, cos, sin)
    assert torch.allclose(r[0], q[0])  # position 0 is not rotated
    assert torch.allclose(r.norm(dim=-1), q.norm(dim=-1))  # a rotation keeps lengths
    # attention: first query sees only the first key
    k, v = torch.randn(3, 1, 8, dtype=torch.float64), torch.randn(3, 1, 8, dtype=torch.float64)
    o = causal_gqa_attention(q, k, v)
    assert torch.allclose(o[0, 0], v[0, 0]) and torch.allclose(o[0, 1], v[0, 0])
    o2 = causal_gqa_attention(q, k, v, window=1)  # a window of one: each query sees only its own key
    assert torch.allclose(o2[:, 0], v[:, 0])
