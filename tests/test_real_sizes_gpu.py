"""The float32 engine against the plain implementation at the layer sizes of real models: two layers of
Llama-3.2-1B's sizes (hidden 2,048, 32 heads of 64 on 8 kv heads, inner 8,192, vocabulary 128,256, tied head, llama3
rotary scaling with factor 32 over 8,192 positions) and one layer of Llama-3.1-8B's (hidden 4,096, heads of 128,
inner 14,336, a head of its own, factor 8).  The plain implementation runs in float64 (and in float32, for the
tolerance) with torch on the GPU: it is the yardstick, not the product.  One request of 301 tokens: whole, in
portions of changing size, and with its last 16 tokens decoded one by one.  Then the bfloat16 engine against the
same float64 logits.  A fault that the float32 and bfloat16 paths share at these sizes (the planner, block tables,
the FP32 product at 128,256 columns, the rotary bands) would show here and nowhere else."""

import numpy as np
import pytest
import torch

import cuttings
from plain_llama import PlainLlama, rope_inv_freq

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def config(sizes: str) -> dict:
    cfg = dict(architectures=["LlamaForCausalLM"], model_type="llama", num_hidden_layers=2, hidden_size=2048,
               num_attention_heads=32, num_key_value_heads=8, intermediate_size=8192, vocab_size=128256,
               rope_theta=500000.0, rope_scaling=dict(rope_type="llama3", factor=32.0, low_freq_factor=1.0,
                                                      high_freq_factor=4.0, original_max_position_embeddings=8192),
               rms_norm_eps=1e-5, tie_word_embeddings=True, max_position_embeddings=131072)
    if sizes == "8b":
        cfg.update(num_hidden_layers=1, hidden_size=4096, intermediate_size=14336, tie_word_embeddings=False)
        cfg["rope_scaling"] = dict(cfg["rope_scaling"], factor=8.0)
    return cfg


def replay(folder, dtype, steps):
    from tokasaurus_b200.engine.trace import TraceReplayer

    rp = TraceReplayer(str(folder), dtype, cuttings.max_live_tokens(steps), page_size=16, max_requests=4)
    outs = []
    for st in steps:
        outs.append(rp.run_step(st))
        rp.runner.cache.check()
    got = cuttings.collect(steps, outs)
    del rp
    torch.cuda.empty_cache()
    return got


@pytest.mark.parametrize("sizes", ["1b", "8b"])
def test_real_layer_sizes_against_plain(tmp_path, sizes):
    from tokasaurus_b200.parts import RotaryEncoding
    from tokasaurus_b200.weights import write_model_folder

    cfg = config(sizes)
    hd = cfg["hidden_size"] // cfg["num_attention_heads"]
    rs = cfg["rope_scaling"]
    # the real rotary settings: all three bands of the llama3 formula occur among the head's frequencies, and the
    # engine's inverse frequencies equal the plain formula's bit for bit
    plain_inv = rope_inv_freq(hd, cfg["rope_theta"], rs)
    base = rope_inv_freq(hd, cfg["rope_theta"], None)
    ratio = (base / plain_inv).numpy()
    assert (ratio == 1).any() and np.isclose(ratio, rs["factor"]).any() and ((ratio > 1.001) & (ratio < rs["factor"] * 0.999)).any()
    ours = RotaryEncoding(hd, cfg["rope_theta"], "llama3", rs["factor"], rs["low_freq_factor"], rs["high_freq_factor"],
                          rs["original_max_position_embeddings"]).inv_freq()
    assert torch.equal(ours.cpu().float(), plain_inv)

    folder = write_model_folder(tmp_path / sizes, cfg, seed=0, std=0.02, norm_init="uniform")
    toks = cuttings.random_tokens(301, cfg["vocab_size"], 77)
    reqs = {"a": toks}
    with torch.no_grad():
        p = PlainLlama(folder, torch.float64, DEV)
        p64 = {"a": p.logits(toks).cpu().numpy()}
        del p
        torch.cuda.empty_cache()
        p = PlainLlama(folder, torch.float32, DEV)
        p32 = {"a": p.logits(toks).double().cpu().numpy()}
        del p
        torch.cuda.empty_cache()
    tol32 = cuttings.tolerance("float32", p64["a"], p32["a"])
    cuts = dict(whole=cuttings.whole(reqs), portions=cuttings.changing_portions(reqs),
                decoded=cuttings.prefix_then_single(reqs, tail=16))
    for name, steps in cuts.items():
        got = replay(folder, "float32", steps)["a"]
        err = np.abs(got - p64["a"]).max(axis=1)
        bad = np.nonzero(err > tol32)[0]
        assert bad.size == 0, (f"float32 {sizes} {name}: first wrong token at position {bad[0]} (error {err[bad[0]]:.3g}, "
                               f"tolerance {tol32:.3g}, plain float32 spread {np.abs(p32['a'] - p64['a']).max():.3g})")
        srt = np.sort(p64["a"], axis=1)
        clear = (srt[:, -1] - srt[:, -2]) > 4 * tol32
        assert np.array_equal(got.argmax(1)[clear], p64["a"].argmax(1)[clear])
    tol16 = cuttings.tolerance("bfloat16", p64["a"])
    for name in ("whole", "decoded"):
        got = replay(folder, "bfloat16", cuts[name])["a"]
        err = np.abs(got - p64["a"]).max(axis=1)
        bad = np.nonzero(err > tol16)[0]
        assert bad.size == 0, (f"bfloat16 {sizes} {name}: first wrong token at position {bad[0]} (error {err[bad[0]]:.3g}, "
                               f"tolerance {tol16:.3g})")
