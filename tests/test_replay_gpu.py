"""Trace replay on the GPU against the plain implementation: the same requests whole, with the
last 32 tokens one by one, in portions of changing size, and mixed with other requests in a pool
so small that pages are used again; in float32 and in bfloat16."""

import json
import os
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

import cuttings
from plain_llama import TINY_WEIGHTS, tiny_configs

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


def requests_for(cfg_index: int) -> dict[str, list[int]]:
    cfg = tiny_configs()[cfg_index]
    lengths = [100, 37, 64, 5, 81, 128, 50] if cfg_index == 0 else [200, 1, 63, 100, 40, 256, 17]
    return {f"r{i}": cuttings.random_tokens(n, cfg["vocab_size"], 100 * cfg_index + i)
            for i, n in enumerate(lengths)}


def replay(model_dir, dtype, steps, page_size, max_tokens=None, max_requests=64):
    from tokasaurus_b200.engine.trace import TraceReplayer

    if max_tokens is None:
        max_tokens = cuttings.max_live_tokens(steps)
    rp = TraceReplayer(str(model_dir), dtype, max_tokens, page_size=page_size, max_requests=max_requests)
    outs = []
    for st in steps:
        outs.append(rp.run_step(st))
        rp.runner.cache.check()
    assert not rp.runner.cache.requests, "every request was ended, so nothing may be held"
    assert all(f == g.allocator.num_pages for f, g in zip(rp.runner.cache.num_free_pages(), rp.runner.cache.groups))
    return cuttings.collect(steps, outs)


def compare(got, want64, want32, dtype):
    for rid, ref in want64.items():
        tol = cuttings.tolerance(dtype, ref, want32[rid] if want32 else None)
        err = np.abs(got[rid] - ref).max(axis=1)
        bad = np.nonzero(err > tol)[0]
        assert bad.size == 0, (f"{dtype}: request {rid}: first wrong token at position {bad[0]} "
                               f"(error {err[bad[0]]:.3g}, tolerance {tol:.3g}); {bad.size} of {len(err)} wrong")
        if dtype == "float32":
            # same argmax wherever the plain implementation's top two are clearly apart
            srt = np.sort(ref, axis=1)
            clear = (srt[:, -1] - srt[:, -2]) > 4 * tol
            assert np.array_equal(got[rid].argmax(1)[clear], ref.argmax(1)[clear])


CUTS = {
    "whole": cuttings.whole,
    "prefix_then_single": cuttings.prefix_then_single,
    "changing_portions": cuttings.changing_portions,
    "mixed": cuttings.mixed,
}


@pytest.fixture(scope="module")
def plain(tiny_model_dirs):
    out = {}
    for i, d in enumerate(tiny_model_dirs):
        reqs = requests_for(i)
        out[i] = (reqs, cuttings.plain_logits(d, reqs, torch.float64), cuttings.plain_logits(d, reqs, torch.float32))
    return out


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("cut", list(CUTS))
@pytest.mark.parametrize("cfg_index", [0, 1])
def test_cuttings_match_plain(tiny_model_dirs, plain, cfg_index, cut, dtype):
    reqs, p64, p32 = plain[cfg_index]
    steps = CUTS[cut](reqs)
    got = replay(tiny_model_dirs[cfg_index], dtype, steps, TINY_WEIGHTS[cfg_index]["page_size"])
    compare(got, p64, p32, dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_cuttings_agree_with_each_other(tiny_model_dirs, plain, dtype):
    """The logits at a position do not depend on the cutting beyond rounding: compare the cuttings
    with one another, which is a tighter test in bfloat16 than the comparison with the plain
    implementation."""
    reqs, p64, _ = plain[1]
    base = replay(tiny_model_dirs[1], dtype, cuttings.whole(reqs), 8)
    for name in ("prefix_then_single", "changing_portions", "mixed"):
        got = replay(tiny_model_dirs[1], dtype, CUTS[name](reqs), 8)
        for rid in reqs:
            top = np.abs(p64[rid]).max()
            tol = (2e-5 if dtype == "float32" else 2e-2) * top
            err = np.abs(got[rid] - base[rid]).max(axis=1)
            bad = np.nonzero(err > tol)[0]
            assert bad.size == 0, f"{dtype} {name}: request {rid} first differs at position {bad[0]} ({err[bad[0]]:.3g})"


def test_mixed_pool_is_reused(tiny_model_dirs):
    """The mixed cutting must really hand pages out again."""
    from tokasaurus_b200.engine.trace import TraceReplayer

    reqs = requests_for(0)
    steps = cuttings.mixed(reqs)
    rp = TraceReplayer(str(tiny_model_dirs[0]), "float32", cuttings.max_live_tokens(steps), page_size=16)
    seen: dict[int, set] = {}
    for st in steps:
        rp.run_step(dict(st, end=[]))
        for rid, rc in rp.runner.cache.requests.items():
            for p in rc.tables[0]:
                seen.setdefault(p, set()).add(rid)
        for rid in st["end"]:
            rp.runner.cache.free(rid)
            del rp.lengths[rid]
    assert any(len(v) > 1 for v in seen.values()), "no page was used by two requests"


def test_trace_run_program(tiny_model_dirs, tmp_path):
    """bin/trace_run as a user calls it: JSON lines in, 'done <step>' lines and .f32 files out."""
    reqs = {k: v for k, v in list(requests_for(0).items())[:5]}
    steps = cuttings.mixed(reqs, seed=3)
    text = "\n".join(json.dumps(s) for s in steps) + "\n"
    out = tmp_path / "out"
    proc = subprocess.run(
        [sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(tiny_model_dirs[0]), "--dtype", "float32",
         "--out", str(out), "--max-tokens", str(cuttings.max_live_tokens(steps))],
        input=text, capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert proc.stdout.split("\n")[:-1] == [f"done {s['step']}" for s in steps]
    vocab = tiny_configs()[0]["vocab_size"]
    outs = []
    for s in steps:
        n = sum(len(e["want"]) for e in s["entries"])
        f = out / f"{s['step']}.f32"
        if n:
            a = np.fromfile(f, dtype="<f4")
            assert a.size == n * vocab
            outs.append(a.reshape(n, vocab))
        else:
            assert not f.exists()
            outs.append(None)
    got = cuttings.collect(steps, outs)
    p64 = cuttings.plain_logits(tiny_model_dirs[0], reqs, torch.float64)
    p32 = cuttings.plain_logits(tiny_model_dirs[0], reqs, torch.float32)
    compare(got, p64, p32, "float32")


def replay_through_graphs(model_dir, dtype, steps, page_size, max_seqs=8, graph_max=8, graph_step=4):
    """The steps of a cutting, each entry wanting the logits of its last token only (what generation asks of a
    step), run through the engine's CUDA graphs: decode graphs for steps of single tokens, graphs of the padded
    shape for steps with portions.  Returns {request: {position: logits}} and how many steps ran as graphs."""
    from tokasaurus_b200.engine.batch import StepEntry
    from tokasaurus_b200.engine.engine import Engine

    eng = Engine(model=str(model_dir), dtype=dtype, page_size=page_size, kv_cache_num_tokens=cuttings.max_live_tokens(steps),
                 max_seqs_per_forward=max_seqs, cudagraph_max_size=graph_max, cudagraph_step=graph_step,
                 graph_max_tokens=4096)
    cache, graphs = eng.runner.cache, eng.graphs
    lengths, got, n_graph = {}, {}, 0
    for st in steps:
        entries = []
        for e in st["entries"]:
            if e["id"] not in lengths:
                cache.admit(e["id"])
                lengths[e["id"]] = 0
            cache.ensure_capacity(e["id"], lengths[e["id"]] + len(e["tokens"]))
            entries.append(StepEntry(e["id"], list(e["tokens"]), lengths[e["id"]], [len(e["tokens"]) - 1]))
        R = len(entries)
        extra = dict(temperature=np.zeros(R, dtype=np.float32), stream_key=np.zeros(R, dtype=np.int64),
                     sample_pos=np.zeros(R, dtype=np.int32), row_slot=np.full(R, -1, dtype=np.int32))
        prep = None
        if graphs.usable(entries):
            prep = graphs.prepare(entries, extra)
        elif graphs.usable_general(entries):
            prep = graphs.prepare_general(entries, extra)
        if prep is not None:
            graphs.launch(prep)
            logits = graphs.graphs[prep["key"]]["logits"][:R].float().cpu().numpy()
            n_graph += 1
        else:
            logits = eng.runner.step(entries).float().cpu().numpy()
        eng.runner.check_status()
        for en, row in zip(entries, logits):
            lengths[en.request] += en.n_tokens
            got.setdefault(en.request, {})[lengths[en.request] - 1] = row
        for rid in st["end"]:
            cache.free(rid)
            del lengths[rid]
        cache.check()
    assert not cache.requests
    return got, n_graph


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("cut", ["prefix_then_single", "changing_portions", "mixed"])
@pytest.mark.parametrize("cfg_index", [0, 1])
def test_cuttings_through_step_graphs_match_plain(tiny_model_dirs, plain, cfg_index, cut, dtype):
    reqs, p64, p32 = plain[cfg_index]
    steps = CUTS[cut](reqs)
    got, n_graph = replay_through_graphs(tiny_model_dirs[cfg_index], dtype, steps, TINY_WEIGHTS[cfg_index]["page_size"])
    assert n_graph > len(steps) // 2
    for rid, ref in p64.items():
        tol = cuttings.tolerance(dtype, ref, p32[rid])
        for pos, row in got[rid].items():
            err = float(np.abs(row - ref[pos]).max())
            assert err <= tol, f"{dtype} {cut}: request {rid} position {pos}: error {err:.3g}, tolerance {tol:.3g}"


@pytest.mark.parametrize("hd", [64, 128])
def test_wide_heads_and_long_requests_match_plain(tmp_path, monkeypatch, hd):
    """Head sizes 64 and 128 in bfloat16 take the kernels that the tiny models' heads of 16 and 32 never reach:
    attention for portions on tcgen05, and whole tiles of keys by TMA in the split-key kernel, which needs
    work items of more than three tiles: the planner is told of a GPU that holds one block, so that it leaves
    requests of several hundred tokens whole.  Whole, decoded at the end, in portions, mixed, and the decoded
    tail through the step graphs (rotation and cache write inside the attention kernel)."""
    import tokasaurus_b200.parts.attention as attention
    from tokasaurus_b200.weights import write_model_folder

    monkeypatch.setattr(attention, "decode_block_slots", lambda head_dim, limits=None: 1)
    cfg = dict(architectures=["LlamaForCausalLM"], model_type="llama", num_hidden_layers=2, hidden_size=2 * hd,
               num_attention_heads=2, num_key_value_heads=1, intermediate_size=96, vocab_size=300, rope_theta=10000.0,
               rope_scaling=None, rms_norm_eps=1e-5, tie_word_embeddings=True, max_position_embeddings=1024)
    d = write_model_folder(tmp_path / "wide", cfg, seed=3, std=0.05, norm_init="uniform")
    reqs = {f"w{i}": cuttings.random_tokens(n, 300, 500 + i) for i, n in enumerate([700, 289, 513, 64])}
    p64 = cuttings.plain_logits(d, reqs, torch.float64)
    for cut in ("whole", "prefix_then_single", "changing_portions", "mixed"):
        steps = CUTS[cut](reqs)
        compare(replay(d, "bfloat16", steps, 16), p64, None, "bfloat16")
    steps = cuttings.prefix_then_single(reqs)
    got, n_graph = replay_through_graphs(d, "bfloat16", steps, 16)
    assert n_graph > len(steps) // 2
    for rid, ref in p64.items():
        tol = cuttings.tolerance("bfloat16", ref, None)
        for pos, row in got[rid].items():
            err = float(np.abs(row - ref[pos]).max())
            assert err <= tol, f"request {rid} position {pos}: error {err:.3g}, tolerance {tol:.3g}"


def many_requests(n: int, vocab: int, longest: int, seed: int) -> dict[str, list[int]]:
    """2 * n requests (two waves of n) whose lengths cross page edges and the 64-key tiles of the attention kernels
    while their last six tokens are decoded."""
    rng = np.random.default_rng(seed)
    edges = [7, 8, 9, 15, 17, 62, 64, 66, 68, 70, 126, 128, 131, 133, 190, 193, 255, 256]
    lengths = [e for e in edges if e <= longest] + [int(x) for x in rng.integers(7, longest + 1, size=2 * n)]
    rng.shuffle(lengths)
    return {f"m{i}": cuttings.random_tokens(lengths[i], vocab, seed * 1000 + i) for i in range(2 * n)}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("n", [20, 33, 64, 65, 128])
def test_decode_steps_of_many_requests_match_plain(tiny_model_dirs, n, dtype):
    """Decode steps of 20, 33, 64, 65 and 128 single-token requests (in bfloat16: the tcgen05 small-batch products
    whose slices the attention kernel adds from 17 rows on, the library products with the separate rotary kernel from
    65 on, graphs padded from 20 to 32, 33 to 48, 65 to 80 rows), eagerly and through the step graphs with the
    reference's default graph sizes (step 16 up to 128), two waves in a pool that holds one."""
    d, cfg = tiny_model_dirs[1], tiny_configs()[1]
    reqs = many_requests(n, cfg["vocab_size"], 250, n)
    p64 = cuttings.plain_logits(d, reqs, torch.float64)
    p32 = cuttings.plain_logits(d, reqs, torch.float32) if dtype == "float32" else None
    steps = cuttings.waves_of_decoding(reqs, n)
    assert max(len(st["entries"]) for st in steps) == n
    compare(replay(d, dtype, steps, 8, max_requests=128), p64, p32, dtype)
    got, n_graph = replay_through_graphs(d, dtype, steps, 8, max_seqs=128, graph_max=128, graph_step=16)
    assert n_graph >= 12  # every decode step of both waves
    for rid, ref in p64.items():
        tol = cuttings.tolerance(dtype, ref, p32[rid] if p32 else None)
        for pos, row in got[rid].items():
            err = float(np.abs(row - ref[pos]).max())
            assert err <= tol, f"{dtype} n={n}: request {rid} position {pos}: error {err:.3g}, tolerance {tol:.3g}"


@pytest.mark.parametrize("n", [20, 64, 65, 128])
@pytest.mark.parametrize("hd", [64, 128])
def test_decode_steps_of_many_requests_wide_heads(tmp_path, n, hd):
    """The same with heads of 64 and 128 in bfloat16: whole tiles of keys by TMA, four query heads a kv head."""
    from tokasaurus_b200.weights import write_model_folder

    cfg = dict(architectures=["LlamaForCausalLM"], model_type="llama", num_hidden_layers=2, hidden_size=4 * hd,
               num_attention_heads=4, num_key_value_heads=1, intermediate_size=96, vocab_size=300, rope_theta=10000.0,
               rope_scaling=None, rms_norm_eps=1e-5, tie_word_embeddings=True, max_position_embeddings=1024)
    d = write_model_folder(tmp_path / "wide", cfg, seed=4, std=0.04, norm_init="uniform")
    reqs = many_requests(n, 300, 420, 7 * n + hd)
    p64 = cuttings.plain_logits(d, reqs, torch.float64)
    steps = cuttings.waves_of_decoding(reqs, n)
    compare(replay(d, "bfloat16", steps, 16, max_requests=128), p64, None, "bfloat16")
    got, n_graph = replay_through_graphs(d, "bfloat16", steps, 16, max_seqs=128, graph_max=128, graph_step=16)
    assert n_graph >= 12
    for rid, ref in p64.items():
        tol = cuttings.tolerance("bfloat16", ref, None)
        for pos, row in got[rid].items():
            err = float(np.abs(row - ref[pos]).max())
            assert err <= tol, f"hd={hd} n={n}: request {rid} position {pos}: error {err:.3g}, tolerance {tol:.3g}"
