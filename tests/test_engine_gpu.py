"""The engine on the GPU through its Python entry point and command line: greedy generation,
chunked prefill beside decoding, requests pushed out for lack of pages, temperature sampling,
long decoding and the first tokens of a sequence."""

import json
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

import cuttings
from plain_llama import PlainLlama, TINY_WEIGHTS, tiny_configs

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


def make_engine(model_dir, **kw):
    from tokasaurus_b200.engine.engine import Engine

    opts = dict(dtype="float32", kv_cache_num_tokens=2048, allocator_sanity_checks=True)
    opts.update(kw)
    return Engine(model=str(model_dir), **opts)


def near_best(plain, prompt, completion, frac=0.03):
    logits = plain.logits(prompt + completion[:-1])[len(prompt) - 1:]
    top = logits.abs().max().item()
    return all(logits[i, t] >= logits[i].max() - frac * top for i, t in enumerate(completion))


@pytest.mark.parametrize("cfg_index", [0, 1])
def test_greedy_generation_float32_equals_plain(tiny_model_dirs, cfg_index):
    d = tiny_model_dirs[cfg_index]
    vocab = tiny_configs()[cfg_index]["vocab_size"]
    lengths = (5, 17, 32) if cfg_index == 0 else (1, 40, 63, 100)
    prompts = [cuttings.random_tokens(n, vocab, 40 + n) for n in lengths]
    plain = PlainLlama(d, torch.float64)
    want = [plain.greedy(p, 16) for p in prompts]
    eng = make_engine(d, page_size=TINY_WEIGHTS[cfg_index]["page_size"])
    outs = eng.generate(prompts, max_num_tokens=16, ignore_eos=True)
    assert [o.completion_ids for o in outs] == want
    # chunked prefill (24 tokens a step) mixed with decoding gives the same tokens
    eng2 = make_engine(d, page_size=TINY_WEIGHTS[cfg_index]["page_size"], max_tokens_per_forward=24)
    outs2 = eng2.generate(prompts, max_num_tokens=16, ignore_eos=True)
    assert [o.completion_ids for o in outs2] == want
    for o, o2 in zip(outs, outs2):
        np.testing.assert_allclose(o.logprobs, o2.logprobs, atol=1e-4)
    assert not eng2.runner.cache.requests


@pytest.mark.parametrize("cfg_index", [0, 1])
def test_greedy_generation_bfloat16(tiny_model_dirs, cfg_index):
    d = tiny_model_dirs[cfg_index]
    vocab = tiny_configs()[cfg_index]["vocab_size"]
    prompts = [cuttings.random_tokens(n, vocab, 90 + n) for n in (3, 29, 64)]
    plain = PlainLlama(d, torch.float64)
    eng = make_engine(d, dtype="bfloat16", page_size=TINY_WEIGHTS[cfg_index]["page_size"], max_tokens_per_forward=40)
    outs = eng.generate(prompts, max_num_tokens=20, ignore_eos=True)
    for p, o in zip(prompts, outs):
        assert len(o.completion_ids) == 20 and near_best(plain, p, o.completion_ids)


def test_pushed_out_requests_give_the_same_tokens(tiny_model_dirs):
    d = tiny_model_dirs[0]
    prompts = [cuttings.random_tokens(n, 256, 11 * n) for n in (30, 28, 31, 20)]
    plain = PlainLlama(d, torch.float64)
    want = [plain.greedy(p, 20) for p in prompts]
    eng = make_engine(d, kv_cache_num_tokens=128, bump_city_population_me=True)
    outs = eng.generate(prompts, max_num_tokens=20, ignore_eos=True)
    assert eng.scheduler.stats["bumps"] > 0
    assert [o.completion_ids for o in outs] == want


@pytest.mark.parametrize("seed", [0, 1])
def test_random_arrivals_in_a_small_pool_every_way_of_running(tiny_model_dirs, seed):
    """Thirty requests of random lengths and limits, some with stop tokens, arriving at random steps into a pool
    of 128 tokens, which holds a few of them at a time: worst-case reserve, no reserve (requests are pushed out and fed again) and
    admission by simulation; with step graphs and three steps of run-ahead, and without either.  Greedy float32
    tokens equal the plain implementation's every time, and every page and slot comes back."""
    import random
    from tokasaurus_b200 import SamplingParams

    cfg_index = seed % 2
    d = tiny_model_dirs[cfg_index]
    vocab = PlainLlama(d).cfg["vocab_size"]
    page = TINY_WEIGHTS[cfg_index]["page_size"]
    rng = random.Random(100 + seed)
    reqs = [(cuttings.random_tokens(rng.randint(1, 70), vocab, 1000 * seed + i), rng.randint(1, 25)) for i in range(30)]
    plain = PlainLlama(d, torch.float64)
    full = [plain.greedy(p, m) for p, m in reqs]
    stops, want = [], []
    for i, f in enumerate(full):
        if i % 4 == 0 and len(f) > 3:  # stops where it first produces its fourth token
            stops.append([f[3]])
            want.append(f[: f.index(f[3]) + 1])
        else:
            stops.append([])
            want.append(f)
    arrive = sorted(rng.randint(0, 40) for _ in reqs)
    ways = [dict(), dict(bump_city_population_me=True), dict(admission="simulate"),
            dict(use_cudagraphs=False, scheduling_steps_ahead=0, bump_city_population_me=True),
            dict(scheduling_steps_ahead=3, admission="simulate", greedy_prefill=False, prefill_round_up_multiple=4)]
    for way in ways:
        eng = make_engine(d, page_size=page, kv_cache_num_tokens=128, max_seqs_per_forward=6,
                          max_tokens_per_forward=48, cudagraph_max_size=8, cudagraph_step=4,
                          **{"scheduling_steps_ahead": 3, **way})
        ids, done, step, nxt = [], [], 0, 0
        while nxt < len(reqs) or eng.has_work():
            while nxt < len(reqs) and arrive[nxt] <= step:
                p, m = reqs[nxt]
                ids.append(eng.add_request(p, SamplingParams(), max_num_tokens=m, ignore_eos=True,
                                           stop_token_ids=stops[nxt]))
                nxt += 1
            if eng.has_work():
                done += eng.step()
            step += 1
        by_id = {o.id: o for o in done}
        assert [by_id[i].completion_ids for i in ids] == want, f"way {way}"
        assert not eng.runner.cache.requests and not eng.has_work()
        assert eng.runner.cache.num_free_pages() == [g.allocator.num_pages for g in eng.runner.cache.groups]
        if way.get("bump_city_population_me"):
            assert eng.scheduler.stats["bumps"] > 0, f"way {way}: the pool was meant to be too small"


def test_temperature_sampling_seeded(tiny_model_dirs):
    from tokasaurus_b200 import SamplingParams

    d = tiny_model_dirs[1]
    prompts = [cuttings.random_tokens(n, 509, n) for n in (1, 40, 63, 100)]
    sp = SamplingParams(temperature=0.7, seed=7)
    a = make_engine(d, page_size=8, max_tokens_per_forward=24).generate(prompts, sp, max_num_tokens=20, ignore_eos=True)
    b = make_engine(d, page_size=8).generate(prompts, sp, max_num_tokens=20, ignore_eos=True)
    assert [o.completion_ids for o in a] == [o.completion_ids for o in b]
    c = make_engine(d, page_size=8).generate(prompts, SamplingParams(temperature=0.7, seed=8), max_num_tokens=20,
                                             ignore_eos=True)
    assert [o.completion_ids for o in a] != [o.completion_ids for o in c]
    # the sampled tokens have the log-probabilities the plain implementation gives them at T = 0.7
    plain = PlainLlama(d, torch.float64)
    o = a[1]
    logits = plain.logits(prompts[1] + o.completion_ids[:-1])[len(prompts[1]) - 1:]
    lp = torch.log_softmax(logits / 0.7, -1)
    want = [lp[i, t].item() for i, t in enumerate(o.completion_ids)]
    np.testing.assert_allclose(o.logprobs, want, atol=2e-4)
    assert len(set(o.completion_ids)) > 3


def test_topk_logprobs_through_the_entry_point(tiny_model_dirs):
    d = tiny_model_dirs[0]
    p = cuttings.random_tokens(9, 256, 1)
    eng = make_engine(d, max_topk_logprobs=4)
    o = eng.generate([p], max_num_tokens=5, ignore_eos=True, topk_logprobs=3)[0]
    assert len(o.topk_ids) == 5 and all(len(t) == 3 for t in o.topk_ids)
    for t, ids, lps, lp in zip(o.completion_ids, o.topk_ids, o.topk_logprobs, o.logprobs):
        assert ids[0] == t and abs(lps[0] - lp) < 1e-5 and lps == sorted(lps, reverse=True)
    with pytest.raises(ValueError):
        eng.add_request(p, topk_logprobs=9)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding(tiny_model_dirs, dtype):
    """A short prompt and then 248 single-token steps up to the model's last position."""
    from test_replay_gpu import compare, replay

    d = tiny_model_dirs[1]
    reqs = {"long": cuttings.random_tokens(256, 509, 77)}
    steps = cuttings.prefix_then_single(reqs, tail=248)
    got = replay(d, dtype, steps, 8)
    compare(got, cuttings.plain_logits(d, reqs), cuttings.plain_logits(d, reqs, torch.float32), dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_first_tokens_of_a_sequence(tiny_model_dirs, dtype):
    """Positions 0, 1, 2: one token alone; two tokens; a token, then a token, then a token."""
    from test_replay_gpu import compare, replay

    for i, d in enumerate(tiny_model_dirs):
        vocab = tiny_configs()[i]["vocab_size"]
        reqs = {"a": cuttings.random_tokens(1, vocab, 1), "b": cuttings.random_tokens(2, vocab, 2),
                "c": cuttings.random_tokens(3, vocab, 3)}
        p64, p32 = cuttings.plain_logits(d, reqs), cuttings.plain_logits(d, reqs, torch.float32)
        for cut in (cuttings.whole, lambda r: cuttings.prefix_then_single(r, tail=2)):
            compare(replay(d, dtype, cut(reqs), TINY_WEIGHTS[i]["page_size"]), p64, p32, dtype)


def test_command_line(tiny_model_dirs, tmp_path):
    d = tiny_model_dirs[0]
    p = cuttings.random_tokens(12, 256, 5)
    want = PlainLlama(d, torch.float64).greedy(p, 6)
    proc = subprocess.run([sys.executable, str(ROOT / "bin" / "toka"), f"model={d}", "dtype=float32",
                           "kv_cache_num_tokens=(16*64)", f"prompt_ids={json.dumps(p)}", "max_num_tokens=6",
                           "ignore_eos=T"], capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    rec = json.loads(proc.stdout.strip().split("\n")[-1])
    assert rec["completion_ids"] == want and rec["finish_reason"] == "length"
    bad = subprocess.run([sys.executable, str(ROOT / "bin" / "toka"), f"model={d}", "nonsense=1"], capture_output=True,
                         text=True, timeout=120)
    assert bad.returncode == 2 and "unknown option" in bad.stderr
    # the options of the command that reach the scheduler: two prompts, a reserve, a deeper run-ahead
    q = cuttings.random_tokens(7, 256, 6)
    proc = subprocess.run([sys.executable, str(ROOT / "bin" / "toka"), f"model={d}", "dtype=float32",
                           "kv_cache_num_tokens=(16*64)", f"prompt_ids={json.dumps([p, q])}", "max_num_tokens=6",
                           "ignore_eos=T", "admission=reserve", "kv_reserve_fraction=0.5", "scheduling_steps_ahead=4"],
                          capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    recs = [json.loads(line) for line in proc.stdout.strip().split("\n")[-2:]]
    assert recs[0]["completion_ids"] == want and recs[1]["completion_ids"] == PlainLlama(d, torch.float64).greedy(q, 6)
    bad = subprocess.run([sys.executable, str(ROOT / "bin" / "toka"), f"model={d}", f"prompt_ids={json.dumps(p)}",
                          "admission=hopeful"], capture_output=True, text=True, timeout=120)
    assert bad.returncode != 0 and "admission" in bad.stderr


def test_bad_token_id_is_refused_on_the_host(tiny_model_dirs):
    eng = make_engine(tiny_model_dirs[0])
    with pytest.raises(ValueError, match="vocabulary"):
        eng.add_request([1, 2, 256])


def test_no_cuda_no_engine(tiny_model_dirs):
    from tokasaurus_b200.engine.engine import Engine

    with pytest.raises(RuntimeError, match="no CPU execution path"):
        Engine(model=str(tiny_model_dirs[0]), device="cpu")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_cuda_graph_decode_equals_eager(tiny_model_dirs, dtype):
    """Decode steps replayed from CUDA graphs give the tokens and log-probabilities of the eager
    path, over batch sizes that need padding and contexts that cross pages and work-list capacities."""
    from tokasaurus_b200 import SamplingParams

    d = tiny_model_dirs[1]
    prompts = [cuttings.random_tokens(n, 509, 5 * n) for n in (7, 30, 64, 3, 12)]
    sp = [SamplingParams(temperature=t, seed=3) for t in (0.0, 0.8, 0.0, 1.2, 0.0)]
    outs = {}
    for graphs in (False, True):
        # prompt steps launched kernel by kernel in both runs (their graphs have tests of their own): with the same
        # kernels on the same shapes the two runs agree bit for bit, so sampled tokens cannot part ways
        eng = make_engine(d, dtype=dtype, page_size=8, use_cudagraphs=graphs, cudagraph_step=4, cudagraph_max_size=8,
                          graph_max_tokens=0)
        outs[graphs] = eng.generate(prompts, sp, max_num_tokens=40, ignore_eos=True)
        if graphs:
            assert eng.graphs is not None and len(eng.graphs.graphs) >= 1
            assert not eng.runner.cache.requests
    for a, b in zip(outs[False], outs[True]):
        assert a.completion_ids == b.completion_ids
        np.testing.assert_allclose(a.logprobs, b.logprobs, atol=1e-5)


def test_cuda_graph_decode_with_requests_ending_at_different_times(tiny_model_dirs):
    """Requests that end by length at different steps and on stop tokens, and late arrivals: the engine launches
    the next steps (one, two, five of them) before it has read the current one, on a guess that is wrong again and
    again; the rows of requests that had ended after all must be dropped, with and without that run-ahead."""
    from tokasaurus_b200 import SamplingParams

    d = tiny_model_dirs[0]
    prompts = [cuttings.random_tokens(n, 256, 9 * n) for n in (7, 30, 64, 3, 12, 20)]
    limits = [5, 17, 40, 2, 33, 1]
    plain = PlainLlama(d, torch.float64)
    full = [plain.greedy(p, m) for p, m in zip(prompts, limits)]
    stop_at = full[2][9]  # request 2 stops when it first produces this token
    want = [list(f) for f in full]
    want[2] = full[2][: full[2].index(stop_at) + 1]
    for graphs, ahead in ((False, 1), (True, 0), (True, 1), (True, 2), (True, 5)):
        eng = make_engine(d, use_cudagraphs=graphs, cudagraph_step=4, cudagraph_max_size=8, scheduling_steps_ahead=ahead)
        assert eng.steps_ahead == ahead
        ids = []
        for i, (p, m) in enumerate(zip(prompts[:4], limits[:4])):
            ids.append(eng.add_request(p, SamplingParams(), max_num_tokens=m, ignore_eos=True,
                                       stop_token_ids=[stop_at] if i == 2 else ()))
        done = []
        for _ in range(6):
            done += eng.step()
        for p, m in zip(prompts[4:], limits[4:]):  # arrivals while the others decode
            ids.append(eng.add_request(p, SamplingParams(), max_num_tokens=m, ignore_eos=True))
        done += eng.run_until_done()
        by_id = {o.id: o for o in done}
        assert [by_id[i].completion_ids for i in ids] == want, f"graphs={graphs} steps ahead={ahead}"
        assert by_id[ids[2]].finish_reason == "stop"
        assert not eng.runner.cache.requests and not eng.has_work()


def test_run_ahead_with_stop_tokens_under_sampling(tiny_model_dirs):
    """Several requests with temperature sampling that stop on tokens at different steps: the same outputs with
    and without the run-ahead, and every page given back."""
    from tokasaurus_b200 import SamplingParams

    d = tiny_model_dirs[1]
    prompts = [cuttings.random_tokens(n, 509, 3 * n + 1) for n in (9, 31, 5, 18, 2)]
    sp = [SamplingParams(temperature=t, seed=11 + i) for i, t in enumerate((0.9, 0.0, 1.1, 0.7, 0.0))]
    ref = make_engine(d, dtype="bfloat16", page_size=8, run_ahead=False).generate(prompts, sp, max_num_tokens=30, ignore_eos=True)
    stops = [[o.completion_ids[4 + 3 * i]] for i, o in enumerate(ref)]
    outs = {}
    deepest = 0
    for ahead in (0, 1, 3):
        eng = make_engine(d, dtype="bfloat16", page_size=8, scheduling_steps_ahead=ahead)
        ids = [eng.add_request(p, s, max_num_tokens=30, ignore_eos=True, stop_token_ids=st)
               for p, s, st in zip(prompts, sp, stops)]
        done = []
        while eng.has_work():
            done += eng.step()
            deepest = max(deepest, len(eng._inflight)) if ahead == 3 else deepest
        by_id = {o.id: o for o in done}
        outs[ahead] = [by_id[i] for i in ids]
        assert not eng.runner.cache.requests and not eng.has_work()
    assert deepest == 3  # three steps were in flight beyond the one being read
    for a, b, c, r, st in zip(outs[0], outs[1], outs[3], ref, stops):
        assert a.completion_ids == b.completion_ids == c.completion_ids
        assert a.finish_reason == b.finish_reason == c.finish_reason == "stop"
        assert a.completion_ids == r.completion_ids[: r.completion_ids.index(st[0]) + 1]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_graphs_of_steps_with_prompt_portions_equal_eager(tiny_model_dirs, dtype):
    """Steps that mix prompt portions (cut by a small token budget) with decoded tokens, replayed from CUDA graphs
    of their padded shape, against the same steps launched kernel by kernel; arrivals while others decode,
    requests ending at different times.  float32: the same tokens and log-probabilities (its products add in the
    same order whatever the padding).  bfloat16: library products pick their kernel by the padded row count, so
    the runs agree to rounding; greedy tokens of both must be (nearly) the best under the plain model."""
    from tokasaurus_b200 import SamplingParams

    d = tiny_model_dirs[1]
    prompts = [cuttings.random_tokens(n, 509, 11 * n + 2) for n in (7, 30, 64, 3, 12, 45, 2)]
    temps = (0.0, 0.8, 0.0, 1.2, 0.0, 0.6, 0.0) if dtype == "float32" else (0.0,) * 7
    sp = [SamplingParams(temperature=t, seed=5) for t in temps]
    limits = [9, 25, 14, 3, 30, 1, 18]
    outs = {}
    for max_tokens in (0, 1024):
        eng = make_engine(d, dtype=dtype, page_size=8, max_tokens_per_forward=20, cudagraph_step=4, cudagraph_max_size=8,
                          graph_max_tokens=max_tokens)
        ids = [eng.add_request(p, s, max_num_tokens=m, ignore_eos=True) for p, s, m in zip(prompts[:4], sp, limits)]
        done = []
        for _ in range(5):
            done += eng.step()
        ids += [eng.add_request(p, s, max_num_tokens=m, ignore_eos=True)
                for p, s, m in zip(prompts[4:], sp[4:], limits[4:])]
        done += eng.run_until_done()
        by_id = {o.id: o for o in done}
        outs[max_tokens] = [by_id[i] for i in ids]
        assert not eng.runner.cache.requests and not eng.has_work()
        general = [k for k in eng.graphs.graphs if k[0] == "general"]
        assert bool(general) == bool(max_tokens)
    if dtype == "float32":
        for a, b, m in zip(outs[0], outs[1024], limits):
            assert a.completion_ids == b.completion_ids and len(a.completion_ids) == m
            np.testing.assert_allclose(a.logprobs, b.logprobs, atol=1e-5)
    else:
        plain = PlainLlama(d, torch.float64)
        for mode in (0, 1024):
            for o, p, m in zip(outs[mode], prompts, limits):
                assert len(o.completion_ids) == m and near_best(plain, p, o.completion_ids), mode


def test_everything_at_once_equals_the_plain_path(tiny_model_dirs):
    """Twenty requests of random lengths arriving over time into a pool so tight that requests are pushed out,
    some ending on stop tokens, some sampled with a temperature: with CUDA graphs for decode steps and for steps
    with prompt portions and with the run-ahead, the engine gives, in float32, exactly what it gives with all of
    that switched off."""
    from tokasaurus_b200 import SamplingParams

    d = tiny_model_dirs[1]
    rng = np.random.default_rng(4)
    prompts = [cuttings.random_tokens(int(n), 509, 1000 + i) for i, n in enumerate(rng.integers(1, 90, size=20))]
    limits = [int(x) for x in rng.integers(1, 40, size=20)]
    temps = [float(t) for t in rng.choice([0.0, 0.0, 0.7, 1.3], size=20)]
    arrive = sorted(int(x) for x in rng.integers(0, 60, size=20))
    outs = {}
    stops = None
    for fancy in (False, True):
        eng = make_engine(d, page_size=8, kv_cache_num_tokens=256, max_tokens_per_forward=48, max_seqs_per_forward=6,
                          kv_reserve_fraction=0.0, use_cudagraphs=fancy, cudagraph_step=2, cudagraph_max_size=6,
                          run_ahead=fancy, graph_max_tokens=1024 if fancy else 0)
        if stops is None:
            # stop tokens taken from an unconstrained run of every fourth request, so that they are really met
            probe = make_engine(d, page_size=8, kv_cache_num_tokens=4096, use_cudagraphs=False)
            full = probe.generate(prompts, [SamplingParams(temperature=t, seed=9) for t in temps], max_num_tokens=40,
                                  ignore_eos=True)
            stops = [[o.completion_ids[min(len(o.completion_ids) - 1, 5)]] if i % 4 == 0 else [] for i, o in enumerate(full)]
        ids, done, step, nxt = [], [], 0, 0
        while nxt < len(prompts) or eng.has_work():
            while nxt < len(prompts) and arrive[nxt] <= step:
                ids.append(eng.add_request(prompts[nxt], SamplingParams(temperature=temps[nxt], seed=9),
                                           max_num_tokens=limits[nxt], ignore_eos=True, stop_token_ids=stops[nxt]))
                nxt += 1
            done += eng.step()
            step += 1
            assert step < 5000
        by_id = {o.id: o for o in done}
        outs[fancy] = [by_id[i] for i in ids]
        assert not eng.runner.cache.requests and not eng.has_work()
        if fancy:
            assert eng.scheduler.stats["bumps"] > 0 and any(k[0] == "general" for k in eng.graphs.graphs)
    for a, b in zip(outs[False], outs[True]):
        assert a.completion_ids == b.completion_ids and a.finish_reason == b.finish_reason
        np.testing.assert_allclose(a.logprobs, b.logprobs, atol=1e-5)
    assert any(o.finish_reason == "stop" for o in outs[True]) and any(o.finish_reason == "length" for o in outs[True])


def test_warm_up_records_the_decode_graphs(tiny_model_dirs):
    """After ``warm_up`` decoding records nothing more, and the tokens are those of an engine that was not warmed."""
    d = tiny_model_dirs[0]
    prompts = [cuttings.random_tokens(n, 256, 3 * n) for n in (5, 17, 32)]
    cold = make_engine(d, graph_max_tokens=0)
    want = [o.completion_ids for o in cold.generate(prompts, max_num_tokens=12, ignore_eos=True)]
    eng = make_engine(d, graph_max_tokens=0, max_seqs_per_forward=8, cudagraph_step=4, cudagraph_max_size=8)
    made = eng.warm_up()
    assert made == len(eng.graphs.sizes) == len(eng.graphs.graphs) and not eng.runner.cache.requests
    eng.runner.cache.check()
    assert [o.completion_ids for o in eng.generate(prompts, max_num_tokens=12, ignore_eos=True)] == want
    assert len(eng.graphs.graphs) == made
    with pytest.raises(RuntimeError):
        eng.add_request(prompts[0], max_num_tokens=4)
        eng.warm_up()
    # bfloat16: the attention picks its kernel by the length of the step's work items, so each batch size is
    # recorded twice, at a short and at a long context, and decoding at either records nothing more
    eng = make_engine(d, dtype="bfloat16", graph_max_tokens=0, max_seqs_per_forward=8, cudagraph_step=4, cudagraph_max_size=8,
                      kv_cache_num_tokens=8 * 16384)  # this model's items pass three tiles only at contexts of 16,384
    made = eng.warm_up()
    assert made == 2 * len(eng.graphs.sizes) == len(eng.graphs.graphs) and not eng.runner.cache.requests
    eng.runner.cache.check()
    eng.generate(prompts, max_num_tokens=12, ignore_eos=True)
    eng.generate([cuttings.random_tokens(100, 256, 5)] * 3, max_num_tokens=20, ignore_eos=True)
    assert len(eng.graphs.graphs) == made


@pytest.mark.parametrize("sizes", ["1b", "8b"])
def test_llama_layer_sizes_bfloat16_against_float32(sizes):
    """Two layers of the sizes the benchmark runs (hidden 2,048, 32 heads of 64 on 8 kv heads, inner 8,192,
    vocabulary 128,256), or one layer of Llama-3.1-8B's (hidden 4,096, 32 heads of 128 on 8 kv heads, inner
    14,336; vocabulary 32,000, untied), random weights: the bfloat16 path (tcgen05 attention and gate/up product for the
    prompts, K-split products, fused rotary + split-key attention with TMA tiles and the step graph for the
    decoded tokens) against the float32 path of the same engine, which the tiny models tie to the plain
    implementation.  Eight prompts of about 1,800 tokens, so that the split-key kernel gets work items of four
    tiles; then five decoded tokens each (the float32 path's greedy choice is fed to both)."""
    from tokasaurus_b200.engine.batch import StepEntry
    from tokasaurus_b200.engine.engine import Engine

    cfg = dict(architectures=["LlamaForCausalLM"], model_type="llama", num_hidden_layers=2, hidden_size=2048,
               num_attention_heads=32, num_key_value_heads=8, intermediate_size=8192, vocab_size=128256,
               rope_theta=500000.0, rope_scaling=dict(rope_type="llama3", factor=32.0, low_freq_factor=1.0,
                                                      high_freq_factor=4.0, original_max_position_embeddings=8192),
               rms_norm_eps=1e-5, tie_word_embeddings=True, max_position_embeddings=131072)
    if sizes == "8b":
        cfg.update(num_hidden_layers=1, hidden_size=4096, intermediate_size=14336, vocab_size=32000,
                   tie_word_embeddings=False)
    lengths = [1850, 1787, 1740, 1861, 1826, 1752, 1905, 1810]
    prompts = [cuttings.random_tokens(n, cfg["vocab_size"], 900 + i) for i, n in enumerate(lengths)]
    ids = [f"p{i}" for i in range(len(prompts))]

    def run(dtype, feed=None):
        eng = Engine(config_dict=cfg, random_weights=0, dtype=dtype, page_size=16, kv_cache_num_tokens=8 * 2048,
                     max_tokens_per_forward=8192, max_seqs_per_forward=8)
        runner, cache = eng.runner, eng.runner.cache
        rows = []  # [step][request] -> logits
        for rid, p in zip(ids, prompts):
            cache.admit(rid)
            cache.ensure_capacity(rid, len(p) + 6)
        first = []
        for half in (slice(0, 4), slice(4, 8)):
            entries = [StepEntry(rid, p, 0, [len(p) - 1]) for rid, p in zip(ids[half], prompts[half])]
            first.append(runner.step(entries).float().cpu())
        rows.append(torch.cat(first))
        for t in range(5):
            tokens = rows[-1].argmax(-1).tolist() if feed is None else feed[t]
            entries = [StepEntry(rid, [tok], len(p) + t, [0]) for rid, p, tok in zip(ids, prompts, tokens)]
            R = len(entries)
            extra = dict(temperature=np.zeros(R, dtype=np.float32), stream_key=np.zeros(R, dtype=np.int64),
                         sample_pos=np.zeros(R, dtype=np.int32), row_slot=np.full(R, -1, dtype=np.int32))
            if dtype == "bfloat16" and eng.graphs is not None and eng.graphs.usable(entries):
                prep = eng.graphs.prepare(entries, extra)
                assert int(prep["plans"][next(iter(prep["plans"]))]["counts"][5]) == 1, "work items of four tiles expected"
                eng.graphs.launch(prep)
                rows.append(eng.graphs.graphs[prep["key"]]["logits"][:R].float().cpu())
            else:
                rows.append(runner.step(entries).float().cpu())
        runner.check_status()
        return rows

    want = run("float32")
    feed = [w.argmax(-1).tolist() for w in want[:-1]]
    got = run("bfloat16", feed)
    for t, (g, w) in enumerate(zip(got, want)):
        tol = 0.03 * w.abs().max().item()
        err = (g - w).abs().max(dim=1).values
        print(f"step {t}: largest error {err.max().item():.3g} of max |logit| {w.abs().max().item():.3g} (tolerance {tol:.3g})")
        assert (err <= tol).all(), f"step {t}: largest error {err.max().item():.3g}, tolerance {tol:.3g}, rows {err.tolist()}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_page_id_beyond_the_pool_is_refused_not_read(tiny_model_dirs, dtype):
    """A block table that names a page beyond the pool (a fault of the host's books): the kernels that read keys
    through it, not only those that write, skip the access, zeros stand in, and the step's status check raises."""
    from tokasaurus_b200.engine.runner import DeviceStatusError
    from tokasaurus_b200.engine.trace import TraceReplayer

    toks = cuttings.random_tokens(40, 256, 5)
    rp = TraceReplayer(str(tiny_model_dirs[0]), dtype, 256, page_size=16)
    rp.run_step(dict(step=0, entries=[dict(id="a", tokens=toks[:20], want=[19])], end=[]))
    rc = rp.runner.cache.requests["a"]
    good = rc.tables[0][0]
    rc.tables[0][0] = rp.runner.cache.num_pages + 5  # the page that holds keys 0..15, which every later query reads
    rc.arrays.clear()
    for step, chunk in ((1, toks[20:33]), (2, toks[33:34])):  # a portion, then a single token
        with pytest.raises(DeviceStatusError, match="page id outside the pool"):
            rp.run_step(dict(step=step, entries=[dict(id="a", tokens=chunk, want=[len(chunk) - 1])], end=[]))
    rc.tables[0][0] = good
    rc.arrays.clear()
    out = rp.run_step(dict(step=3, entries=[dict(id="a", tokens=toks[34:36], want=[1])], end=["a"]))
    assert np.isfinite(out).all()
