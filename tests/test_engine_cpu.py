"""Scheduler, sampler glue and Python entry point on the CPU (plain kernel statements in the
kernels' place): greedy generation equals the plain implementation under chunked prefill and
when requests are pushed out for lack of pages."""

import pytest
import torch

import cuttings
import kernel_refs
from plain_llama import PlainLlama, TINY_WEIGHTS, tiny_configs


@pytest.fixture()
def cpu_kernels(monkeypatch):
    kernel_refs.install_cpu_kernels(monkeypatch)


def make_engine(model_dir, **kw):
    from tokasaurus_b200.engine.engine import Engine

    opts = dict(dtype="float32", device="cpu", use_cudagraphs=False, page_size=16, kv_cache_num_tokens=1024,
                allocator_sanity_checks=True)
    opts.update(kw)
    return Engine(model=str(model_dir), **opts)


def test_greedy_generation_matches_plain(cpu_kernels, tiny_model_dirs):
    d = tiny_model_dirs[0]
    prompts = [cuttings.random_tokens(n, 256, 40 + n) for n in (5, 17, 32)]
    eng = make_engine(d)
    outs = eng.generate(prompts, max_num_tokens=8, ignore_eos=True)
    plain = PlainLlama(d, torch.float64)
    for p, o in zip(prompts, outs):
        assert o.completion_ids == plain.greedy(p, 8)
        assert o.finish_reason == "length" and len(o.logprobs) == 8
    eng.runner.cache.check()
    assert not eng.runner.cache.requests


def test_chunked_prefill_mixed_with_decode(cpu_kernels, tiny_model_dirs):
    d = tiny_model_dirs[1]
    prompts = [cuttings.random_tokens(n, 509, 3 * n) for n in (1, 40, 63, 30)]
    plain = PlainLlama(d, torch.float64)
    want = [plain.greedy(p, 6) for p in prompts]
    eng = make_engine(d, page_size=8, max_tokens_per_forward=24, kv_cache_num_tokens=512)
    outs = eng.generate(prompts, max_num_tokens=6, ignore_eos=True)
    assert [o.completion_ids for o in outs] == want
    assert eng.scheduler.stats["steps"] > 6  # prompts were cut


def test_pushed_out_requests_give_the_same_tokens(cpu_kernels, tiny_model_dirs):
    d = tiny_model_dirs[0]
    prompts = [cuttings.random_tokens(n, 256, 11 * n) for n in (30, 28, 31, 20)]
    plain = PlainLlama(d, torch.float64)
    want = [plain.greedy(p, 20) for p in prompts]
    # 8 pages of 16: four prompts take 2 pages each, and each wants a third and fourth page while decoding
    eng = make_engine(d, kv_cache_num_tokens=128, bump_city_population_me=True)
    outs = eng.generate(prompts, max_num_tokens=20, ignore_eos=True)
    assert eng.scheduler.stats["bumps"] > 0
    assert [o.completion_ids for o in outs] == want
    assert sum(o.num_preemptions for o in outs) == eng.scheduler.stats["bumps"]
    assert not eng.runner.cache.requests


def test_temperature_sampling_is_keyed_by_request_not_by_batch(cpu_kernels, tiny_model_dirs):
    from tokasaurus_b200 import SamplingParams

    d = tiny_model_dirs[1]
    prompts = [cuttings.random_tokens(n, 509, n) for n in (9, 21, 14)]
    sp = SamplingParams(temperature=0.7, seed=7)
    together = make_engine(d, page_size=8).generate(prompts, sp, max_num_tokens=10, ignore_eos=True)
    again = make_engine(d, page_size=8).generate(prompts, sp, max_num_tokens=10, ignore_eos=True)
    assert [o.completion_ids for o in together] == [o.completion_ids for o in again]
    # chunked differently: the draws are the same because the key is (seed, request, position)
    chunked = make_engine(d, page_size=8, max_tokens_per_forward=8).generate(prompts, sp, max_num_tokens=10,
                                                                              ignore_eos=True)
    assert [o.completion_ids for o in together] == [o.completion_ids for o in chunked]
    other = make_engine(d, page_size=8).generate(prompts, SamplingParams(temperature=0.7, seed=8), max_num_tokens=10,
                                                 ignore_eos=True)
    assert [o.completion_ids for o in together] != [o.completion_ids for o in other]


def test_stop_tokens_and_eos(cpu_kernels, tiny_model_dirs):
    d = tiny_model_dirs[0]
    p = cuttings.random_tokens(12, 256, 5)
    full = PlainLlama(d, torch.float64).greedy(p, 8)
    eng = make_engine(d)
    out = eng.generate([p], max_num_tokens=8, stop_token_ids=[full[3]])[0]
    first = full.index(full[3])
    assert out.completion_ids == full[:first + 1] and out.finish_reason == "stop"


def test_statistics_are_logged(cpu_kernels, tiny_model_dirs, caplog):
    """``stats_report_seconds`` and ``log_level`` keep the reference's meaning: a line of counts and rates at
    level INFO every so many seconds (0: after every step); nothing at WARNING."""
    import logging

    d = tiny_model_dirs[0]
    prompts = [cuttings.random_tokens(n, 256, 7 * n) for n in (9, 20)]
    with caplog.at_level(logging.DEBUG, logger="tokasaurus_b200"):
        eng = make_engine(d, stats_report_seconds=0.0, log_level="INFO")
        eng.generate(prompts, max_num_tokens=5, ignore_eos=True)
    lines = [r.getMessage() for r in caplog.records if r.name == "tokasaurus_b200"]
    assert len(lines) == eng.scheduler.stats["steps"] and all("new tokens" in m and "free pages" in m for m in lines)
    assert sum(int(m.split("prompt tokens ")[1].split(" ")[0]) for m in lines) == 29
    assert sum(int(m.split("new tokens ")[1].split(" ")[0]) for m in lines) == 2 * 5 - 2  # the first of each comes with its prompt
    caplog.clear()
    eng = make_engine(d, stats_report_seconds=0.0, log_level="WARNING")
    eng.generate(prompts, max_num_tokens=5, ignore_eos=True)
    assert not [r for r in caplog.records if r.name == "tokasaurus_b200"]
    with pytest.raises(ValueError, match="log_level"):
        make_engine(d, log_level="LOUD")


def test_steps_ahead_and_paced_prefill_options_reach_the_engine(cpu_kernels, tiny_model_dirs):
    d = tiny_model_dirs[0]
    eng = make_engine(d, scheduling_steps_ahead=0, greedy_prefill=False, prefill_round_up_multiple=4)
    assert eng.run_ahead is False and eng.scheduler.greedy_prefill is False and eng.scheduler.prefill_multiple == 4
    eng = make_engine(d, scheduling_steps_ahead=8)
    assert eng.run_ahead is True and eng.steps_ahead == 8 and eng.scheduler.greedy_prefill is True
    assert len(eng.sampler.host) == 10  # a landing place for every step in flight and the one being read, and one spare
    # paced prefill changes when tokens run, not which tokens come out
    prompts = [cuttings.random_tokens(n, 256, 5 * n) for n in (30, 3, 40, 25)]
    plain = PlainLlama(d, torch.float64)
    eng = make_engine(d, greedy_prefill=False, prefill_round_up_multiple=4, max_seqs_per_forward=2, max_tokens_per_forward=32)
    outs = eng.generate(prompts, max_num_tokens=6, ignore_eos=True)
    assert [o.completion_ids for o in outs] == [plain.greedy(p, 6) for p in prompts]


def test_admission_by_simulated_cache_use_through_the_entry_point(cpu_kernels, tiny_model_dirs):
    """A pool that cannot hold every request at its longest: admitted by the simulation of future page use, the
    requests run side by side where a worst-case reserve would take them in turn, nothing is pushed out, and the
    tokens are the plain implementation's."""
    d = tiny_model_dirs[0]
    prompts = [cuttings.random_tokens(n, 256, 7 * n) for n in (20, 9, 14, 30, 5)]
    limits = [40, 6, 8, 5, 10]
    plain = PlainLlama(d, torch.float64)
    want = [plain.greedy(p, m) for p, m in zip(prompts, limits)]
    most = {}
    for admission in ("reserve", "simulate"):
        eng = make_engine(d, page_size=16, kv_cache_num_tokens=8 * 16, max_seqs_per_forward=8, admission=admission)
        ids = [eng.add_request(p, max_num_tokens=m, ignore_eos=True) for p, m in zip(prompts, limits)]
        done, most[admission] = [], 0
        while eng.has_work():
            done += eng.step()
            most[admission] = max(most[admission], len(eng.scheduler.running()))
        by_id = {o.id: o for o in done}
        assert [by_id[i].completion_ids for i in ids] == want
        assert eng.scheduler.stats["bumps"] == 0 and not eng.runner.cache.requests
    assert most["simulate"] > most["reserve"]
    with pytest.raises(ValueError, match="admission"):
        make_engine(d, admission="optimistic")
    # the simulation is what an engine admits by unless it is asked for the optimistic reserve
    assert make_engine(d).scheduler.admission == "simulate"
    assert make_engine(d, bump_city_population_me=True).scheduler.admission == "reserve"
    assert make_engine(d, kv_reserve_fraction=0.5).scheduler.admission == "reserve"


def test_random_arrivals_in_a_small_pool(cpu_kernels, tiny_model_dirs):
    """Sixteen requests of random lengths and limits arriving at random steps into a pool of 96 tokens, under the
    worst-case reserve, with no reserve (requests are pushed out and fed again), under admission by simulation and
    with a paced prefill: the plain implementation's greedy tokens every time, and every page given back."""
    import random

    d = tiny_model_dirs[1]
    rng = random.Random(5)
    reqs = [(cuttings.random_tokens(rng.randint(1, 60), 509, 70 + i), rng.randint(1, 16)) for i in range(16)]
    plain = PlainLlama(d, torch.float64)
    want = [plain.greedy(p, m) for p, m in reqs]
    arrive = sorted(rng.randint(0, 25) for _ in reqs)
    for way in (dict(), dict(bump_city_population_me=True), dict(admission="simulate"),
                dict(admission="simulate", greedy_prefill=False, prefill_round_up_multiple=4)):
        eng = make_engine(d, page_size=8, kv_cache_num_tokens=96, max_seqs_per_forward=5, max_tokens_per_forward=40, **way)
        ids, done, step, nxt = [], [], 0, 0
        while nxt < len(reqs) or eng.has_work():
            while nxt < len(reqs) and arrive[nxt] <= step:
                ids.append(eng.add_request(reqs[nxt][0], max_num_tokens=reqs[nxt][1], ignore_eos=True))
                nxt += 1
            if eng.has_work():
                done += eng.step()
            step += 1
        by_id = {o.id: o for o in done}
        assert [by_id[i].completion_ids for i in ids] == want, f"way {way}"
        assert not eng.runner.cache.requests and eng.runner.cache.num_free_pages() == [12]
        if way.get("bump_city_population_me"):
            assert eng.scheduler.stats["bumps"] > 0


def test_windowed_attention_through_scheduler_and_cache(cpu_kernels, tmp_path):
    """A toy model whose attention sees a window of 21 keys (pages of 8): prompts longer than the window, decoding
    across several page releases, first with room for everything, then in a pool so small that requests are pushed
    out and fed again through the windowed group.  The tokens equal a plain windowed implementation's."""
    import test_window_gpu as tw
    from tokasaurus_b200.config import unregister_architecture
    from tokasaurus_b200.weights import write_model_folder

    tw.define_toy()
    try:
        c = tw.SMALL
        folder = write_model_folder(tmp_path / "toy", c, seed=11, std=0.08, norm_init="uniform")
        p64 = tw.PlainWindowed(folder, c)
        prompts = [cuttings.random_tokens(n, c["vocab_size"], 300 + n) for n in (45, 9, 30, 26, 52)]
        want = [p64.greedy(p, 24) for p in prompts]
        for pool, opts in ((1024, {}), (104, dict(bump_city_population_me=True))):
            eng = make_engine(folder, page_size=8, kv_cache_num_tokens=pool, max_tokens_per_forward=24,
                              max_seqs_per_forward=4, **opts)
            outs = eng.generate(prompts, max_num_tokens=24, ignore_eos=True)
            assert [o.completion_ids for o in outs] == want
            # a windowed group's pool is no larger than what four requests can hold at once: a window and a
            # step's tokens each, (21 + 24 + 1 tokens -> 6 pages) + 1
            sized = min(pool // 8, 4 * 7)
            assert not eng.runner.cache.requests and eng.runner.cache.num_free_pages() == [sized]
            if opts:
                assert eng.scheduler.stats["bumps"] > 0
    finally:
        unregister_architecture(tw.NAME)
