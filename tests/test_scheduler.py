"""The scheduler's decisions, with a cache manager that keeps books only and a stand-in for the
model: admission, portions under the token budget, decoding, finishing, and pushing requests
out when pages run out."""

import pytest

from tokasaurus_b200.cache import CacheManager, NoSpaceError
from tokasaurus_b200.engine.scheduler import RequestTooLongError, Scheduler
from tokasaurus_b200.parts.base import PagedCacheNeed
from tokasaurus_b200.sampling.params import Request, SamplingParams


def make(num_pages=64, page_size=4, max_tokens=16, max_seqs=8, **kw):
    cache = CacheManager({0: PagedCacheNeed(1, 16)}, page_size=page_size, num_pages=num_pages, max_requests=max_seqs)
    return Scheduler(cache, max_tokens, max_seqs, sanity_checks=True, **kw), cache


def req(i, n, max_new=4, **kw):
    return Request(f"r{i}", list(range(1, n + 1)), max_new, SamplingParams(), **kw)


def run(s, token=lambda seq: 7, limit=10_000):
    finished, plans = [], []
    while s.has_work() and limit:
        limit -= 1
        plan = s.schedule()
        plans.append(plan)
        sampled = [token(p.seq) for p in plan.portions if p.samples]
        finished += s.complete(plan, sampled, [0.0] * len(sampled))
    return finished, plans


def test_portions_follow_the_budget():
    s, cache = make(max_tokens=16)
    s.add_request(req(0, 40, 3))
    s.add_request(req(1, 5, 3))
    plan = s.schedule()
    assert [(p.seq.id, p.start, p.n_tokens, p.samples) for p in plan.portions] == [("r0", 0, 16, False)]
    s.complete(plan, [])
    plan = s.schedule()
    assert [(p.seq.id, p.start, p.n_tokens) for p in plan.portions] == [("r0", 16, 16)]
    s.complete(plan, [])
    plan = s.schedule()  # r0's last 8 tokens, then r1's 5 fit in the same step
    assert [(p.seq.id, p.start, p.n_tokens, p.samples) for p in plan.portions] == [("r0", 32, 8, True), ("r1", 0, 5, True)]
    s.complete(plan, [7, 7])
    plan = s.schedule()  # both decode from the device's last-token table
    assert [(p.seq.id, p.start, p.n_tokens, p.from_device) for p in plan.portions] == [("r0", 40, 1, True), ("r1", 5, 1, True)]
    assert cache.pages_for(41) == len(cache.table("r0", 0))


def test_decodes_come_first_and_prompt_is_cut_where_the_budget_ends():
    s, _ = make(max_tokens=8)
    s.add_request(req(0, 3, 10))
    s.add_request(req(1, 3, 10))
    fin, plans = run(s, limit=2)
    s.add_request(req(2, 30, 2))
    plan = s.schedule()
    assert [(p.seq.id, p.n_tokens, p.from_device) for p in plan.portions] == [("r0", 1, True), ("r1", 1, True), ("r2", 6, False)]


def test_finish_by_length_stop_and_eos():
    s, cache = make(eos_token_ids=(9,))
    s.add_request(req(0, 3, 5))
    s.add_request(req(1, 3, 5, stop_token_ids=(8,)))
    s.add_request(req(2, 3, 5, ignore_eos=True))
    seqs = iter([1, 1, 1, 9, 8, 9, 2, 2, 2])
    fin, _ = run(s, token=lambda seq: {"r0": [1, 9], "r1": [1, 8], "r2": [1, 9, 9, 9, 9]}[seq.id][len(seq.output.completion_ids)])
    by = {o.id: o for o in fin}
    assert by["r0"].completion_ids == [1, 9] and by["r0"].finish_reason == "stop"
    assert by["r1"].completion_ids == [1, 8] and by["r1"].finish_reason == "stop"
    assert by["r2"].completion_ids == [1, 9, 9, 9, 9] and by["r2"].finish_reason == "length"
    assert not cache.requests and cache.num_free_pages() == [64]


def test_worst_case_reservation_never_pushes_out():
    s, cache = make(num_pages=12, page_size=4, max_tokens=64)
    for i in range(6):
        s.add_request(req(i, 8, 9))  # each can come to hold 4 pages: only 3 fit at a time
    plan = s.schedule()
    assert len(plan.portions) == 3 and len(s.queued) == 3
    s.complete(plan, [7] * 3)
    fin, _ = run(s)
    assert s.stats["bumps"] == 0 and len(fin) == 6


def test_pages_run_out_the_youngest_goes_back_to_the_head_of_the_queue():
    s, cache = make(num_pages=6, page_size=4, max_tokens=64, bump_city_population_me=True)
    for i in range(3):
        s.add_request(req(i, 8, 12))  # 2 pages each at first: the pool is full after admission
    plan = s.schedule()
    assert [p.seq.id for p in plan.portions] == ["r0", "r1", "r2"] and cache.num_free_pages() == [0]
    s.complete(plan, [7] * 3)
    plan = s.schedule()  # all three want a third page for position 8
    assert plan.bumped == ["r2"]  # the youngest; its two pages serve r0 and r1
    assert [p.seq.id for p in plan.portions] == ["r0", "r1"]
    assert [q.id for q in s.queued] == ["r2"] and cache.num_free_pages() == [0]
    s.add_request(req(3, 4, 2))
    assert [q.id for q in s.queued] == ["r2", "r3"]  # a pushed-out request waits at the head of the queue
    s.complete(plan, [7, 7])
    fin, plans = run(s)
    assert sorted(o.id for o in fin) == ["r0", "r1", "r2", "r3"]
    assert all(len(o.completion_ids) == 12 for o in fin if o.id != "r3")
    # a pushed-out request is fed its prompt and what it had produced again, as one prompt
    again = [p for pl in plans for p in pl.portions if p.seq.id == "r2" and not p.from_device]
    assert again and again[0].start == 0 and again[0].n_tokens == 8 + 1
    assert not cache.requests and cache.num_free_pages() == [6]


def test_request_that_can_never_fit_is_refused():
    s, _ = make(num_pages=4, page_size=4)
    with pytest.raises(RequestTooLongError):
        s.add_request(req(0, 10, 10))
    s2, _ = make(max_num_tokens_per_request=12)
    with pytest.raises(RequestTooLongError):
        s2.add_request(req(0, 10, 3))
    with pytest.raises(ValueError):
        s.add_request(Request("e", [], 3))
    with pytest.raises(ValueError):
        s.add_request(Request("p", [1], 3, SamplingParams(top_p=0.9)))


def test_slots_limit_admission():
    s, _ = make(max_seqs=2, max_tokens=64)
    for i in range(4):
        s.add_request(req(i, 3, 2))
    plan = s.schedule()
    assert len(plan.portions) == 2
    fin, _ = run(s)
    assert len(fin) == 4


def test_prefill_without_greed_is_paced():
    """``greedy_prefill=F``: all that fits while nobody queues; exactly the first prompt while nobody decodes;
    else the prompt tokens outstanding by the time a decoding sequence ends and makes room for the queue's
    head, spread over the steps until then and rounded up to ``prefill_round_up_multiple``."""
    def scene(**kw):
        s, cache = make(num_pages=200, page_size=4, max_tokens=32, max_seqs=2, greedy_prefill=False, **kw)
        s.add_request(req(0, 3, 21))  # 3 + 21 - 1 = 23 tokens go through the model
        plan = s.schedule()
        assert [(p.seq.id, p.n_tokens) for p in plan.portions] == [("r0", 3)]  # nobody queues: all that fits
        s.complete(plan, [7], [0.0])
        s.add_request(req(1, 100, 2))
        s.add_request(req(2, 60, 2))
        s.add_request(req(3, 10, 2))
        return s

    # r0 ends 20 steps from now; its slot then goes to r2 (r3 still waits), so 100 + 60 prompt tokens are due
    # in 20 steps: 8 a step
    s = scene(prefill_round_up_multiple=4)
    plan = s.schedule()
    assert [(p.seq.id, p.n_tokens, p.from_device) for p in plan.portions] == [("r0", 1, True), ("r1", 8, False)]
    s = scene(prefill_round_up_multiple=16)
    plan = s.schedule()
    assert [(p.seq.id, p.n_tokens) for p in plan.portions] == [("r0", 1), ("r1", 16)]
    # and everything still ends
    fin, plans = run(s)
    assert sorted(o.id for o in fin) == ["r0", "r1", "r2", "r3"]
    assert all(p.n_tokens <= 32 for p in plans)

    # nobody decodes, somebody queues: exactly the first prompt, although the second would fit beside it
    s, _ = make(num_pages=200, page_size=4, max_tokens=32, max_seqs=2, greedy_prefill=False)
    for i in range(3):
        s.add_request(req(i, 5, 3))
    plan = s.schedule()
    assert [(p.seq.id, p.n_tokens) for p in plan.portions] == [("r0", 5)]
    greedy, _ = make(num_pages=200, page_size=4, max_tokens=32, max_seqs=2)
    for i in range(3):
        greedy.add_request(req(i, 5, 3))
    assert [(p.seq.id, p.n_tokens) for p in greedy.schedule().portions] == [("r0", 5), ("r1", 5)]


def test_paced_prefill_counts_pages_as_admission_does():
    """The queue's head does not fit when the first decoding sequence has given its pages back, only when the
    second has: each end is a candidate (what is outstanding by then over the steps until then), the smallest
    wins, and ends after the one at which the whole queue fits ask for nothing slower."""
    def scene(extra):
        s, cache = make(num_pages=40, page_size=4, max_tokens=64, max_seqs=8, greedy_prefill=False,
                        prefill_round_up_multiple=1)
        s.add_request(req(0, 4, 9))    # 12 tokens, 3 pages, ends 8 steps after its prompt
        s.add_request(req(1, 4, 41))   # 44 tokens, 11 pages, ends 40 steps after its prompt
        plan = s.schedule()
        s.complete(plan, [7, 7], [0.0, 0.0])
        s.add_request(req(2, 40, 5))   # 44 tokens, 11 pages: admitted; 15 pages are left beside the reserves
        s.add_request(req(3, 72, 5))   # 76 tokens, 19 pages: waits; r0's 3 pages do not make room, r1's 11 do
        for r in extra:
            s.add_request(r)
        return s

    s = scene([])
    plan = s.schedule()
    assert [q.id for q in s.queued] == ["r3"]
    # r0's end: r3 still waits, 40 tokens in 8 steps; r1's end: the queue is empty, no further candidate
    assert [(p.seq.id, p.n_tokens) for p in plan.portions] == [("r0", 1), ("r1", 1), ("r2", 5)]
    s = scene([req(4, 40, 5)])
    plan = s.schedule()
    assert [q.id for q in s.queued] == ["r3", "r4"]
    # r1's end: r3 is in, r4 waits behind it: 40 + 72 tokens in 40 steps, slower than 40 in 8
    assert [(p.seq.id, p.n_tokens) for p in plan.portions] == [("r0", 1), ("r1", 1), ("r2", 3)]
    fin, _ = run(s)
    assert sorted(o.id for o in fin) == ["r0", "r1", "r2", "r3", "r4"]


@pytest.mark.parametrize("seed", range(6))
def test_paced_prefill_under_random_load_always_ends(seed):
    """Whatever the mix of prompts, lengths, pool and reserve: without greed every request still ends, a step
    never passes the token budget, no page is lost, and the produced tokens are those of the greedy scheduler
    (only when a token runs changes)."""
    import random

    rnd = random.Random(seed)
    reqs = [(rnd.randint(1, 60), rnd.randint(1, 30)) for _ in range(rnd.randint(5, 25))]
    kw = dict(num_pages=rnd.choice([40, 64, 200]), page_size=rnd.choice([4, 8]), max_tokens=rnd.choice([8, 16, 48]),
              max_seqs=rnd.choice([2, 4, 8]), kv_reserve_fraction=rnd.choice([1.0, 0.5, 0.0]))
    outs = {}
    for greedy in (True, False):
        s, cache = make(greedy_prefill=greedy, prefill_round_up_multiple=rnd.choice([1, 4, 16]), **kw)
        pending = list(enumerate(reqs))
        finished, steps = [], 0
        while s.has_work() or pending:
            for _ in range(rnd.randint(0, 2)):
                if pending:
                    i, (n, new) = pending.pop(0)
                    s.add_request(req(i, n, new))
            if not s.has_work():
                continue
            plan = s.schedule()
            assert 0 < plan.n_tokens <= kw["max_tokens"]
            sampled = [(len(p.seq.output.completion_ids) * 31 + p.seq.index) % 97 for p in plan.portions if p.samples]
            finished += s.complete(plan, sampled, [0.0] * len(sampled))
            cache.check()
            steps += 1
            assert steps < 20_000
        assert sorted(o.id for o in finished) == sorted(f"r{i}" for i in range(len(reqs)))
        assert not cache.requests
        outs[greedy] = {o.id: o.completion_ids for o in finished}
    assert outs[True] == outs[False]


def test_a_request_id_in_use_is_refused():
    s, _ = make()
    s.add_request(req(0, 5, 3))
    with pytest.raises(ValueError, match="already queued or running"):
        s.add_request(req(0, 7, 3))
    s.complete(s.schedule(), [7])
    with pytest.raises(ValueError, match="already queued or running"):
        s.add_request(req(0, 7, 3))
    run(s)
    s.add_request(req(0, 7, 3))  # the first owner has ended: the id is free again


def test_reserve_is_kept_per_cache_group():
    """Two cache groups, the FIRST with a window: a sequence of a windowed group never holds more pages than the
    window and one step's tokens take, so the full group is what limits admission, and nothing is ever pushed
    out under the worst-case reserve."""
    needs = {0: PagedCacheNeed(1, 16, window=6), 1: PagedCacheNeed(1, 16)}
    cache = CacheManager(needs, page_size=4, num_pages=12, max_requests=8)
    assert [g.need.window for g in cache.groups] == [6, None]
    s = Scheduler(cache, 8, 8, sanity_checks=True)
    for i in range(5):
        s.add_request(req(i, 8, 9))  # each comes to hold 4 pages of the full group: 3 fit at a time
    plan = s.schedule()
    assert len(s.prefilling) == 3 and len(s.queued) == 2
    # the windowed group: at most pages_for(6 + 8) + 1 = 5 live pages a sequence, so it sets aside less than the
    # 4 - 2 a sequence of the full group still needs only when the cap bites; here both groups ask for 2 more each
    assert s._headroom() == [12 - 6 - 6, 12 - 6 - 6]
    fin, plans = run(s)
    assert len(fin) == 5 and s.stats["bumps"] == 0
    assert cache.num_free_pages() == [12, 12]
    # pages of the windowed group came back while their sequences ran: its tables hold -1 at the front
    s.add_request(req(9, 20, 12))
    for _ in range(6):
        plan = s.schedule()
        s.complete(plan, [7] * sum(p.samples for p in plan.portions))
    rc = cache.requests["r9"]
    assert rc.tables[0][0] == -1 and rc.tables[1][0] >= 0
    assert s._still_needed(s.running()[0], 0) <= s._still_needed(s.running()[0], 1)


def test_long_requests_in_a_windowed_pool_smaller_than_their_length():
    """With a window in every group, the reserve per sequence is capped by what a window and a step's tokens take,
    so requests far longer than the pool run side by side without being pushed out."""
    cache = CacheManager({0: PagedCacheNeed(1, 16, window=8)}, page_size=4, num_pages=16, max_requests=8)
    s = Scheduler(cache, 4, 8, sanity_checks=True)
    for i in range(2):
        s.add_request(req(i, 4, 60))  # 63 positions = 16 pages each without the window
    fin, plans = run(s)
    assert len(fin) == 2 and s.stats["bumps"] == 0
    assert max(len(p.portions) for p in plans) == 2  # they did run together


def test_a_windowed_group_has_a_pool_of_its_own_size_and_long_prompts_pass_through_it():
    """The pool of a group with a window is sized by what the request slots can hold at once, not by the token
    count that sizes the groups that see all keys; a prompt longer than that pool takes its pages there portion by
    portion while the pages behind the window come back."""
    needs = {0: PagedCacheNeed(1, 16), 1: PagedCacheNeed(1, 16, window=8)}
    cache = CacheManager(needs, page_size=4, num_pages=128, max_requests=2, max_step_tokens=8)
    # window 8 + step 8 + 1 token ahead = 17 tokens -> 5 pages, + 1 for where the window starts: 6 a request
    assert [g.allocator.num_pages for g in cache.groups] == [128, 12]
    s = Scheduler(cache, 8, 2, sanity_checks=True)
    for i in range(3):
        s.add_request(req(i, 150 + i, 20))  # 38 pages of prompt each: three times the windowed pool
    fin, plans = run(s)
    assert len(fin) == 3 and s.stats["bumps"] == 0
    assert all(sum(p.n_tokens for p in plan.portions) <= 8 for plan in plans)
    assert max(len(plan.portions) for plan in plans) == 2
    assert cache.num_free_pages() == [128, 12]


def test_prompt_portions_shrink_when_a_windowed_pool_is_short():
    """A windowed pool too small for two requests at full pace: portions are cut to the pages that are free, a
    request that cannot go on at all waits for the other or pushes it out, and every request ends."""
    cache = CacheManager({0: PagedCacheNeed(1, 16, window=8)}, page_size=4, num_pages=7, max_requests=4,
                         max_step_tokens=12)
    assert cache.groups[0].allocator.num_pages == 7
    s = Scheduler(cache, 12, 4, sanity_checks=True)
    for i in range(3):
        s.add_request(req(i, 40 + 3 * i, 10))
    fin, plans = run(s)
    assert sorted(o.id for o in fin) == ["r0", "r1", "r2"]
    assert all(len(o.completion_ids) == 10 for o in fin)
    sizes = {p.n_tokens for plan in plans for p in plan.portions if not p.from_device}
    assert min(sizes) < 12  # some portion was cut short of the budget by the pages
    assert cache.num_free_pages() == [7]
    with pytest.raises(RequestTooLongError, match="cache group 0"):
        small = CacheManager({0: PagedCacheNeed(1, 16, window=8)}, page_size=4, num_pages=3, max_requests=4)
        Scheduler(small, 12, 4).add_request(req(0, 40, 10))  # a window of 8 and the next token can span 4 pages


def make_sim(num_pages, max_tokens=16, max_seqs=8, page_size=4, **kw):
    cache = CacheManager({0: PagedCacheNeed(1, 16)}, page_size=page_size, num_pages=num_pages, max_requests=max_seqs)
    return Scheduler(cache, max_tokens, max_seqs, sanity_checks=True, admission="simulate", **kw), cache


def test_simulated_peak_is_the_highest_use_before_some_end():
    """Two decoding sequences that end at different times: the peak is the larger of (both, when the first ends)
    and (the second alone at its longest), worked out by hand."""
    s, cache = make_sim(64)
    s.add_request(req(0, 8, 5))    # 12 positions at most: 3 pages
    s.add_request(req(1, 8, 21))   # 28 positions at most: 7 pages
    s.complete(s.schedule(), [7, 7])
    assert [q.fed for q in s.decoding] == [8, 8]
    # r0 ends after 4 more steps with 12 tokens (3 pages) while r1 has 12 too (3 pages): 6; r1 alone at its end: 7
    assert s._simulated_peak() == [7]
    # a third that is as long as r0 adds 3 pages at the first end and nothing at the second
    s.add_request(req(2, 8, 5))
    assert s._simulated_peak([s.queued[0]]) == [9]
    # one as long as r1, admitted now, is fed in the next step and ends one step after r1: 7 + 7 just before r1 ends
    s.queued.clear()
    s.add_request(req(3, 8, 21))
    assert s._simulated_peak([s.queued[0]]) == [14]


def test_simulated_admission_lets_in_what_a_worst_case_reserve_keeps_out():
    """Sequences of very different lengths in a pool that cannot hold all of them at their longest at once: the
    reserve admits them one after the other, the simulation sees that the short ones are gone before the long one
    grows, admits them together, and still nothing is pushed out."""
    def requests(s):
        s.add_request(req(0, 8, 41))  # 48 positions: 12 pages at its end
        for i in range(1, 5):
            s.add_request(req(i, 8, 5))  # 12 positions: 3 pages each
    cache = CacheManager({0: PagedCacheNeed(1, 16)}, page_size=4, num_pages=16, max_requests=8)
    reserve = Scheduler(cache, 64, 8, sanity_checks=True)
    requests(reserve)
    reserve.schedule()
    assert len(reserve.prefilling) == 2  # 12 + 3 of 16 pages spoken for
    sim, cache = make_sim(16, max_tokens=64)
    requests(sim)
    sim.schedule()
    assert len(sim.prefilling) == 5  # when the short ones end they hold 4 * 3 pages and the long one 3: 15
    fin, plans = run(sim)
    assert len(fin) == 5 and sim.stats["bumps"] == 0
    assert cache.num_free_pages() == [16]


def test_simulated_admission_keeps_out_what_would_not_fit():
    sim, cache = make_sim(16, max_tokens=64)
    sim.add_request(req(0, 8, 41))  # 12 pages at its end
    sim.add_request(req(1, 8, 37))  # 11 pages at its end, one step before the other ends: 11 + 12 > 16
    sim.schedule()
    assert len(sim.prefilling) == 1 and len(sim.queued) == 1
    fin, _ = run(sim)
    assert [o.id for o in fin] == ["r0", "r1"] and sim.stats["bumps"] == 0


@pytest.mark.parametrize("seed", range(4))
def test_simulated_admission_random_workloads_never_push_out(seed):
    """With prompts fed at the full token budget (greedy prefill) the simulation's assumptions hold, so requests
    of random lengths arriving at random steps all end without anyone being pushed out, in pools of two sizes."""
    import random
    rng = random.Random(seed)
    for pages in (24, 60):
        sim, cache = make_sim(pages, max_tokens=32, max_seqs=6)
        pending = [req(i, rng.randint(1, 30), rng.randint(1, 40)) for i in range(25)]
        finished = []
        while pending or sim.has_work():
            for _ in range(rng.randint(0, 2)):
                if pending:
                    sim.add_request(pending.pop())
            if not sim.has_work():
                continue
            plan = sim.schedule()
            finished += sim.complete(plan, [7] * sum(p.samples for p in plan.portions))
            assert all(pk <= g.allocator.num_pages for pk, g in zip(sim._simulated_peak(), cache.groups))
        assert len(finished) == 25 and sim.stats["bumps"] == 0
        assert cache.num_free_pages() == [pages]


def test_many_sequences_are_told_apart_by_identity_and_stage():
    """Six hundred sequences with the same prompt at once: the scheduler's membership questions are answered by a
    sequence's stage and identity (two sequences with equal fields are different sequences), so a step's decisions
    take time in proportion to the sequences, and every one of them ends with its own tokens."""
    import time
    s, cache = make(num_pages=600 * 8, page_size=4, max_tokens=4096, max_seqs=600)
    seqs = [s.add_request(Request(f"same{i}", [1, 2, 3, 4, 5], 20, SamplingParams())) for i in range(600)]
    assert seqs[0] != seqs[1] and seqs[0] == seqs[0]
    assert {q.stage for q in seqs} == {"queued"}
    t0 = time.perf_counter()
    plan = s.schedule()
    assert {q.stage for q in seqs} == {"prefilling"} and len(plan.portions) == 600
    s.complete(plan, list(range(600)))
    assert {q.stage for q in seqs} == {"decoding"}
    fin, plans = run(s, token=lambda seq: seq.index)
    assert len(fin) == 600 and all(o.completion_ids[1:] == [int(o.id[4:])] * 19 for o in fin)
    assert {q.stage for q in seqs} == {"queued"} and not s._live_ids
    assert time.perf_counter() - t0 < 20.0  # 21 steps of 600 sequences: seconds even on a slow machine, not minutes


@pytest.mark.parametrize("seed", range(12))
def test_simulated_peak_is_what_really_happens(seed):
    """Random sets of requests, all admitted, some in mid-prompt: the most pages the cache really holds from then on
    (no one else comes, prompts fed greedily) is exactly the simulated peak."""
    import random
    rng = random.Random(seed)
    cache = CacheManager({0: PagedCacheNeed(1, 16)}, page_size=4, num_pages=4000, max_requests=40)
    s = Scheduler(cache, 24, 40, sanity_checks=True, admission="simulate")
    for i in range(rng.randint(3, 30)):
        s.add_request(req(i, rng.randint(1, 50), rng.randint(1, 60)))
    for _ in range(rng.randint(1, 4)):  # a few steps in: some decode, some are in mid-prompt, some still queued
        plan = s.schedule()
        s.complete(plan, [7] * sum(p.samples for p in plan.portions))
    while s.queued:  # everyone in (the pool is large); what follows is what the simulation speaks about
        plan = s.schedule()
        s.complete(plan, [7] * sum(p.samples for p in plan.portions))
        if not s.has_work():
            return
    predicted = s._simulated_peak()[0]
    used = lambda: cache.groups[0].allocator.num_pages - cache.groups[0].allocator.num_free  # noqa: E731
    most = used()
    while s.has_work():
        plan = s.schedule()
        most = max(most, used())
        s.complete(plan, [7] * sum(p.samples for p in plan.portions))
    assert most == predicted  # under a greedy prefill the simulation is what happens


@pytest.mark.parametrize("seed", range(8))
def test_the_head_taken_in_one_go_is_the_head_taken_one_by_one(seed):
    """Admission by simulation finds the longest head of the queue that fits by halving; it is the same head that
    asking request by request gives, and the next one in the queue would not have fitted."""
    import random
    rng = random.Random(seed)
    s, cache = make_sim(rng.randint(20, 120), max_tokens=32, max_seqs=rng.randint(3, 12))
    for i in range(20):
        s.add_request(req(i, rng.randint(1, 40), rng.randint(1, 50)))
    for _ in range(rng.randint(0, 5)):
        plan = s.schedule()
        s.complete(plan, [7] * sum(p.samples for p in plan.portions))
    head = s._fitting_by_simulation()
    pool = cache.groups[0].allocator.num_pages
    slots = min(len(s.queued), s.max_seqs - len(s.running()), cache.slots.num_free)
    one_by_one, free = 0, cache.groups[0].allocator.num_free
    while one_by_one < slots:
        nxt = s.queued[one_by_one]
        free -= cache.pages_for(nxt.n_known)
        if free < 0 or s._simulated_peak([s.queued[i] for i in range(one_by_one + 1)])[0] > pool:
            break
        one_by_one += 1
    assert [q.id for q in head] == [s.queued[i].id for i in range(one_by_one)]
