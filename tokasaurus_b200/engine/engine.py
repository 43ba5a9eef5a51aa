"""The Python entry point: an engine that takes token ids and gives back generated token ids.

The reference is reached over HTTP; its in-process pieces are ``server_manager``
(tokasaurus/entry.py:90-111) and the hand wiring of tokasaurus/benchmarks/bench_model.py:119-283.
This class is the whole of that in one process: scheduler and cache manager on the host, the step
function and the sampler on the GPU.

    engine = Engine(model="/path/to/folder", dtype="bfloat16", kv_cache_num_tokens=65536)
    outs = engine.generate([[1, 2, 3], [4, 5]], SamplingParams(temperature=0.7, seed=7), max_num_tokens=20)
    outs[0].completion_ids
"""

from __future__ import annotations

import logging
import time
from collections import deque
from dataclasses import dataclass, field
from typing import Any, Sequence

import numpy as np
import torch

from tokasaurus_b200.config.engine_config import EngineConfig
from tokasaurus_b200.cache.pages import NoSpaceError
from tokasaurus_b200.engine.batch import StepEntry
from tokasaurus_b200.engine.runner import ModelRunner
from tokasaurus_b200.engine.scheduler import ScheduledPortion, Scheduler, StepPlan
from tokasaurus_b200.sampling.params import Request, RequestOutput, SamplingParams, stream_key
from tokasaurus_b200.sampling.sampler import Sampler


@dataclass
class _InFlight:
    """A decode step that has been launched and whose results are on their way to the host."""
    plan: StepPlan
    rows: int    # rows of the plan
    slot: int    # the sampler's landing place on the host
    h2d: int
    produced: dict = field(default_factory=dict)  # id(sequence) -> completion tokens it has once this step is read


class Engine:
    def __init__(self, model: str | None = None, config: EngineConfig | None = None,
                 config_dict: dict[str, Any] | None = None, seed: int = 0, kv_reserve_fraction: float = 1.0,
                 run_ahead: bool = True, graph_max_tokens: int = 1024, admission: str | None = None,
                 **options: Any):
        """``model``: folder with config.json and model.safetensors.  ``options``: fields of
        ``EngineConfig`` (the reference's option names).  ``config_dict`` with
        ``random_weights=<seed>`` builds a model without a folder.  ``run_ahead``: launch the next decode step
        before the results of the current one have been read, up to ``scheduling_steps_ahead`` steps deep (see
        ``step``).  ``graph_max_tokens``: steps with prompt
        portions of up to this many tokens are replayed from CUDA graphs of their padded shape, like decode steps
        (0: only decode steps are).  ``kv_reserve_fraction``, ``admission``: how queued requests get in
        (``Scheduler``); by default by a simulation of future page use, as the reference admits, unless a reserve
        fraction below 1 or ``bump_city_population_me`` asks for the optimistic reserve."""
        cfg = config or EngineConfig()
        if model is not None:
            cfg.model = model
        for k, v in options.items():
            if not hasattr(cfg, k):
                raise TypeError(f"unknown engine option {k!r}")
            setattr(cfg, k, v)
        if cfg.max_seqs_per_forward > cfg.max_tokens_per_forward:
            cfg.max_seqs_per_forward = cfg.max_tokens_per_forward
        if admission is None:
            admission = "reserve" if (kv_reserve_fraction != 1.0 or cfg.bump_city_population_me) else "simulate"
        self.config = cfg
        self.seed = seed
        self.runner = ModelRunner(cfg, config_dict)
        self.scheduler = Scheduler(
            self.runner.cache, cfg.max_tokens_per_forward, cfg.max_seqs_per_forward,
            cfg.max_num_tokens_per_request, self.runner.eos_token_ids, kv_reserve_fraction,
            cfg.bump_city_population_me, cfg.allocator_sanity_checks, cfg.greedy_prefill,
            cfg.prefill_round_up_multiple, admission)
        # steps launched beyond the one whose results are being read (tokasaurus/common_types.py:89, where the
        # default is 8; here every step ahead is a row wasted for a request that ends on a stop token)
        self.steps_ahead = max(0, int(cfg.scheduling_steps_ahead)) if run_ahead else 0
        self.sampler = Sampler(self.runner.rt.device, max(64, cfg.max_seqs_per_forward, cfg.cudagraph_max_size),
                               cfg.enable_chosen_logprobs, landing_places=self.steps_ahead + 2)
        self.graphs = None
        if cfg.use_cudagraphs and self.runner.rt.device.type == "cuda":
            from tokasaurus_b200.engine.graphs import DecodeGraphs

            self.graphs = DecodeGraphs(self.runner, self.sampler, cfg.cudagraph_max_size, cfg.cudagraph_step,
                                       graph_max_tokens, cfg.cudagraph_max_kv_indices_per_seq,
                                       host_buffers=self.steps_ahead + 1)
        self._auto_id = 0
        self.run_ahead = self.steps_ahead >= 1
        self._inflight: deque[_InFlight] = deque()  # launched steps, oldest first
        self._next_slot = 0
        self.last_step_bytes = dict(h2d=0, d2h=0)
        # a line of statistics every ``stats_report_seconds`` at level INFO, as the reference's manager reports
        # (tokasaurus/manager/manager.py: stats_report_seconds); ``log_level`` is this logger's level
        self.log = logging.getLogger("tokasaurus_b200")
        level = logging.getLevelName(str(cfg.log_level).upper())
        if not isinstance(level, int):
            raise ValueError(f"log_level={cfg.log_level!r} is not a logging level")
        self.log.setLevel(level)
        self._stats_at = time.monotonic()
        self._stats_last = dict(self.scheduler.stats)

    # ------------------------------------------------------------------ requests
    def add_request(self, input_ids: Sequence[int], sampling_params: SamplingParams | None = None,
                    max_num_tokens: int = 16, ignore_eos: bool = False, stop_token_ids: Sequence[int] = (),
                    topk_logprobs: int | None = None, request_id: str | None = None) -> str:
        vocab = self.runner.vocab
        ids = [int(t) for t in input_ids]
        bad = [t for t in ids if not 0 <= t < vocab]
        if bad:
            raise ValueError(f"token ids {bad[:5]} are outside the vocabulary of {vocab}")
        if topk_logprobs is not None:
            limit = self.config.max_topk_logprobs
            if limit is None or topk_logprobs > limit:
                raise ValueError(f"topk_logprobs={topk_logprobs} exceeds max_topk_logprobs={limit}")
        if request_id is None:
            request_id = f"req-{self._auto_id}"
            self._auto_id += 1
        req = Request(request_id, ids, int(max_num_tokens), sampling_params or SamplingParams(), ignore_eos,
                      tuple(int(t) for t in stop_token_ids), topk_logprobs)
        self.scheduler.add_request(req)
        return request_id

    def has_work(self) -> bool:
        return self.scheduler.has_work() or bool(self._inflight)

    # ------------------------------------------------------------------ one step
    def _sampling_arrays(self, plan: StepPlan) -> dict[str, np.ndarray]:
        rows = [p for p in plan.portions if p.samples]
        temp = np.asarray([p.seq.request.sampling_params.temperature for p in rows], dtype=np.float32)
        keys = np.asarray([self._stream_key(p.seq) for p in rows], dtype=np.int64)
        pos = np.asarray([p.start + p.n_tokens for p in rows], dtype=np.int32)
        slot = np.asarray([self.runner.cache.slot(p.seq.id) for p in rows], dtype=np.int32)
        return dict(temperature=temp, stream_key=keys, sample_pos=pos, row_slot=slot)

    def _stream_key(self, seq) -> int:
        """The key of the request's random stream (its seed, or the engine's, and its running number): worked out
        once a request, not once a step."""
        key = getattr(seq, "stream_key", None)
        if key is None:
            sp = seq.request.sampling_params
            key = seq.stream_key = stream_key(sp.seed if sp.seed is not None else self.seed, seq.index)
        return key

    def step(self) -> list[RequestOutput]:
        """Run one step and account for it; return the requests that ended in it.

        Decode steps that run as CUDA graphs are pipelined, as the reference overlaps its manager with its
        model worker (tokasaurus/manager/manager.py:981-1023 keeps steps queued ahead of the model): before the
        results of step t are read, steps t+1 .. t+``scheduling_steps_ahead`` are launched on the guess that every
        request of step t goes on (the token each feeds is still on the device, in the last-token table).  If a
        request of step t ends on an end-of-sequence or stop token after all, its rows of the steps in flight are
        thrown away: wasted rows, no wrong result, and its pages, freed meanwhile, are not written again by
        anything that follows in the stream before their next owner's own writes.  Ends by length are known
        beforehand and never guessed.  Steps are launched ahead only while the scheduler has nothing to decide
        (nothing queued or mid-prompt, a page for every request); a request that arrives waits until the steps
        in flight have been read."""
        done = self._step()
        self._report_stats()
        return done

    def _step(self) -> list[RequestOutput]:
        if not self._inflight:
            done = self._start()
            if done is not None:
                return done
        while len(self._inflight) <= self.steps_ahead:
            following = self._launch_following(self._inflight[-1])
            if following is None:
                break
            self._inflight.append(following)
        return self._finish(self._inflight.popleft())

    def _report_stats(self) -> None:
        now = time.monotonic()
        dt = now - self._stats_at
        if dt < self.config.stats_report_seconds or not self.log.isEnabledFor(logging.INFO):
            return
        st, last, sched = self.scheduler.stats, self._stats_last, self.scheduler
        d = {k: st[k] - last.get(k, 0) for k in st}
        dt = max(dt, 1e-9)
        self.log.info(
            "steps %d (%.1f/s), prompt tokens %d (%.0f/s), new tokens %d (%.0f/s), finished %d, pushed out %d; "
            "decoding %d, in prompt %d, queued %d; free pages %s",
            d["steps"], d["steps"] / dt, d["prefill_tokens"], d["prefill_tokens"] / dt, d["decode_tokens"],
            d["decode_tokens"] / dt, d["finished"], d["bumps"], len(sched.decoding), len(sched.prefilling),
            len(sched.queued), self.runner.cache.num_free_pages())
        self._stats_at = now
        self._stats_last = dict(st)

    def _launch(self, plan: StepPlan, entries: list[StepEntry], extra: dict[str, np.ndarray],
                prep: dict | None = None) -> _InFlight:
        padded = self.graphs.launch(prep if prep is not None else self.graphs.prepare(entries, extra))
        slot = self._next_slot
        self._next_slot = (slot + 1) % len(self.sampler.host)
        self.sampler.start_read(padded, slot, self.runner.stager.status)
        return _InFlight(plan, padded, slot, self.runner.last_upload_bytes)

    def _start(self) -> list[RequestOutput] | None:
        """Schedule a step.  A decode step that runs as a graph is launched and left in flight (returns None);
        anything else runs to its end here."""
        plan = self.scheduler.schedule()
        if not plan.portions:
            return []
        entries = []
        for p in plan.portions:
            toks = None if p.from_device else p.seq.tokens[p.start:p.start + p.n_tokens]
            entries.append(StepEntry(p.seq.id, toks, p.start, [p.n_tokens - 1] if p.samples else []))
        extra = self._sampling_arrays(plan)
        wants_topk = any(p.seq.request.topk_logprobs for p in plan.portions if p.samples)
        if self.graphs is not None and not wants_topk:
            prep = None
            if self.graphs.usable(entries):
                flight = self._launch(plan, entries, extra)
            elif self.graphs.usable_general(entries) and (prep := self.graphs.prepare_general(entries, extra)) is not None:
                flight = self._launch(plan, entries, extra, prep)
            else:
                flight = None
            if flight is not None:
                flight.produced = {id(p.seq): len(p.seq.output.completion_ids) + 1 for p in plan.portions if p.samples}
                self._inflight.append(flight)
                return None
        logits = self.runner.step(entries, extra)
        R = logits.shape[0]
        ids: list[int] = []
        lps: list[float] = []
        topk = None
        if R:
            ex = self.runner.last_context.extra
            self.sampler.sample(logits, ex["temperature"], ex["stream_key"], ex["sample_pos"], ex["row_slot"],
                                self.runner.cache.last_token)
            kmax = max((p.seq.request.topk_logprobs or 0) for p in plan.portions if p.samples)
            if kmax:
                ti, tl = self.sampler.topk(logits, ex["temperature"], kmax)
            ids, lps = self.sampler.read(R)
            if kmax:
                topk = list(zip(ti.tolist(), tl.tolist()))
        self.runner.check_status()
        self.last_step_bytes = dict(h2d=self.runner.last_upload_bytes, d2h=self.sampler.bytes_last_read if R else 4)
        return self.scheduler.complete(plan, ids, lps if self.config.enable_chosen_logprobs else None, topk)

    def _finish(self, cur: _InFlight) -> list[RequestOutput]:
        """Wait for an in-flight step and account for it.  Rows of requests that ended in the step before it
        (it was launched before that was known) are dropped."""
        ids, lps, status = self.sampler.finish_read(cur.rows, cur.slot)
        self.runner.check_status(status)
        running = set(map(id, self.scheduler.decoding)) | set(map(id, self.scheduler.prefilling))
        portions, kept_ids, kept_lps = [], [], []
        k = 0  # the k-th portion that samples owns the k-th row of the results
        for p in cur.plan.portions:
            alive = id(p.seq) in running
            if alive:
                portions.append(p)
            if p.samples:
                if alive:
                    kept_ids.append(ids[k])
                    kept_lps.append(lps[k])
                k += 1
        plan = cur.plan if len(portions) == len(cur.plan.portions) else StepPlan(portions, cur.plan.bumped)
        self.last_step_bytes = dict(h2d=cur.h2d, d2h=self.sampler.bytes_last_read)
        return self.scheduler.complete(plan, kept_ids, kept_lps if self.config.enable_chosen_logprobs else None, None)

    def _launch_following(self, cur: _InFlight) -> _InFlight | None:
        """Launch the decode step after ``cur`` (the newest step in flight) before ``cur``'s results are known:
        every request of ``cur`` that is still running and does not end by length in ``cur`` brings the token
        ``cur`` samples for it.  None if the scheduler has decisions to make first (something is queued or
        mid-prompt, a page is missing)."""
        sched = self.scheduler
        if sched.queued or sched.prefilling:
            return None
        running = set(map(id, sched.decoding))
        portions, entries, produced = [], [], {}
        try:
            for p in cur.plan.portions:
                seq = p.seq
                if id(seq) not in running:
                    continue  # ended in a step that has been read since ``cur`` was launched
                if not p.samples:
                    return None  # a prompt portion that goes on: the scheduler cuts the next one
                made = cur.produced[id(seq)]
                if made >= seq.request.max_num_tokens:
                    continue  # ends by length in ``cur``
                produced[id(seq)] = made + 1
                start = p.start + p.n_tokens
                self.runner.cache.ensure_capacity(seq.id, start + 1)
                portions.append(ScheduledPortion(seq, start, 1, True, from_device=True))
                entries.append(StepEntry(seq.id, None, start, [0]))
        except (NoSpaceError, KeyError):
            return None  # no page free: the scheduler decides who is pushed out
        if not entries or not self.graphs.usable(entries):
            return None
        plan = StepPlan(portions)
        flight = self._launch(plan, entries, self._sampling_arrays(plan))
        flight.produced = produced
        return flight

    def warm_up(self, batch_sizes: Sequence[int] | None = None) -> int:
        """Record the CUDA graphs of decode steps before the first request needs them, as the reference records
        its graphs at start-up (tokasaurus/model/utils.py:839-882); else a batch size is recorded (some tens of
        milliseconds) the first time it comes up.  ``batch_sizes``: padded sizes to record (all that the request
        slots allow by default).  Returns how many graphs were recorded.  Only with no request in the engine."""
        if self.graphs is None:
            return 0
        if self.has_work() or self.runner.cache.requests:
            raise RuntimeError("warm_up() wants an engine without requests")
        cache = self.runner.cache
        made = 0
        page = self.runner.config.page_size
        # without work plans (float32) nothing depends on the context
        contexts = (1, 256, 1024, 4096, 16384, 65536) if self.runner.model.planners() else (1,)
        for bp in (batch_sizes if batch_sizes is not None else self.graphs.sizes):
            # A graph holds the kernels chosen when it was recorded, and the attention's choice depends on how long
            # the step's work items are: each batch size is recorded at context 1 and again at the shortest of a
            # few longer contexts that the free pages allow and that gives another graph (what the pages hold
            # does not matter here: nothing is read back).
            seen = set()
            for context in contexts:
                if len(seen) >= 2:
                    break
                need = bp * -(-context // page)
                if bp > cache.slots.num_free or any(need > f for f in cache.num_free_pages()):
                    break
                ids = [f"__warm_up_{i}" for i in range(bp)]
                try:
                    for rid in ids:
                        cache.admit(rid)
                        cache.ensure_capacity(rid, context)
                    entries = [StepEntry(rid, [0], context - 1, [0]) for rid in ids]
                    if not self.graphs.usable(entries):
                        break
                    # rows without a slot: the sampler leaves the last-token table alone
                    extra = dict(temperature=np.zeros(bp, dtype=np.float32), stream_key=np.zeros(bp, dtype=np.int64),
                                 sample_pos=np.full(bp, context, dtype=np.int32), row_slot=np.full(bp, -1, dtype=np.int32))
                    prep = self.graphs.prepare(entries, extra)
                    seen.add(prep["key"])
                    if prep["key"] not in self.graphs.graphs:
                        self.graphs.launch(prep)
                        made += 1
                finally:
                    for rid in ids:
                        if rid in cache.requests:
                            cache.free(rid)
        if self.runner.rt.device.type == "cuda":
            torch.cuda.synchronize(self.runner.rt.device)
        self.runner.check_status()
        return made

    def run_until_done(self) -> list[RequestOutput]:
        done: list[RequestOutput] = []
        while self.has_work():
            done.extend(self.step())
        return done

    def generate(self, prompts: Sequence[Sequence[int]], sampling_params: SamplingParams | Sequence[SamplingParams] | None = None,
                 max_num_tokens: int = 16, ignore_eos: bool = False, stop_token_ids: Sequence[int] = (),
                 topk_logprobs: int | None = None) -> list[RequestOutput]:
        """Generate for every prompt (lists of token ids); outputs come back in the prompts' order."""
        ids = []
        for i, p in enumerate(prompts):
            sp = sampling_params[i] if isinstance(sampling_params, (list, tuple)) else sampling_params
            ids.append(self.add_request(p, sp, max_num_tokens, ignore_eos, stop_token_ids, topk_logprobs))
        by_id = {o.id: o for o in self.run_until_done()}
        return [by_id[i] for i in ids]
