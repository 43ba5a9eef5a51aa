"""The scheduler: admits requests, cuts prompts into portions under a token budget, decodes,
finishes and frees.

In the manner of the reference's manager (tokasaurus/manager/manager.py:981-1023 loop,
tokasaurus/manager/scheduler.py:576-637 ``schedule``, :640-684 ``apply_decision``), much smaller:

* Three FIFO stages: queued -> prefilling -> decoding (tokasaurus/manager/types.py:150-250).
* Every decoding sequence is in every step with one token.  What is left of
  ``max_tokens_per_forward`` goes to prompts, first come first served, and a prompt is cut
  wherever the budget ends (``make_scheduling_decision``, scheduler.py:541-573; with
  ``greedy_prefill``, the default, the reference too takes all that fits, scheduler.py:604-637; without it
  the prompts are paced, see ``_prefill_budget``).
* Admission: a queued request enters when a slot is free and the pool has pages for its whole
  prompt (allocated at once, as ``allocate_with_prefix_match`` does, allocator.py:324-384) on top
  of what is set aside for running requests.  ``kv_reserve_fraction`` = 1 sets aside every page a
  running request can still come to need (no request is ever pushed out); smaller values admit
  more and rely on the next rule; ``bump_city_population_me`` (the reference's debugging flag,
  common_types.py:125) sets nothing aside.
  With ``admission="simulate"`` the request enters instead when the pages in use at every future step,
  worked out as if every running request went on to its limit, stay within the pool with it
  (``calc_block_usage_over_time`` and the onboarding around it, scheduler.py:46-216, manager.py:486-656).
* When a decoding sequence needs a page and none is free, the most recently admitted running
  sequence is pushed out ("bumped", manager.py:745-813): its pages and slot are given back and it
  returns to the HEAD of the queue.  Unlike the reference, which restarts it from the bare prompt
  and samples anew, it keeps the tokens it has produced: they are fed again as part of its
  prompt, so its output is the same as without the bump.
* A sequence ends on ``max_num_tokens``, on an end-of-sequence id (unless ``ignore_eos``) or on
  one of its ``stop_token_ids`` (manager.py:201-206); its pages and slot are given back then.
"""

from __future__ import annotations

import bisect
from collections import deque
from dataclasses import dataclass, field

import numpy as np

from tokasaurus_b200.cache.manager import CacheManager
from tokasaurus_b200.cache.pages import NoSpaceError
from tokasaurus_b200.sampling.params import Request, RequestOutput


class RequestTooLongError(ValueError):
    pass


@dataclass(eq=False)  # a sequence equals itself only: membership tests compare identities, not token lists
class Sequence:
    request: Request
    index: int  # running number of the request within the engine (random stream, admission order)
    output: RequestOutput
    fed: int = 0  # tokens of prompt + completion that have gone through the model
    admitted_at: int = -1
    stage: str = "queued"  # "queued", "prefilling" or "decoding": which of the scheduler's lists holds it

    @property
    def id(self) -> str:
        return self.request.id

    @property
    def tokens(self) -> list[int]:
        """Everything known of the sequence: prompt, then what it has produced."""
        return self.request.input_ids + self.output.completion_ids

    @property
    def n_known(self) -> int:
        return len(self.request.input_ids) + len(self.output.completion_ids)

    def max_total(self) -> int:
        # the last produced token is never fed back (tokasaurus/manager/types.py:117-122)
        return len(self.request.input_ids) + self.request.max_num_tokens - 1


@dataclass
class ScheduledPortion:
    seq: Sequence
    start: int
    n_tokens: int
    samples: bool  # the last of these tokens yields the sequence's next token
    from_device: bool  # single token that is still in the device's last-token table


@dataclass
class StepPlan:
    portions: list[ScheduledPortion] = field(default_factory=list)
    bumped: list[str] = field(default_factory=list)

    @property
    def n_tokens(self) -> int:
        return sum(p.n_tokens for p in self.portions)


class Scheduler:
    def __init__(self, cache: CacheManager, max_tokens_per_forward: int, max_seqs_per_forward: int,
                 max_num_tokens_per_request: int | None = None, eos_token_ids: tuple[int, ...] = (),
                 kv_reserve_fraction: float = 1.0, bump_city_population_me: bool = False,
                 sanity_checks: bool = False, greedy_prefill: bool = True, prefill_round_up_multiple: int = 16,
                 admission: str = "reserve"):
        """``admission``: how a queued sequence gets in.  ``"reserve"``: its prompt's pages must be free after
        ``kv_reserve_fraction`` of what the running sequences can still ask for is set aside (1.0: the worst case,
        nothing is ever pushed out; 0, or ``bump_city_population_me``: nothing is set aside).  ``"simulate"``: the
        pages in use at every future step are worked out as if each sequence ran to its longest and then gave its
        pages back, and the sequence gets in if the highest of these, with it, fits the pool
        (``_simulated_peak``; the reference decides so, tokasaurus/manager/scheduler.py:46-216): sequences that
        end at different times share room that a worst-case reserve counts for each of them."""
        if admission not in ("reserve", "simulate"):
            raise ValueError(f"admission={admission!r}: 'reserve' or 'simulate'")
        self.admission = admission
        self.cache = cache
        self.greedy_prefill = greedy_prefill
        self.prefill_multiple = max(1, int(prefill_round_up_multiple))
        self.max_tokens = max_tokens_per_forward
        self.max_seqs = max_seqs_per_forward
        self.max_request_tokens = max_num_tokens_per_request
        self.eos = set(eos_token_ids)
        self.reserve_fraction = 0.0 if bump_city_population_me else kv_reserve_fraction
        self.sanity_checks = sanity_checks
        self.queued: deque[Sequence] = deque()
        self.prefilling: list[Sequence] = []
        self.decoding: list[Sequence] = []
        self._live_ids: set[str] = set()  # ids of the requests that are queued or running
        self._counter = 0
        self._admissions = 0
        self.stats = dict(steps=0, prefill_tokens=0, decode_tokens=0, bumps=0, finished=0)

    # ------------------------------------------------------------------ intake
    def add_request(self, request: Request) -> Sequence:
        request.sampling_params.validate()
        n = len(request.input_ids)
        if n == 0:
            raise ValueError(f"request {request.id!r} has an empty prompt")
        if request.max_num_tokens <= 0:
            raise ValueError(f"request {request.id!r}: max_num_tokens must be positive")
        total = n + request.max_num_tokens
        if self.max_request_tokens is not None and total > self.max_request_tokens:
            raise RequestTooLongError(
                f"request {request.id!r}: prompt {n} + max_num_tokens {request.max_num_tokens} exceeds "
                f"max_num_tokens_per_request={self.max_request_tokens}")
        for g, group in enumerate(self.cache.groups):
            need = self.cache.pages_for(total - 1)
            if group.need.window:  # the least with which a token still sees its whole window
                need = min(need, self.cache.pages_for(group.need.window + 1) + 1)
            if need > group.allocator.num_pages:
                raise RequestTooLongError(
                    f"request {request.id!r} can need {need} pages of cache group {g}, its pool has "
                    f"{group.allocator.num_pages}")
        if request.id in self._live_ids:
            raise ValueError(f"request id {request.id!r} is already queued or running (the cache is keyed by it)")
        seq = Sequence(request, self._counter, RequestOutput(request.id))
        self._counter += 1
        self.queued.append(seq)
        self._live_ids.add(request.id)
        return seq

    def has_work(self) -> bool:
        return bool(self.queued or self.prefilling or self.decoding)

    def running(self) -> list[Sequence]:
        return self.decoding + self.prefilling

    # ------------------------------------------------------------------ pages
    def _still_needed(self, seq: Sequence, g: int, held: int | None = None) -> int:
        """Pages of cache group ``g`` that the sequence can still ask for on top of the ``held`` it holds (None:
        what its table holds now; 0 for a sequence that is not admitted yet).  Every group's table grows with the
        sequence's length; in a group with a window, pages behind the window come back, so a sequence never holds
        more than the window and one step's tokens take."""
        group = self.cache.groups[g]
        total = self.cache.pages_for(seq.max_total())
        if held is None:
            rc = self.cache.requests[seq.id]
            allocated, held = len(rc.tables[g]), len(rc.tables[g]) - rc.released[g]
        else:
            allocated = held
        need = max(0, total - allocated)
        if group.need.window:
            need = min(need, max(0, self._most_live(g) - held))
        return need

    def _most_live(self, g: int) -> int:
        """Most pages a sequence holds at a time in the windowed group ``g``: the window, a step's tokens (and the
        one token of a step launched ahead) and a page for where the window starts inside a page."""
        return self.cache.pages_for(self.cache.groups[g].need.window + self.max_tokens + 1) + 1

    def _first_windowed_tokens(self, seq: Sequence) -> int:
        """How far windowed groups are filled at admission: the first step's tokens at most; the rest of a prompt
        takes its pages there portion by portion (``_fit_portion``)."""
        return min(seq.n_known, self.max_tokens)

    def _headroom(self) -> list[int]:
        """Per cache group: free pages less what running sequences may still ask for, scaled by the reserve fraction."""
        f = self.reserve_fraction
        out = []
        for g, group in enumerate(self.cache.groups):
            reserved = 0
            if f > 0:
                reserved = int(sum(self._still_needed(s, g) for s in self.running()) * f + 0.999999)
            out.append(group.allocator.num_free - reserved)
        return out

    def _admission_need(self, seq: Sequence) -> list[int]:
        """Per cache group: pages a queued sequence takes at admission (its whole prompt, as the reference's
        ``allocate_with_prefix_match`` does) plus its share of the reserve."""
        full = self.cache.pages_for(seq.n_known)
        windowed = self.cache.pages_for(self._first_windowed_tokens(seq))
        f = self.reserve_fraction
        out = []
        for g, group in enumerate(self.cache.groups):
            first_need = windowed if group.need.window else full
            out.append(first_need + (int(max(0, self._still_needed(seq, g, first_need)) * f + 0.999999) if f > 0 else 0))
        return out

    def _simulated_peak(self, candidates: list[Sequence] = ()) -> list[int]:
        """Per cache group: the most pages in use at any step from now on, if every running sequence, and then
        ``candidates`` (admitted now, fed after the prompts that are already on their way), decodes a token a step
        up to its longest and gives its pages back when it ends, and no one else comes.  Between two ends the use only
        grows, so the highest use is just before some sequence ends: these moments are looked at (all of them up to
        256 sequences; beyond that 256 of them, each standing for the interval since the one before it with
        everything alive in it at its length of the interval's end, which can only overstate).

        What this rests on, as in the reference (``calc_block_usage_over_time``,
        tokasaurus/manager/scheduler.py:46-216, where an early-stop predictor may shorten the lengths; here they are
        the requests' limits, so ends on a stop token only free pages sooner): prompts go through as a greedy
        prefill feeds them, in the order of admission.  If they go slower than that (a paced prefill), a sequence
        lives longer than assumed and pushing out remains the last resort."""
        cache = self.cache
        seqs = self.decoding + self.prefilling + list(candidates)
        if not seqs:
            return [0] * len(cache.groups)
        n_dec = len(self.decoding)
        start = np.zeros(len(seqs), dtype=np.int64)   # step at which the sequence decodes its first token
        base = np.zeros(len(seqs), dtype=np.int64)    # tokens it has in the cache then
        for i, s in enumerate(self.decoding):
            base[i] = s.fed
        # The prompts, step by step as a greedy prefill feeds them: what the decoding sequences leave of the token
        # budget goes to the prompts in order, and a prompt that is through decodes from the next step on (and takes
        # a token of the budget itself).
        ends = sorted(s.max_total() - s.fed for s in self.decoding)   # a decoding sequence runs in steps 0 .. end - 1
        through: list[tuple[int, int]] = []                           # (first, one past the last) decoding step
        left = [s.n_known - (s.fed if s.stage == "prefilling" else 0) for s in seqs[n_dec:]]
        at, k = 0, 0
        while at < len(left):
            running = len(ends) - bisect.bisect_right(ends, k) + sum(1 for a, b in through if a <= k < b)
            budget = self.max_tokens - running
            while budget > 0 and at < len(left):
                take = min(budget, left[at])
                left[at] -= take
                budget -= take
                if left[at] == 0:
                    s = seqs[n_dec + at]
                    start[n_dec + at] = k + 1
                    base[n_dec + at] = s.n_known
                    through.append((k + 1, k + 1 + s.max_total() - s.n_known))
                    at += 1
            k += 1
        end = start + np.asarray([s.max_total() for s in seqs], dtype=np.int64) - base  # its last step
        end = np.maximum(end, start)
        moments = np.unique(end)
        if moments.shape[0] > 256:
            moments = moments[np.unique(np.linspace(0, moments.shape[0] - 1, 256).astype(np.int64))]
        before = np.concatenate([[-1], moments[:-1]])
        alive = end[None, :] > before[:, None]                                    # [moments, sequences]
        at = np.minimum(moments[:, None], end[None, :])
        tokens = base[None, :] + np.maximum(0, at - start[None, :])
        pages = -(-tokens // cache.page_size)
        peaks = []
        for g, group in enumerate(cache.groups):
            p = np.minimum(pages, self._most_live(g)) if group.need.window else pages
            peaks.append(int((p * alive).sum(axis=1).max()))
        return peaks

    def _min_free(self) -> int:
        free = self.cache.num_free_pages()
        return min(free) if free else 1 << 30

    def _admit(self) -> None:
        if self.admission == "simulate":
            for seq in self._fitting_by_simulation():
                self._take_in(seq)
            return
        room = None  # the headroom, worked out once and kept up to date while sequences get in
        while self.queued and len(self.prefilling) + len(self.decoding) < self.max_seqs \
                and self.cache.slots.num_free > 0:
            seq = self.queued[0]
            if room is None:
                room = self._headroom()
            need = self._admission_need(seq)
            if any(r < n for r, n in zip(room, need)):
                break
            room = [r - n for r, n in zip(room, need)]
            self._take_in(seq)

    def _take_in(self, seq: Sequence) -> None:
        """Admit the head of the queue: a slot, the prompt's pages, into the list of those in prompt."""
        assert self.queued[0] is seq
        self.queued.popleft()
        self.cache.admit(seq.id)
        self.cache.ensure_capacity(seq.id, seq.n_known, windowed_tokens=self._first_windowed_tokens(seq))
        seq.fed = 0
        seq.admitted_at = self._admissions
        self._admissions += 1
        seq.stage = "prefilling"
        self.prefilling.append(seq)

    def _fitting_by_simulation(self) -> list[Sequence]:
        """The longest head of the queue that gets in under admission by simulation: slots for all of them, their
        prompts' pages free now, and the simulated peak with all of them within every pool.  A longer head never
        has a lower peak, so the longest one that fits is found by halving (the reference takes its queue in
        batches with a binary back-off too, tokasaurus/manager/manager.py:561-656): a few simulations an
        admission round instead of one a sequence."""
        limit = min(len(self.queued), self.max_seqs - len(self.prefilling) - len(self.decoding),
                    self.cache.slots.num_free)
        if limit <= 0:
            return []
        head = [self.queued[i] for i in range(limit)]
        groups = self.cache.groups
        # how many of them find their first pages free
        free = [g.allocator.num_free for g in groups]
        for n, seq in enumerate(head):
            for i, g in enumerate(groups):
                free[i] -= self.cache.pages_for(self._first_windowed_tokens(seq) if g.need.window else seq.n_known)
            if min(free) < 0:
                head = head[:n]
                break

        def fits(k: int) -> bool:
            return all(peak <= g.allocator.num_pages for peak, g in zip(self._simulated_peak(head[:k]), groups))

        if not head or fits(len(head)):
            return head
        lo, hi = 0, len(head) - 1  # fits(lo) holds (with nobody new the running ones fit); find the largest that does
        while lo < hi:
            mid = (lo + hi + 1) // 2
            if fits(mid):
                lo = mid
            else:
                hi = mid - 1
        return head[:lo]

    def _bump_one(self, protect: Sequence) -> Sequence | None:
        """Push out the most recently admitted running sequence other than ``protect``."""
        victims = [s for s in self.running() if s is not protect]
        if not victims:
            return None
        victim = max(victims, key=lambda s: s.admitted_at)
        self._release(victim)
        victim.fed = 0
        victim.output.num_preemptions += 1
        self.queued.appendleft(victim)
        self.stats["bumps"] += 1
        return victim

    def _release(self, seq: Sequence) -> None:
        if seq.stage == "decoding":
            self.decoding.remove(seq)
        elif seq.stage == "prefilling":
            self.prefilling.remove(seq)
        seq.stage = "queued"
        self.cache.free(seq.id)

    # ------------------------------------------------------------------ one step
    def schedule(self) -> StepPlan:
        plan = StepPlan()
        # 1. pages for the next token of every decoding sequence, pushing sequences out if the pool is dry
        for seq in sorted(self.decoding, key=lambda s: s.admitted_at):
            if seq.stage != "decoding":
                continue  # was pushed out a moment ago
            while True:
                try:
                    self.cache.ensure_capacity(seq.id, seq.fed + 1)
                    break
                except NoSpaceError:
                    victim = self._bump_one(protect=seq)
                    if victim is None:
                        raise
                    plan.bumped.append(victim.id)
        # 2. admission
        self._admit()
        if not self.decoding and not self.prefilling and self.queued:
            seq = self.queued[0]
            raise NoSpaceError(
                f"request {seq.id!r} needs {self.cache.pages_for(seq.n_known)} pages for its prompt and "
                f"{self._min_free()} are free with nothing running")
        # 3. the batch: one token for each decoding sequence, then prompt portions under the budget
        for seq in self.decoding:
            plan.portions.append(ScheduledPortion(seq, seq.fed, 1, True, from_device=True))
        budget = self._prefill_budget(self.max_tokens - len(plan.portions))
        for seq in list(self.prefilling):
            if budget <= 0:
                break
            if seq.stage != "prefilling":
                continue  # was pushed out a moment ago
            n = self._fit_portion(seq, min(budget, seq.n_known - seq.fed))
            while n == 0 and not plan.portions:
                # nothing else runs in this step and this prompt cannot go on: push out a later sequence for it
                victim = self._bump_one(protect=seq)
                if victim is None:
                    raise NoSpaceError(
                        f"request {seq.id!r} cannot go on at token {seq.fed}: a windowed cache group has "
                        f"{self._min_free()} free pages with nothing else running")
                plan.bumped.append(victim.id)
                n = self._fit_portion(seq, min(budget, seq.n_known - seq.fed))
            if n == 0:
                continue
            plan.portions.append(ScheduledPortion(seq, seq.fed, n, seq.fed + n == seq.n_known, from_device=False))
            budget -= n
        return plan

    def _fit_portion(self, seq: Sequence, n: int) -> int:
        """Pages of the windowed groups for the next ``n`` prompt tokens of ``seq``; fewer tokens if their pools
        have no more, 0 if not one token fits.  (The groups that see all keys hold the whole prompt since
        admission.)"""
        rc = self.cache.requests[seq.id]
        for g, group in enumerate(self.cache.groups):
            if group.need.window:
                reach = (len(rc.tables[g]) + group.allocator.num_free) * self.cache.page_size
                n = min(n, reach - seq.fed)
        if n <= 0:
            return 0
        self.cache.ensure_capacity(seq.id, seq.n_known, windowed_tokens=seq.fed + n)
        return n

    # ------------------------------------------------------------------ how much of the prompts goes into a step
    def _prefill_budget(self, room: int) -> int:
        """Prompt tokens for this step, of the ``room`` that the decoding sequences leave under
        ``max_tokens_per_forward``.  With ``greedy_prefill`` (the default, here and in the reference): all that
        fits.  Without it, as the reference decides (tokasaurus/manager/scheduler.py:604-637): all that fits when
        nobody waits in the queue (everything outstanding is in the cache already, so it may as well start);
        exactly the first prompt when nobody decodes; else a paced amount (``_paced_prefill``), rounded up to
        ``prefill_round_up_multiple``."""
        if self.greedy_prefill or not self.prefilling or not self.queued:
            return room
        if not self.decoding:
            first = self.prefilling[0]
            return min(room, first.n_known - first.fed)
        pace = self._paced_prefill()
        if pace == float("inf"):
            return room
        m = self.prefill_multiple
        return min(room, max(m, -(-int(pace + 0.999999) // m) * m))

    def _paced_prefill(self) -> float:
        """Prompt tokens a step such that the prompts are through the model just when the cache has room for what
        follows them, instead of all at once at the cost of the decoding sequences' latency: the idea of the
        reference's ``calc_prefill_per_forward`` (tokasaurus/manager/scheduler.py:434-538) in this scheduler's
        own page accounting.  The decoding sequences are taken in the order in which they end by length; after
        each end, queued sequences are admitted in thought, first come first served, while slots and pages
        (those the ended sequences give back, less what the admitted ones reserve) allow; the prompt tokens
        outstanding by then, spread over the steps until then, are one candidate, and the smallest candidate
        wins.  Once the whole queue fits, later ends ask for nothing slower."""
        cache, f = self.cache, self.reserve_fraction
        groups = range(len(cache.groups))
        outstanding = sum(s.n_known - s.fed for s in self.prefilling)
        available = self._headroom()
        running = len(self.prefilling) + len(self.decoding)
        slots = min(self.max_seqs, running + cache.slots.num_free)
        queue = list(self.queued)
        at = 0  # next queued sequence to admit in thought
        onboarded = 0
        pace = float("inf")
        for seq in sorted(self.decoding, key=lambda s: s.max_total() - s.fed):
            steps = max(1, seq.max_total() - seq.fed)  # steps from now after which this sequence has ended
            rc = cache.requests[seq.id]
            for g in groups:
                # what it holds comes back, and its share of the reserve is no longer set aside
                available[g] += len(rc.tables[g]) - rc.released[g] + int(f * self._still_needed(seq, g))
            running -= 1
            while at < len(queue) and running < slots:
                need = self._admission_need(queue[at])
                if any(n > a for n, a in zip(need, available)):
                    break
                for g in groups:
                    available[g] -= need[g]
                onboarded += queue[at].n_known
                running += 1
                at += 1
            if at == len(queue):
                break
            pace = min(pace, (outstanding + onboarded) / steps)
        return pace

    def complete(self, plan: StepPlan, sampled: list[int], logprobs: list[float] | None = None,
                 topk: list[tuple[list[int], list[float]]] | None = None) -> list[RequestOutput]:
        """Account for a step that has run.  ``sampled`` holds one id per portion with ``samples``,
        in plan order.  Returns the outputs of the requests that ended."""
        finished: list[RequestOutput] = []
        k = 0
        self.stats["steps"] += 1
        for p in plan.portions:
            seq = p.seq
            seq.fed += p.n_tokens
            if p.from_device:
                self.stats["decode_tokens"] += 1
            else:
                self.stats["prefill_tokens"] += p.n_tokens
            self.cache.release_behind_window(seq.id, seq.fed)
            if not p.samples:
                continue
            tok = int(sampled[k])
            seq.output.completion_ids.append(tok)
            if logprobs is not None:
                seq.output.logprobs.append(float(logprobs[k]))
            if topk is not None and seq.request.topk_logprobs:
                seq.output.topk_ids.append(topk[k][0][: seq.request.topk_logprobs])
                seq.output.topk_logprobs.append(topk[k][1][: seq.request.topk_logprobs])
            k += 1
            if seq.stage == "prefilling":
                self.prefilling.remove(seq)
                self.decoding.append(seq)
                seq.stage = "decoding"
            reason = None
            if (not seq.request.ignore_eos and tok in self.eos) or tok in seq.request.stop_token_ids:
                reason = "stop"
            elif len(seq.output.completion_ids) >= seq.request.max_num_tokens:
                reason = "length"
            if reason:
                seq.output.finish_reason = reason
                self._release(seq)
                self._live_ids.discard(seq.id)
                finished.append(seq.output)
                self.stats["finished"] += 1
        if k != len(sampled):
            raise ValueError(f"the step sampled {len(sampled)} tokens, the plan wanted {k}")
        if self.sanity_checks:
            self.cache.check()
        return finished
