"""Continuous-batching scheduler: admission, prompt portions under a token budget,
decoding, finishing, and what happens when pages run out.

Taken from the reference: first-come admission behind ``max_concurrent_requests``,
re-run whenever a request finishes (mstar/conductor/conductor.py:573-607, 794-825); a
cap on requests per batch (largest captured decode batch, 64: mstar/engine/
cuda_graph_runner.py:45); finishing on the stop token unless ``ignore_eos``, or on
``max_output_tokens`` (mstar/model/orpheus/submodules.py:277-290, mstar/model/base.py:30).

Designed here (the reference has neither a token budget, nor prompt portions, nor
mixed batches, mstar/worker/micro_scheduler.py:97-103, 272-273): each step first gives
every running request that is decoding its one token, then fills the rest of
``max_num_batched_tokens`` with prompt portions, oldest request first, admitting
waiting requests while slots and pages allow.

When pages run out: the reference holds the batch and retries every 50 ms, optionally
offloading a victim's pages to host memory (mstar/worker/worker.py:1245-1293).  Here
the decision is pre-emption by recomputation: the request admitted last gives back
all its pages and returns to the head of the waiting queue; its prompt plus the tokens
it has generated are computed again once all of that fits in the free pages.  Decoding requests are never
starved by prompts: prompt portions only take pages that decoding does not need in
this step.  A request that cannot fit even alone in the whole pool is finished with
reason "cache_exhausted" instead of waiting forever.
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from typing import Callable, Hashable, Optional, Sequence

from ..cache.manager import CacheManager
from ..sampling.params import SamplingParams


@dataclass
class SchedulerConfig:
    max_num_batched_tokens: int = 2048
    max_concurrent_requests: Optional[int] = None   # None: as many as there are slots
    max_batch_size: int = 64                        # requests per step
    # positions the model was built for (max_position_embeddings; the reference's
    # max_seq_len, mstar/model/orpheus/orpheus_model.py:88-95); None: no limit
    max_seq_len: Optional[int] = None

    def validate(self) -> None:
        if self.max_num_batched_tokens < 1:
            raise ValueError("max_num_batched_tokens must be >= 1")
        if self.max_batch_size < 1:
            raise ValueError("max_batch_size must be >= 1")
        if self.max_concurrent_requests is not None and self.max_concurrent_requests < 1:
            raise ValueError("max_concurrent_requests must be >= 1")
        if self.max_seq_len is not None and self.max_seq_len < 2:
            raise ValueError("max_seq_len must be >= 2")


@dataclass
class Request:
    request_id: Hashable
    prompt: list
    params: SamplingParams
    output: list = field(default_factory=list)
    num_computed: int = 0          # tokens whose keys and values are in the cache
    status: str = "waiting"        # waiting | running | finished
    finish_reason: Optional[str] = None
    slot: int = -1
    preemptions: int = 0
    # most tokens it may generate: max_output_tokens, cut to what the model's positions
    # leave after the prompt (set when the request is added)
    output_limit: Optional[int] = None

    def all_tokens(self) -> list:
        return self.prompt + self.output

    def num_pending(self) -> int:
        return len(self.prompt) + len(self.output) - self.num_computed


@dataclass
class ScheduledEntry:
    request: Request
    tokens: list
    samples: bool      # the portion ends at the request's last token: sample after it


@dataclass
class StepPlan:
    entries: list = field(default_factory=list)
    admitted: list = field(default_factory=list)
    preempted: list = field(default_factory=list)
    finished: list = field(default_factory=list)   # finished without running (errors)

    def num_tokens(self) -> int:
        return sum(len(e.tokens) for e in self.entries)


class Scheduler:
    def __init__(self, config: SchedulerConfig, manager: CacheManager,
                 stop_token_ids: Sequence[int] = (),
                 admit: Optional[Callable] = None, release: Optional[Callable] = None):
        config.validate()
        self.config = config
        self.manager = manager
        self.stop_token_ids = frozenset(int(t) for t in stop_token_ids)
        self._admit = admit or manager.add_request
        self._release = release or manager.free_request
        self.waiting: deque = deque()
        self.running: list = []       # in order of admission
        self.finished: list = []

    # -- queue ------------------------------------------------------------
    def add(self, request: Request) -> None:
        if not request.prompt:
            raise ValueError(f"request {request.request_id!r} has an empty prompt")
        request.params.validate()
        limit = request.params.max_output_tokens
        longest = self.config.max_seq_len
        if longest is not None:
            if len(request.prompt) >= longest:
                raise ValueError(
                    f"request {request.request_id!r} has a prompt of {len(request.prompt)} "
                    f"tokens; the model takes sequences of up to {longest} (prompt and "
                    "generated tokens together)")
            # it then finishes with reason "length" where the positions end
            limit = min(limit, longest - len(request.prompt))
        request.output_limit = limit
        request.status = "waiting"
        self.waiting.append(request)

    def abort(self, request_id: Hashable) -> bool:
        for r in list(self.waiting):
            if r.request_id == request_id:
                self.waiting.remove(r)
                self._finish(r, "abort", held=False)
                return True
        for r in self.running:
            if r.request_id == request_id:
                self._finish(r, "abort", held=True)
                return True
        return False

    def has_work(self) -> bool:
        return bool(self.waiting or self.running)

    def may_admit(self) -> bool:
        """Whether the next ``schedule`` could take a request from the waiting queue: one
        waits, and neither the cap on running requests, the batch size nor the state slots
        stand in the way (pages are not looked at)."""
        if not self.waiting:
            return False
        cap = self.config.max_concurrent_requests
        if cap is not None and len(self.running) >= cap:
            return False
        if len(self.running) >= self.config.max_batch_size:
            return False
        return self.manager.free_slots() >= 1

    # -- helpers ----------------------------------------------------------
    def _finish(self, r: Request, reason: str, held: bool) -> None:
        if held:
            self._release(r.request_id)
            self.running.remove(r)
        r.status = "finished"
        r.finish_reason = reason
        self.finished.append(r)

    def _capacity_tokens(self) -> int:
        """Tokens one request can hold if it has every page of the smallest pool."""
        if not self.manager.groups:
            return 1 << 62
        return min(g.num_pages * g.page_size for g in self.manager.groups)

    def _need(self, r: Request, count: int) -> list:
        """New pages per group that ``count`` more tokens of ``r`` take.  The need of a
        batch is the sum over its requests, so a step's bookkeeping is one call per
        request and decision instead of one per batch tried."""
        return self.manager.pages_needed([r.request_id], [count])

    def _free(self) -> list:
        return [self.manager.free_pages(g) for g in range(len(self.manager.groups))]

    def _preempt_last(self, plan: StepPlan, keep: Optional[Request] = None) -> bool:
        """Take the pages of the request admitted last (other than ``keep``)."""
        for victim in reversed(self.running):
            if victim is keep:
                continue
            self._release(victim.request_id)
            self.running.remove(victim)
            victim.status = "waiting"
            victim.num_computed = 0
            victim.slot = -1
            victim.preemptions += 1
            self.waiting.appendleft(victim)
            plan.preempted.append(victim)
            plan.entries = [e for e in plan.entries if e.request is not victim]
            return True
        return False

    # -- one step ---------------------------------------------------------
    def schedule(self) -> StepPlan:
        cfg = self.config
        plan = StepPlan()
        budget = cfg.max_num_batched_tokens
        groups = range(len(self.manager.groups))
        chosen: list = []        # requests of this step, their token counts and page needs
        counts: list = []
        needs: list = []
        total = [0 for _ in groups]      # pages the chosen requests take, per group
        free = self._free()

        def fits(extra: list) -> bool:
            return all(total[g] + extra[g] <= free[g] for g in groups)

        def take(r: Request, n: int, need: list) -> None:
            chosen.append(r)
            counts.append(n)
            needs.append(need)
            for g in groups:
                total[g] += need[g]

        def after_preemption() -> None:
            """A victim gave its pages back: it leaves the batch, the pools have grown."""
            nonlocal chosen, counts, needs, total, free
            kept = [i for i, c in enumerate(chosen) if c.status == "running"]
            chosen = [chosen[i] for i in kept]
            counts = [counts[i] for i in kept]
            needs = [needs[i] for i in kept]
            total = [sum(n[g] for n in needs) for g in groups]
            free = self._free()

        def portion(r: Request) -> tuple:
            """Largest portion of r's pending tokens that the budget and the free pages
            (after what is already chosen) allow, with its page need; 0 if not even one
            token fits."""
            hi = min(r.num_pending(), budget)
            if hi <= 0:
                return 0, None
            need = self._need(r, hi)
            if fits(need):
                return hi, need
            lo, lo_need = 0, None            # largest count known to fit (0: none yet)
            while hi - lo > 1:               # invariant: lo fits (or is 0), hi does not
                mid = (lo + hi) // 2
                need = self._need(r, mid)
                if fits(need):
                    lo, lo_need = mid, need
                else:
                    hi = mid
            return lo, lo_need

        # 1. one token for every request that is decoding, oldest first
        for r in list(self.running):
            if r.status != "running" or r.num_pending() != 1:
                continue
            if len(chosen) >= cfg.max_batch_size or budget < 1:
                break
            need = self._need(r, 1)
            while not fits(need):
                if not self._preempt_last(plan, keep=r):
                    break
                after_preemption()
            if not fits(need):
                # alone and still no page: the pool cannot hold this request
                self._finish(r, "cache_exhausted", held=True)
                plan.finished.append(r)
                free = self._free()
                continue
            take(r, 1, need)
            budget -= 1

        # 2. prompt portions of running requests, oldest first
        decoding = {id(r) for r in chosen}
        for r in list(self.running):
            if id(r) in decoding or r.num_pending() < 1:
                continue
            if len(chosen) >= cfg.max_batch_size or budget < 1:
                break
            n, need = portion(r)
            if n > 0:
                take(r, n, need)
                budget -= n

        # 3. admit waiting requests while slots, the cap and pages allow
        while (self.waiting and not plan.preempted and budget >= 1
               and len(chosen) < cfg.max_batch_size):
            cap = cfg.max_concurrent_requests
            if cap is not None and len(self.running) >= cap:
                break
            if self.manager.free_slots() < 1:
                break
            r = self.waiting[0]
            if len(r.prompt) + len(r.output) + 1 > self._capacity_tokens():
                self.waiting.popleft()
                self._finish(r, "cache_exhausted", held=False)
                plan.finished.append(r)
                continue
            r.slot = self._admit(r.request_id)
            n, need = portion(r)
            if n > 0 and r.preemptions and not fits(self._need(r, r.num_pending() + 1)):
                n = 0    # a pre-empted request returns only when all it had fits again
            if n <= 0:
                self._release(r.request_id)   # no page for even one token now
                r.slot = -1
                break
            self.waiting.popleft()
            r.status = "running"
            self.running.append(r)
            plan.admitted.append(r)
            take(r, n, need)
            budget -= n

        # nothing can run although requests hold pages: they block one another (or one
        # alone is too large).  The oldest keeps its pages; the newest gives its up.
        if not chosen and self.running and not plan.preempted:
            oldest = self.running[0]
            if len(self.running) == 1:
                self._finish(oldest, "cache_exhausted", held=True)
                plan.finished.append(oldest)
            else:
                self._preempt_last(plan, keep=oldest)

        for r, n in zip(chosen, counts):
            if n == 1 and r.num_pending() == 1:
                toks = [r.output[-1] if r.output else r.prompt[-1]]
            else:
                toks = r.all_tokens()[r.num_computed:r.num_computed + n]
            plan.entries.append(ScheduledEntry(r, toks, r.num_computed + n == len(r.prompt)
                                               + len(r.output)))
        return plan

    # -- after the forward pass -------------------------------------------
    # A step's bookkeeping is split in two so that the engine can launch the next step
    # before it has read this one's tokens: ``advance`` right after the launch (counts, a
    # place for each sampled token, the finish on max_output_tokens, which needs no
    # value), ``resolve`` when the values have arrived (the finish on a stop token, which
    # therefore takes effect one step late, as in the reference's worker,
    # mstar/worker/worker.py:1612-1629).  ``update`` is both at once.
    def advance(self, plan: StepPlan) -> None:
        """The plan has been launched: its tokens count as computed, every entry that
        samples gets a place (None) at the end of its request's output."""
        for e in plan.entries:
            r = e.request
            r.num_computed += len(e.tokens)
            if not e.samples:
                continue
            r.output.append(None)
            limit = r.params.max_output_tokens if r.output_limit is None else r.output_limit
            if len(r.output) >= limit and r.status == "running":
                self._finish(r, "length", held=True)

    def resolve(self, plan: StepPlan, sampled: dict) -> list:
        """``sampled``: request id -> token for every entry of the (advanced) plan with
        ``samples``.  Fills the places, finishes on stop tokens and frees.  Returns the
        requests that finished with this step."""
        done = []
        for e in plan.entries:
            if not e.samples:
                continue
            r = e.request
            where = len(r.output)              # the first of the (at most two) open places
            while where > 0 and r.output[where - 1] is None:
                where -= 1
            if where == len(r.output):
                continue        # stopped a step ago: this token was computed in vain
            tok = int(sampled[r.request_id])
            r.output[where] = tok
            if r.finish_reason == "abort":
                continue                       # given up while this step was under way
            if (not r.params.ignore_eos) and tok in self.stop_token_ids:
                del r.output[where + 1:]       # the place the step after took, if any
                if r.status == "finished":
                    r.finish_reason = "stop"   # the last allowed token was a stop token
                elif r.status == "running":
                    self._finish(r, "stop", held=True)
                else:                          # pre-empted meanwhile: it holds nothing
                    self.waiting.remove(r)
                    self._finish(r, "stop", held=False)
                done.append(r)
            elif r.status == "finished" and where == len(r.output) - 1:
                done.append(r)                 # finished on its length, now complete
        return done

    def update(self, plan: StepPlan, sampled: dict) -> list:
        """``advance`` and ``resolve`` in one: for callers that read a step's tokens before
        they plan the next."""
        self.advance(plan)
        return self.resolve(plan, sampled)
