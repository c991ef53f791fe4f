"""Python entry point: load a model folder, generate tokens for token-id prompts.

    from mstar_b200 import LLM, SamplingParams
    llm = LLM("/models/orpheus", dtype="bfloat16")
    results = llm.generate([[128259, 5, 17, 128009]], SamplingParams(temperature=0))

The reference's Python entry point is an HTTP client (mstar/__init__.py:17-30) and its
engine options live in a YAML file (``max_concurrent_requests``, ``kv_cache:`` with
``page_size`` and ``max_num_pages``; docs/serving.rst:161-238, mstar/engine/kv_store.py:
71-101); the same option names are constructor arguments here.  Prompts are token ids:
tokenisation happens in the reference's API server, which is outside this engine.
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Hashable, Optional, Sequence

import torch

from ..cache.storage import CacheStorage, bytes_per_page, plan_groups
from ..config.base import GenerationDefaults
from ..sampling.params import SamplingParams
from ..sampling.sampler import Sampler
from .model import Model, load_model
from .scheduler import Request, Scheduler, SchedulerConfig
from .step import StepEntry, Stepper


@dataclass
class GenerationResult:
    request_id: Hashable
    prompt_token_ids: list
    token_ids: list
    finish_reason: str
    preemptions: int = 0


@dataclass
class EngineStats:
    steps: int = 0
    prompt_tokens: int = 0
    generated_tokens: int = 0
    preemptions: int = 0
    step_seconds: list = field(default_factory=list)


class LLM:
    def __init__(self, model, dtype: str = "bfloat16", device: str = "cuda:0", *,
                 page_size: int = 16, max_num_pages: Optional[int] = None,
                 kv_cache_memory_fraction: float = 0.85,
                 max_num_batched_tokens: int = 2048,
                 max_concurrent_requests: Optional[int] = 64, max_batch_size: int = 64,
                 log_stats: bool = False):
        """``model``: a folder with config.json and safetensors, or a built ``Model``.
        ``max_num_pages``: pages of ``page_size`` tokens per cache group; None sizes
        the pool from ``kv_cache_memory_fraction`` of the memory free after loading."""
        self.model: Model = model if isinstance(model, Model) else load_model(
            model, dtype=dtype, device=device)
        self.device = self.model.runtime.device
        slots = max_concurrent_requests or max_batch_size
        if max_num_pages is None:
            max_num_pages = self._pages_from_memory(page_size, kv_cache_memory_fraction)
        storage = CacheStorage(self.model.cache_needs, self.model.runtime.dtype, self.device,
                               page_size, max_num_pages, slots)
        self.stepper = Stepper(self.model, storage)
        self.sampler = Sampler(self.model.vocab_size, slots, self.device)
        cfg = self.model.config
        stops = cfg.stop_token_ids() if cfg is not None else ()
        self.scheduler = Scheduler(
            SchedulerConfig(max_num_batched_tokens=max_num_batched_tokens,
                            max_concurrent_requests=max_concurrent_requests,
                            max_batch_size=max_batch_size),
            storage.manager, stops, admit=self.stepper.add_request,
            release=self._release)
        self.log_stats = log_stats
        self.stats = EngineStats()
        self._auto_id = 0
        # a decode step that has been launched but whose tokens have not been read back
        self._inflight = None
        self.pipelined_steps = 0

    def _pages_from_memory(self, page_size: int, fraction: float) -> list:
        free, _ = torch.cuda.mem_get_info(self.device)
        windows, group_of = plan_groups(self.model.cache_needs)
        if not windows:
            return []
        per_group = int(free * fraction) // len(windows)
        pages = []
        for g in range(len(windows)):
            b = bytes_per_page(self.model.cache_needs, group_of, g, page_size,
                               self.model.runtime.dtype)
            pages.append(max(per_group // max(b, 1), 1))
        return pages

    def _release(self, request_id: Hashable) -> None:
        self.stepper.free_request(request_id)
        self.sampler.remove_request(request_id)

    # -- requests ---------------------------------------------------------
    def add_request(self, prompt_token_ids: Sequence[int],
                    sampling_params: Optional[SamplingParams] = None,
                    request_id: Optional[Hashable] = None) -> Hashable:
        if request_id is None:
            request_id = f"req-{self._auto_id}"
            self._auto_id += 1
        params = sampling_params or SamplingParams()
        vocab = self.model.vocab_size
        prompt = [int(t) for t in prompt_token_ids]
        if any(t < 0 or t >= vocab for t in prompt):
            raise ValueError(f"prompt of {request_id!r} has a token id outside [0, {vocab})")
        self.scheduler.add(Request(request_id, prompt, params))
        return request_id

    def has_unfinished(self) -> bool:
        return self.scheduler.has_work() or self._inflight is not None

    # -- one step ---------------------------------------------------------
    # Steady decoding is pipelined one step deep, as the reference's worker does
    # (mstar/worker/worker.py:2118-2211, 1328-1550: step N+1 is built and submitted
    # while step N runs, and a stop takes effect one step late, worker.py:1612-1629):
    # after launching step N the engine does not wait for its tokens; the next call
    # launches step N+1 for the same requests with the tokens taken on the device, and
    # only then reads step N's tokens back.  A request that turns out to have stopped at
    # step N has one token computed in vain; a request that reaches max_output_tokens is
    # foreseen and left out.

    def _launch(self, plan) -> tuple:
        """Run the plan's forward pass and sampling; tokens stay on the device."""
        entries = [StepEntry(e.request.request_id, e.tokens,
                             (len(e.tokens) - 1,) if e.samples else ())
                   for e in plan.entries]
        logits = self.stepper.step(entries)
        sampling = [e.request.request_id for e in plan.entries if e.samples]
        tokens = self.sampler.sample(sampling, logits) if sampling else None
        return sampling, tokens

    def _account(self, plan, sampled: dict) -> list:
        finished = self.scheduler.update(plan, sampled)
        self.stats.steps += 1
        self.stats.prompt_tokens += sum(len(e.tokens) for e in plan.entries if not (
            e.samples and len(e.tokens) == 1))
        self.stats.generated_tokens += len(sampled)
        return finished

    def _try_pipeline(self, prev) -> Optional[tuple]:
        """Launch the decode step that follows the in-flight one, if it can be foreseen:
        no waiting request could be admitted now (a slot that the in-flight step frees is
        filled one step late, as a stop takes effect one step late), and every request of
        the in-flight step was decoding.  Returns the new in-flight record, or None."""
        plan, sampling, tokens = prev
        if self.scheduler.may_admit() or tokens is None or len(sampling) != len(plan.entries):
            return None
        if any(len(e.tokens) != 1 for e in plan.entries):
            return None
        if len(plan.entries) != len(self.scheduler.running):
            return None
        keep = [i for i, e in enumerate(plan.entries)
                if len(e.request.output) + 1 < e.request.params.max_output_tokens]
        if not keep:
            return None
        requests = [plan.entries[i].request for i in keep]
        ids = [r.request_id for r in requests]
        from ..cache.manager import CacheExhausted
        from .scheduler import ScheduledEntry, StepPlan

        source = tokens if len(keep) == len(plan.entries) else tokens[
            torch.tensor(keep, dtype=torch.long, device=self.device)]
        try:
            logits = self.stepper.step_decode_from_device(ids, source)
        except CacheExhausted:
            return None                      # the scheduler decides who gives up pages
        if logits is None:
            return None
        next_tokens = self.sampler.sample(ids, logits)
        next_plan = StepPlan(entries=[ScheduledEntry(r, [None], True) for r in requests])
        self.pipelined_steps += 1
        return next_plan, ids, next_tokens

    def step(self) -> list:
        """Schedule and run one batch; returns the requests that finished."""
        t0 = time.perf_counter()
        finished: list = []
        if self._inflight is not None:
            prev = self._inflight
            nxt = self._try_pipeline(prev)                    # launch N+1 first ...
            plan, sampling, tokens = prev
            sampled = dict(zip(sampling, tokens.tolist()))    # ... then read N back
            finished += self._account(plan, sampled)
            if nxt is not None:
                # requests that stopped at step N ran step N+1 in vain: drop them
                nplan, nids, ntokens = nxt
                alive = [i for i, e in enumerate(nplan.entries) if e.request.status == "running"]
                if len(alive) != len(nplan.entries):
                    nplan.entries = [nplan.entries[i] for i in alive]
                    nids = [nids[i] for i in alive]
                    ntokens = ntokens[torch.tensor(alive, dtype=torch.long, device=self.device)] \
                        if alive else None
                for e in nplan.entries:                       # the token fed was step N's
                    e.tokens = [e.request.output[-1]]
                nxt = (nplan, nids, ntokens) if nplan.entries else None
            self._inflight = nxt
            if self.log_stats:
                self.stats.step_seconds.append(time.perf_counter() - t0)
            return finished
        plan = self.scheduler.schedule()
        finished += list(plan.finished)
        self.stats.preemptions += len(plan.preempted)
        for r in plan.admitted:
            self.sampler.add_request(r.request_id, r.params, r.slot, generated=r.output)
        if plan.entries:
            sampling, tokens = self._launch(plan)
            decode_only = (tokens is not None and len(sampling) == len(plan.entries)
                           and all(len(e.tokens) == 1 for e in plan.entries))
            if decode_only and self.stepper.cuda_graphs:
                self._inflight = (plan, sampling, tokens)     # read back at the next call
            else:
                sampled = dict(zip(sampling, tokens.tolist())) if sampling else {}
                finished += self._account(plan, sampled)
        elif not plan.preempted and not plan.finished and self.scheduler.has_work():
            raise RuntimeError("the scheduler can make no progress: no request fits the cache")
        if self.log_stats:
            self.stats.step_seconds.append(time.perf_counter() - t0)
        return finished

    def generate(self, prompts, sampling_params=None, request_ids=None) -> list:
        """Generate for one prompt (a list of token ids) or several (a list of lists).
        ``sampling_params``: one for all, or one per prompt.  Results come in the order
        of the prompts."""
        single = bool(prompts) and isinstance(prompts[0], int)
        if single:
            prompts = [prompts]
        n = len(prompts)
        if sampling_params is None or isinstance(sampling_params, SamplingParams):
            sampling_params = [sampling_params] * n
        if request_ids is None:
            request_ids = [None] * n
        if len(sampling_params) != n or len(request_ids) != n:
            raise ValueError("sampling_params and request_ids must match the prompts")
        ids = [self.add_request(p, sp, rid)
               for p, sp, rid in zip(prompts, sampling_params, request_ids)]
        done: dict = {}
        while self.has_unfinished():
            for r in self.step():
                done[r.request_id] = r
        results = [GenerationResult(i, done[i].prompt, done[i].output, done[i].finish_reason,
                                    done[i].preemptions) for i in ids]
        return results[0] if single else results

    def generation_defaults(self, folder) -> GenerationDefaults:
        return GenerationDefaults.from_folder(folder)
