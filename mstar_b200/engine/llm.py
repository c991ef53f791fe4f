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

from .. import ops
from ..cache.storage import CacheStorage, bytes_per_page, group_page_sizes, plan_groups
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
                 page_size: int = 64, max_num_pages: Optional[int] = None,
                 kv_cache_memory_fraction: float = 0.85,
                 max_num_batched_tokens: int = 2048,
                 max_concurrent_requests: Optional[int] = 64, max_batch_size: int = 64,
                 log_stats: bool = False):
        """``model``: a folder with config.json and safetensors, or a built ``Model``.
        ``page_size`` and ``max_num_pages``: tokens per page and pages of a cache group, one
        number for all groups or a list with one per group; ``max_num_pages`` None sizes the
        pools from ``kv_cache_memory_fraction`` of the memory free after loading."""
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
                            max_batch_size=max_batch_size,
                            max_seq_len=self.model.max_positions),
            storage.manager, stops, admit=self.stepper.add_request,
            release=self._release)
        self.log_stats = log_stats
        self.stats = EngineStats()
        self._auto_id = 0
        # the step that has been launched but whose tokens have not been read back: (plan,
        # ids of the requests it samples for, their tokens on the device, the pinned host
        # buffer they are copied to, the event after that copy)
        self._inflight = None
        self.pipelined_steps = 0
        self._reported = 0              # finished requests handed to the caller so far
        # pinned landing places of the sampled tokens: two steps can be under way
        # (one more element than tokens: the device's error word travels with them)
        self._host_tokens = [torch.empty(max(max_batch_size, 1) + 1, dtype=torch.int32,
                                         pin_memory=True) for _ in range(3)]
        self._error_word = ops.tcgen05_error_word(self.device)
        self._turn = 0
        self._copy_stream = torch.cuda.Stream(device=self.device)

    def _pages_from_memory(self, page_size, fraction: float) -> list:
        free, _ = torch.cuda.mem_get_info(self.device)
        windows, group_of = plan_groups(self.model.cache_needs)
        if not windows:
            return []
        sizes = group_page_sizes(page_size, len(windows))
        per_group = int(free * fraction) // len(windows)
        pages = []
        for g in range(len(windows)):
            b = bytes_per_page(self.model.cache_needs, group_of, g, sizes[g],
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

    def abort(self, request_id: Hashable) -> bool:
        """Give a request up, waiting or running: its pages and its slot return at once (a
        step under way that still computes for it is ordered before whatever uses them
        next, and its token is dropped when it arrives).  The request is handed back by a
        later ``step`` with finish reason "abort".  False if it is not known or has
        finished (the reference: mstar/conductor/conductor.py:764-792, removal deferred
        while a step is in flight, mstar/worker/worker.py:451-463)."""
        return self.scheduler.abort(request_id)

    def has_unfinished(self) -> bool:
        return (self.scheduler.has_work() or self._inflight is not None
                or self._reported < len(self.scheduler.finished))

    # -- one step ---------------------------------------------------------
    # Steps are pipelined one deep, as in the reference's worker (mstar/worker/worker.py:
    # 2118-2211, 1328-1550: step N+1 is built and submitted while step N runs, and a stop
    # takes effect one step late, worker.py:1612-1629).  A call plans and launches step N+1
    # first and reads step N's tokens back afterwards: the tokens that step N sampled are
    # fed to step N+1 on the device (the embedding takes them from the sampler's output),
    # the scheduler counts them as places whose values arrive later.  So the GPU works on
    # step N+1 while the host reads, finishes requests, and plans; a request that turns out
    # to have stopped at step N has one token computed in vain, a request that reaches
    # max_output_tokens is foreseen and left out.

    def _launch(self, plan, prev) -> tuple:
        """Run the plan's forward pass and sampling; tokens stay on the device."""
        source = {}
        if prev is not None:
            source = {rid: j for j, rid in enumerate(prev[1])}
        entries, pending = [], {}
        for i, e in enumerate(plan.entries):
            tokens = e.tokens
            if tokens[-1] is None:              # sampled by the step in flight
                if len(tokens) != 1 or e.request.request_id not in source:
                    raise RuntimeError("a token is missing that no step in flight will bring")
                pending[i] = source[e.request.request_id]
                tokens = [0]
            entries.append(StepEntry(e.request.request_id, tokens,
                                     (len(tokens) - 1,) if e.samples else ()))
        logits = self.stepper.step(entries, pending, prev[2] if pending else None)
        sampling = [e.request.request_id for e in plan.entries if e.samples]
        if not sampling:
            return None
        tokens = self.sampler.sample(sampling, logits)
        # their copy to the host is queued now, before the next step is: reading it later
        # waits for this step only
        turn = self._turn = (self._turn + 1) % len(self._host_tokens)
        if self._host_tokens[turn].numel() < len(sampling) + 1:
            self._host_tokens[turn] = torch.empty(len(sampling) + 1, dtype=torch.int32,
                                                  pin_memory=True)
        host = self._host_tokens[turn][:len(sampling) + 1]
        # on a stream of its own, so that the next step's input copy and kernels do not
        # queue behind it (``tokens`` stays referenced until it has arrived)
        sampled = torch.cuda.Event()
        sampled.record()
        with torch.cuda.stream(self._copy_stream):
            self._copy_stream.wait_event(sampled)
            host[:-1].copy_(tokens, non_blocking=True)
            # with the tokens comes the word that kernels set when a bounded wait ran out
            host[-1:].copy_(self._error_word, non_blocking=True)
            arrived = torch.cuda.Event()
            arrived.record()
        return plan, sampling, tokens, host, arrived

    def _finished_and_complete(self) -> list:
        """Requests that have finished and whose last tokens have arrived, each once."""
        out = []
        done = self.scheduler.finished
        while self._reported < len(done):
            r = done[self._reported]
            if r.output and r.output[-1] is None:
                break                            # its last token is still in flight
            out.append(r)
            self._reported += 1
        return out

    def step(self) -> list:
        """Plan and launch one batch, then read the tokens of the batch before; returns the
        requests that finished."""
        t0 = time.perf_counter()
        prev = self._inflight
        self._inflight = None
        plan = self.scheduler.schedule()
        self.stats.preemptions += len(plan.preempted)
        for r in plan.admitted:
            self.sampler.add_request(r.request_id, r.params, r.slot, generated=r.output)
        if plan.entries:
            launched = self._launch(plan, prev)
            self.scheduler.advance(plan)
            self.stats.steps += 1
            self.stats.prompt_tokens += sum(len(e.tokens) for e in plan.entries if not (
                e.samples and len(e.tokens) == 1))
            if prev is not None:
                self.pipelined_steps += 1
            self._inflight = launched           # None if the step samples nothing
        elif (prev is None and not plan.preempted and not plan.finished
              and self.scheduler.has_work()):
            raise RuntimeError("the scheduler can make no progress: no request fits the cache")
        if prev is not None:
            old_plan, old_sampling, _, host, arrived = prev
            arrived.synchronize()
            values = host.tolist()
            if values[-1]:
                # a kernel returned with partial output: these tokens are not to be trusted
                self._error_word.zero_()
                ops.raise_on_wait_code(values[-1])
            sampled = dict(zip(old_sampling, values[:-1]))
            self.scheduler.resolve(old_plan, sampled)
            self.stats.generated_tokens += len(sampled)
        if self.log_stats:
            self.stats.step_seconds.append(time.perf_counter() - t0)
        return self._finished_and_complete()

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
