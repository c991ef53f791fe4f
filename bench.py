#!/usr/bin/env python3
"""Headline benchmark: decode tokens/s of the Orpheus-3B-sized Llama decoder (random
weights, bfloat16) at batch 8 with 2,048-token cached prompts and pages of 16 tokens, on
one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--rounds R] [--page-size P]
                    [--impl ours|reference] [--workloads all|none|mixed64|long8]

One JSON line on stdout.  ``value``: decoded tokens per second of the engine's step
function plus greedy sampling, timed on the device with CUDA events: W warm-up steps, then
R rounds of exactly K steps each; ``ms_per_step`` is the median round, the fastest and
slowest are beside it.  ``e2e``: the same through the Python entry point (``LLM.step``),
host token ids in and out.  ``prefill``: one 2,048-token prompt in one step.
``roofline``: bytes a decode step has to read (every weight once, and the cache of the
live requests) over its time, against the measured copy bandwidth.  ``points``: decode at
batch 1 and 64, batch 8 with pages of 64 tokens, and two serving workloads through the
entry point at other sizes of the architecture (64 mixed requests at the Llama 3.2 1B
sizes, 8 long prompts in portions at the Llama 3.1 8B sizes), each as generated tokens per
second and median time to the first token.  A step is one decode step; every step reads
all weights (6.6 GB), far more than the 126 MB L2, so no L2 flush is needed.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

# Layer sizes of the benchmark model: Orpheus 3B / Llama 3.2 3B
# (mstar/model/orpheus/config.py:4-23).
ORPHEUS_3B = dict(
    architectures=["LlamaForCausalLM"], num_hidden_layers=28, hidden_size=3072,
    num_attention_heads=24, num_key_value_heads=8, head_dim=128, intermediate_size=8192,
    vocab_size=156940, tie_word_embeddings=True, rope_theta=500000.0,
    rope_scaling={"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0,
                  "high_freq_factor": 4.0, "original_max_position_embeddings": 8192},
    rms_norm_eps=1e-5, max_position_embeddings=131072, hidden_act="silu",
    torch_dtype="bfloat16",
)
# Further sizes of the same architecture (--sizes): Llama 3.2 1B and Llama 3.1 8B.
LLAMA_1B = dict(ORPHEUS_3B, num_hidden_layers=16, hidden_size=2048, num_attention_heads=32,
                head_dim=64, vocab_size=128256)
LLAMA_8B = dict(ORPHEUS_3B, num_hidden_layers=32, hidden_size=4096, num_attention_heads=32,
                intermediate_size=14336, vocab_size=128256, tie_word_embeddings=False,
                rope_scaling=dict(ORPHEUS_3B["rope_scaling"], factor=8.0))
SIZES = {"orpheus-3b": ("Orpheus 3B / Llama 3.2 3B", ORPHEUS_3B),
         "llama-1b": ("Llama 3.2 1B", LLAMA_1B), "llama-8b": ("Llama 3.1 8B", LLAMA_8B)}
PROMPT_LEN = 2048
CONTEXT = 4096
PAGE_SIZE = 16          # the default of --page-size; kernel_bench reads the global
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


def peaks() -> dict:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.is_file():
        try:
            raw = json.loads(path.read_text())
            return {"hbm_gbs": float(raw["hbm_gbs"]), "bf16_tflops": float(raw["bf16_tflops"]),
                    "source": "measured"}
        except (KeyError, ValueError, TypeError):
            pass
    return dict(FALLBACK_PEAKS)


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region is timed."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")
    NAMES = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")

    def __init__(self):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None

    def _run(self):
        while not self._stop.is_set():
            try:
                out = subprocess.run(
                    ["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}",
                     "--format=csv,noheader,nounits"], capture_output=True, text=True,
                    timeout=5).stdout.strip().splitlines()[0]
                parts = [p.strip() for p in out.split(",")]
                self.samples.append(float(parts[0]))
                self.max_mhz = float(parts[1])
                for name, val in zip(self.NAMES, parts[2:]):
                    if val.lower().startswith("active"):
                        self.reasons.add(name)
            except Exception:
                pass
            self._stop.wait(0.05)

    def __enter__(self):
        self._thread = threading.Thread(target=self._run, daemon=True)
        self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        self._thread.join(timeout=6)

    def summary(self) -> dict:
        return {"sm_mhz": statistics.median(self.samples) if self.samples else None,
                "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(self.samples)}


def flops_of_step(cfg: dict, q_lens, kv_lens, rows: int) -> float:
    """Matrix and attention FLOPs of one step (2 per multiply-add)."""
    L, H, I, V = (cfg["num_hidden_layers"], cfg["hidden_size"], cfg["intermediate_size"],
                  cfg["vocab_size"])
    nq, nkv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    T = sum(q_lens)
    per_token = (H * (nq + 2 * nkv) * hd) + (nq * hd * H) + 3 * H * I
    linear = 2.0 * T * L * per_token + 2.0 * rows * H * V
    attn = 0.0
    for q, kv in zip(q_lens, kv_lens):
        keys = sum(kv - q + i + 1 for i in range(q))     # causal: token i sees kv-q+i+1 keys
        attn += 4.0 * nq * hd * keys
    return linear + L * attn


def bytes_of_decode_step(cfg: dict, model, kv_lens) -> float:
    """Every weight used once (tied head counted once) plus keys and values read."""
    nkv, hd, L = cfg["num_key_value_heads"], cfg["head_dim"], cfg["num_hidden_layers"]
    kv = sum(kv_lens) * 2 * nkv * hd * 2 * L
    return float(model.parameter_bytes() + kv)


def build_model(cfg_raw: dict, seed: int = 0):
    from mstar_b200.config.registry import config_from_dict
    from mstar_b200.engine.model import load_model
    from mstar_b200.weights.random_init import random_checkpoint

    cfg = config_from_dict(cfg_raw)
    tensors = random_checkpoint(cfg, seed, std=0.02, device="cuda:0")
    model = load_model(None, dtype="bfloat16", device="cuda:0", config=cfg, tensors=tensors)
    del tensors
    return model


def prompts(batch: int, vocab: int, length: int, seed: int = 1) -> list:
    import torch

    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (batch, length), generator=g).tolist()


def time_decode(stepper, batch: int, cfg: dict, steps: int, warmup: int, rounds: int = 1) -> dict:
    """B requests with PROMPT_LEN cached tokens each; W warm-up decode steps of the step
    function plus greedy sampling, then ``rounds`` rounds of exactly K steps, each round timed
    with CUDA events.  The median round is the result; fastest and slowest are reported."""
    import torch

    from mstar_b200 import ops
    from mstar_b200.engine.step import StepEntry
    from mstar_b200.ops import lib

    ids = [f"d{batch}-{i}" for i in range(batch)]
    total = warmup + rounds * steps
    toks = prompts(batch, cfg["vocab_size"], PROMPT_LEN + total + 1, seed=batch)
    for rid, t in zip(ids, toks):
        stepper.add_request(rid)
        stepper.step([StepEntry(rid, t[:PROMPT_LEN], ())])
    torch.cuda.synchronize()

    def one(k: int):
        logits = stepper.step([StepEntry(rid, [t[PROMPT_LEN + k]], (0,))
                               for rid, t in zip(ids, toks)])
        return ops.argmax(logits)

    for k in range(warmup):
        one(k)
    torch.cuda.synchronize()
    times, launches = [], 0
    for r in range(rounds):
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        launches0 = lib.launch_count()
        start.record()
        for k in range(warmup + r * steps, warmup + (r + 1) * steps):
            one(k)
        end.record()
        torch.cuda.synchronize()
        times.append(start.elapsed_time(end) / steps)
        launches = lib.launch_count() - launches0
    ops.check_error_word(stepper.device)
    ms = statistics.median(times)
    kv_lens = [PROMPT_LEN + warmup + (rounds * steps) // 2] * batch
    for rid in ids:
        stepper.free_request(rid)
    return {"ms_per_step": ms, "ms_min": min(times), "ms_max": max(times),
            "tokens_per_s": batch / (ms / 1e3), "launches": launches, "kv_lens": kv_lens}


def time_prefill(stepper, cfg: dict, reps: int = 5) -> dict:
    import torch

    from mstar_b200.engine.step import StepEntry

    toks = prompts(reps + 2, cfg["vocab_size"], PROMPT_LEN, seed=99)
    times = []
    for i, t in enumerate(toks):
        rid = f"p{i}"
        stepper.add_request(rid)
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        stepper.step([StepEntry(rid, t, (PROMPT_LEN - 1,))])
        end.record()
        torch.cuda.synchronize()
        stepper.free_request(rid)
        if i >= 2:                                   # two warm-up prompts
            times.append(start.elapsed_time(end))
    ms = statistics.median(times)
    return {"ms": ms, "tokens_per_s": PROMPT_LEN / (ms / 1e3),
            "flops": flops_of_step(cfg, [PROMPT_LEN], [PROMPT_LEN], 1)}


def time_e2e(model, batch: int, cfg: dict, steps: int, warmup: int, num_pages: int,
             page_size: int, rounds: int = 1) -> dict:
    """The same decode steps through the public entry point: host token ids in (pinned
    index buffer copied to the device every step) and sampled token ids read back; wall
    clock around ``rounds`` rounds of K steps, the median round reported."""
    import torch

    from mstar_b200 import LLM, SamplingParams

    llm = LLM(model, page_size=page_size, max_num_pages=num_pages,
              max_num_batched_tokens=PROMPT_LEN, max_concurrent_requests=max(batch, 1),
              max_batch_size=max(batch, 1))
    params = SamplingParams(temperature=0.0, ignore_eos=True,
                            max_output_tokens=warmup + rounds * steps + batch + 8)
    for i, t in enumerate(prompts(batch, cfg["vocab_size"], PROMPT_LEN, seed=7 + batch)):
        llm.add_request(t, params, request_id=f"e{i}")
    while any(r.num_pending() > 1 for r in llm.scheduler.running) or llm.scheduler.waiting:
        llm.step()                                   # prompts, one per step
    for _ in range(warmup):
        llm.step()
    times = []
    for _ in range(rounds):
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(steps):
            llm.step()
        torch.cuda.synchronize()
        times.append((time.perf_counter() - t0) / steps * 1e3)
    ms = statistics.median(times)
    h2d = llm.stepper.last_h2d_bytes
    for r in list(llm.scheduler.running):
        llm.scheduler.abort(r.request_id)
    # tokens out: 4 bytes a request, and the 4-byte word kernels report a given-up wait in
    return {"tokens_per_s": batch / (ms / 1e3), "ms_per_step": ms, "ms_min": min(times),
            "ms_max": max(times), "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4 * batch + 4}


# ------------------------------------------------------------------ serving workloads
WORKLOADS = {
    # 64 requests at once, prompts of 16 to 2,048 tokens, 256 new tokens each
    "mixed64": dict(sizes="llama-1b", requests=64, prompt=(16, 2048), new_tokens=256,
                    budget=2048),
    # 8 prompts of 8,192 tokens, computed in portions of 2,048, 128 new tokens each
    "long8": dict(sizes="llama-8b", requests=8, prompt=(8192, 8192), new_tokens=128,
                  budget=2048),
}


def run_workload(name: str, page_size: int) -> dict:
    """A whole serving run through the entry point: all requests are handed over at time
    zero, the scheduler admits, cuts prompts into portions under its token budget, decodes
    and frees.  Run twice (the first run captures the decode graphs and compiles nothing
    else); the second is timed by the wall clock.  Greedy sampling, no stop token."""
    import numpy as np
    import torch

    from mstar_b200 import LLM, SamplingParams

    w = WORKLOADS[name]
    model_name, cfg = SIZES[w["sizes"]]
    print(f"[bench] workload {name}: {w['requests']} requests at the {model_name} sizes ...",
          file=sys.stderr, flush=True)
    model = build_model(dict(cfg), seed=2)
    rng = np.random.default_rng(5)
    lens = rng.integers(w["prompt"][0], w["prompt"][1] + 1, size=w["requests"]).tolist()
    g = torch.Generator().manual_seed(11)
    prompt_ids = [torch.randint(0, cfg["vocab_size"], (n,), generator=g).tolist() for n in lens]
    pages = sum(-(-(n + w["new_tokens"]) // page_size) for n in lens) + 64
    llm = LLM(model, page_size=page_size, max_num_pages=pages,
              max_num_batched_tokens=w["budget"], max_concurrent_requests=w["requests"],
              max_batch_size=w["requests"])
    params = SamplingParams(temperature=0.0, ignore_eos=True, max_output_tokens=w["new_tokens"])
    result, before = {}, None
    for run in ("warm-up", "timed"):
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        ids = [llm.add_request(p, params, request_id=f"{name}-{run}-{i}")
               for i, p in enumerate(prompt_ids)]
        waiting = {r.request_id: r for r in llm.scheduler.waiting}
        first: dict = {}
        done = 0
        while llm.has_unfinished():
            done += len(llm.step())
            if len(first) < len(ids):
                now = time.perf_counter() - t0
                for rid, r in waiting.items():
                    if rid not in first and r.output and r.output[0] is not None:
                        first[rid] = now
        torch.cuda.synchronize()
        seconds = time.perf_counter() - t0
        assert done == len(ids) and len(first) == len(ids)
        generated = w["requests"] * w["new_tokens"]
        # the two runs decode the same prompts greedily: the same tokens, whatever the
        # batches were that the scheduler formed
        tokens = [list(waiting[rid].output) for rid in ids]
        agree = None if run == "warm-up" else tokens == before
        before = tokens
        result = {"tokens_per_s": generated / seconds, "seconds": seconds, "runs_agree": agree,
                  "ttft_ms_median": statistics.median(first.values()) * 1e3,
                  "ttft_ms_max": max(first.values()) * 1e3,
                  "prompt_tokens": sum(lens), "generated_tokens": generated,
                  "steps": llm.stats.steps, "preemptions": llm.stats.preemptions}
        llm.stats.steps = 0
    del llm, model
    torch.cuda.empty_cache()
    return result


# --------------------------------------------------------------- single kernels
def _time_graph(fn, reps: int = 20, rounds: int = 5) -> float:
    """Median milliseconds of one call of ``fn`` when ``reps`` calls are replayed as one
    CUDA graph (so that launch gaps are what they are inside a captured step)."""
    import torch

    fn()
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        fn()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for _ in range(reps):
            fn()
    # MSTAR_BENCH_WARM_MS=N replays for N ms first: short kernels then see the clocks of a busy
    # GPU (a little faster), long ones its power cap (8,192-token attention 0.41 instead of
    # 0.37 ms); the figures in profiles/ are taken without, like the burst peak they are
    # compared with
    warm = float(os.environ.get("MSTAR_BENCH_WARM_MS", "0"))
    t0 = time.perf_counter()
    while (time.perf_counter() - t0) * 1e3 < warm:
        for _ in range(10):
            graph.replay()
        torch.cuda.synchronize()
    times = []
    for _ in range(rounds):
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        graph.replay()
        end.record()
        torch.cuda.synchronize()
        times.append(start.elapsed_time(end) / reps)
    return statistics.median(times)


def kernel_bench(name: str, batch: int, ctx: int, small: bool, cfg: dict) -> int:
    """Time one kernel alone at the benchmark model's shapes: ``--kernel NAME``.  Inputs
    rotate over copies larger than L2 where the kernel is memory-bound.  ``--small``
    shrinks the case for profiler captures (still larger than L2 where it matters)."""
    import torch

    from mstar_b200 import ops

    nq, nkv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    H, I, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    dev = "cuda:0"
    pk = peaks()
    g = torch.Generator(device=dev).manual_seed(0)

    def rnd(*shape, scale=1.0):
        return (scale * torch.randn(*shape, generator=g, device=dev)).to(torch.bfloat16)

    out = {"kernel": name, "batch": batch, "ctx": ctx}
    if name in ("decode_attention", "prefill_attention"):
        page = PAGE_SIZE
        reqs = batch
        pages_per = -(-ctx // page)
        kv = rnd(reqs * pages_per + 1, 2, nkv, page, hd)
        table = torch.randperm(reqs * pages_per, device=dev).to(torch.int32).view(reqs, pages_per)
        if name == "decode_attention":
            q = rnd(reqs, (nq + 2 * nkv) * hd)
            o = torch.empty(reqs, nq * hd, dtype=torch.bfloat16, device=dev)
            token_req = torch.arange(reqs, dtype=torch.int32, device=dev)
            cache_pos = torch.full((reqs,), ctx - 1, dtype=torch.int32, device=dev)
            fn = lambda: ops.paged_decode_attention(q, q.stride(0), o, kv, table, token_req,
                                                    cache_pos, reqs, nq, nkv, hd, page, 0,
                                                    hd ** -0.5, ctx)
            ms = _time_graph(fn)
            nbytes = reqs * ctx * 2 * nkv * hd * 2
            out.update(ms=ms, gbs=nbytes / ms / 1e6, frac_hbm=nbytes / ms / 1e6 / pk["hbm_gbs"],
                       split=ops.decode_split(reqs, nkv, ctx, ring=os.environ.get("MSTAR_DECODE_ATTENTION") != "per_item"))
        else:
            q = rnd(reqs * ctx, (nq + 2 * nkv) * hd)
            o = torch.empty(reqs * ctx, nq * hd, dtype=torch.bfloat16, device=dev)
            indptr = torch.arange(0, (reqs + 1) * ctx, ctx, dtype=torch.int32, device=dev)
            kvl = torch.full((reqs,), ctx, dtype=torch.int32, device=dev)
            fn = lambda: ops.paged_prefill_attention(q, q.stride(0), o, kv, table, indptr, kvl, 0,
                                                     reqs, ctx, nq, nkv, hd, page, 0, hd ** -0.5)
            ms = _time_graph(fn, reps=5)
            flops = reqs * 4.0 * nq * hd * ctx * (ctx + 1) / 2
            out.update(ms=ms, tflops=flops / ms / 1e9,
                       frac_bf16=flops / ms / 1e9 / pk["bf16_tflops"])
    elif name in ("gemm_qkv", "gemm_o", "gemm_gate_up", "gemm_down", "gemm_lm_head"):
        n, k = {"gemm_qkv": ((nq + 2 * nkv) * hd, H), "gemm_o": (H, nq * hd),
                "gemm_gate_up": (2 * I, H), "gemm_down": (H, I), "gemm_lm_head": (V, H)}[name]
        if small and name == "gemm_lm_head":
            n = 65536
        copies = max(1, -(-(160 << 20) // (n * k * 2)))          # rotate over > L2 bytes
        ws = [rnd(n, k, scale=0.02) for _ in range(copies)]
        x = rnd(batch, k)
        state = {"i": 0}

        def fn():
            w = ws[state["i"] % copies]
            state["i"] += 1
            if name == "gemm_gate_up":
                return ops.gated_up(x, w)
            return ops.linear(x, w, out_dtype=torch.float32 if name == "gemm_lm_head" else None)

        ms = _time_graph(fn, reps=max(copies * 2, 8))
        nbytes = n * k * 2
        flops = 2.0 * batch * n * k
        out.update(ms=ms, n=n, k=k, gbs=nbytes / ms / 1e6,
                   frac_hbm=nbytes / ms / 1e6 / pk["hbm_gbs"], tflops=flops / ms / 1e9)
    elif name == "qkv_rope":
        # the decode form of the mixer's first product: product, rotation and cache write
        n, k = (nq + 2 * nkv) * hd, H
        copies = max(1, -(-(160 << 20) // (n * k * 2)))
        ws = [rnd(n, k, scale=0.02) for _ in range(copies)]
        x = rnd(batch, k)
        pages_per = -(-ctx // PAGE_SIZE)
        kv = rnd(batch * pages_per + 1, 2, nkv, PAGE_SIZE, hd)
        table = torch.arange(batch * pages_per, dtype=torch.int32, device=dev).view(batch, -1)
        pos = torch.full((batch,), ctx - 1, dtype=torch.int32, device=dev)
        req = torch.arange(batch, dtype=torch.int32, device=dev)
        inv = torch.rand(hd // 2, device=dev)
        state = {"i": 0}

        def fn():
            w = ws[state["i"] % copies]
            state["i"] += 1
            return ops.qkv_rope_write(x, w, pos, pos, req, table, inv, kv, nq, nkv, hd, PAGE_SIZE,
                                      static_weights=True)

        ms = _time_graph(fn, reps=max(copies * 2, 8))
        out.update(ms=ms, n=n, k=k, gbs=n * k * 2 / ms / 1e6,
                   frac_hbm=n * k * 2 / ms / 1e6 / pk["hbm_gbs"])
    elif name in ("add_rmsnorm", "rope_kv_write"):
        rows = batch
        if name == "add_rmsnorm":
            resid = torch.randn(rows, H, device=dev)
            delta = rnd(rows, H)
            w = rnd(H)
            fn = lambda: ops.add_rmsnorm(resid, delta, w, 1e-5, torch.bfloat16)
        else:
            qkv = rnd(rows, (nq + 2 * nkv) * hd)
            pos = torch.full((rows,), ctx - 1, dtype=torch.int32, device=dev)
            req = torch.arange(rows, dtype=torch.int32, device=dev)
            kv = rnd(rows * (-(-ctx // PAGE_SIZE)) + 1, 2, nkv, PAGE_SIZE, hd)
            table = torch.arange(rows * (-(-ctx // PAGE_SIZE)), dtype=torch.int32,
                                 device=dev).view(rows, -1)
            inv = torch.rand(hd // 2, device=dev)
            fn = lambda: ops.rope_kv_write(qkv, pos, pos, req, table, inv, kv, nq, nkv, hd, hd,
                                           False, PAGE_SIZE)
        out.update(ms=_time_graph(fn, reps=50))
    else:
        print(f"unknown kernel {name!r}")
        return 2
    out["peaks"] = pk["source"]
    print(json.dumps(out))
    return 0


def reference_arm(args) -> int:
    """The reference's own engine on the same workload, in a process of its own that
    imports nothing of this package (baseline/run_reference.py); its JSON line is passed
    on.  If that process dies without a line, the reason is printed as ``unavailable``."""
    cmd = [sys.executable, str(ROOT / "baseline" / "run_reference.py"), "--steps", str(args.steps),
           "--warmup", str(args.warmup), "--rounds", str(args.rounds), "--batch", str(args.batch),
           "--page-size", str(args.page_size)]
    if args.layers:
        cmd += ["--layers", str(args.layers)]
    try:
        proc = subprocess.run(cmd, stdout=subprocess.PIPE, text=True, timeout=3000)
        lines = [ln for ln in proc.stdout.splitlines() if ln.startswith("{")]
        if lines:
            print(lines[-1])
            return 0
        why = f"baseline/run_reference.py exited with {proc.returncode} and printed no record"
    except subprocess.TimeoutExpired:
        why = "baseline/run_reference.py did not finish within 3000 s"
    print(json.dumps({"impl": "reference", "unavailable": why}))
    return 0


def main() -> int:
    global PAGE_SIZE
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--rounds", type=int, default=5,
                    help="rounds of --steps timed steps; the median round is reported")
    ap.add_argument("--page-size", type=int, default=PAGE_SIZE, help="tokens per cache page")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=None,
                    help="fewer layers than the model has (named in the record)")
    ap.add_argument("--workloads", default="all", choices=["all", "none", *sorted(WORKLOADS)],
                    help="serving workloads through the entry point, reported under points")
    ap.add_argument("--kernel", default=None,
                    help="time one kernel alone (decode_attention, prefill_attention, gemm_qkv, "
                         "gemm_o, gemm_gate_up, gemm_down, gemm_lm_head, qkv_rope, add_rmsnorm, "
                         "rope_kv_write) at --batch rows / requests and --ctx keys")
    ap.add_argument("--ctx", type=int, default=PROMPT_LEN)
    ap.add_argument("--small", action="store_true", help="a smaller case, for profiler captures")
    ap.add_argument("--sizes", default="orpheus-3b", choices=sorted(SIZES),
                    help="layer sizes; the default is the benchmark model")
    args = ap.parse_args()
    model_name, sizes = SIZES[args.sizes]
    PAGE_SIZE = page = args.page_size
    if args.gpus != 1:
        print(f"bench.py measures a single-GPU engine: --gpus {args.gpus} is not supported")
        return 2
    if args.kernel:
        return kernel_bench(args.kernel, args.batch, args.ctx, args.small, sizes)
    if args.impl == "reference":
        return reference_arm(args)
    warmup = max(args.warmup, 3)
    rounds = max(args.rounds, 1)

    import torch

    from mstar_b200.engine.step import make_stepper
    from mstar_b200.ops import lib

    cfg = dict(sizes)
    full_layers = cfg["num_hidden_layers"]
    if args.layers:
        cfg["num_hidden_layers"] = args.layers
    pk = peaks()
    print("[bench] building the random-weight model ...", file=sys.stderr, flush=True)
    model = build_model(cfg)
    max_batch = max(64, args.batch)
    pages = max_batch * (CONTEXT // page) + 64
    stepper = make_stepper(model, page_size=page, num_pages=pages, num_slots=max_batch + 4)

    print("[bench] prefill ...", file=sys.stderr, flush=True)
    pre = time_prefill(stepper, cfg)
    print("[bench] decode ...", file=sys.stderr, flush=True)
    with ClockSampler() as clocks:
        head = time_decode(stepper, args.batch, cfg, args.steps, warmup, rounds)
    # the same steps through the entry point, directly after the device-timed ones (the
    # long batch-64 run below leaves the GPU under its power cap)
    print("[bench] end to end ...", file=sys.stderr, flush=True)
    e2e = time_e2e(model, args.batch, cfg, args.steps, warmup,
                   args.batch * (CONTEXT // page) + 64, page, rounds)
    print("[bench] decode at batch 1 and 64 ...", file=sys.stderr, flush=True)
    points = {}
    for b in (1, 64):
        r = time_decode(stepper, b, cfg, max(args.steps // 2, 8), warmup, min(rounds, 3))
        points[f"decode_b{b}"] = round(r["tokens_per_s"], 1)
    del stepper
    torch.cuda.empty_cache()
    other = 64 if page != 64 else 16
    print(f"[bench] decode with pages of {other} ...", file=sys.stderr, flush=True)
    stepper = make_stepper(model, page_size=other,
                           num_pages=args.batch * (CONTEXT // other) + 64,
                           num_slots=args.batch + 4)
    r = time_decode(stepper, args.batch, cfg, args.steps, warmup, min(rounds, 3))
    points[f"decode_b{args.batch}_page{other}"] = round(r["tokens_per_s"], 1)
    del stepper
    torch.cuda.empty_cache()

    step_bytes = bytes_of_decode_step(cfg, model, head["kv_lens"])
    achieved = step_bytes / (head["ms_per_step"] / 1e3) / 1e9
    parameter_gb = model.parameter_bytes() / 1e9
    del model
    torch.cuda.empty_cache()
    chosen = sorted(WORKLOADS) if args.workloads == "all" else (
        [] if args.workloads == "none" else [args.workloads])
    for name in chosen:
        w = run_workload(name, page)
        tag = f"{name}_{WORKLOADS[name]['sizes'].replace('-', '')}"
        points[f"{tag}_tok_s"] = round(w["tokens_per_s"], 1)
        points[f"{tag}_ttft_ms"] = round(w["ttft_ms_median"], 1)
        points[f"{tag}_seconds"] = round(w["seconds"], 3)
        points[f"{tag}_runs_agree"] = 1.0 if w["runs_agree"] else 0.0
        print(f"[bench] {name}: {json.dumps(w)}", file=sys.stderr, flush=True)

    record = {
        "metric": f"decode tok/s at batch {args.batch} ({model_name.split(' / ')[0]} bf16, "
                  "2,048-token cached prompts)",
        "value": round(head["tokens_per_s"], 1), "unit": "tokens/s", "n_gpus": 1,
        "steps": args.steps, "warmup": warmup, "ms_per_step": round(head["ms_per_step"], 4),
        "rounds": rounds, "ms_per_step_min": round(head["ms_min"], 4),
        "ms_per_step_max": round(head["ms_max"], 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic token ids, random-init weights N(0, 0.02)",
        "config": {
            "model": model_name, "global_batch": args.batch,
            "seq_len": CONTEXT, "prompt_len": PROMPT_LEN, "parallelism": "single GPU",
            "layers": cfg["num_hidden_layers"], "layers_of_model": full_layers,
            "hidden": cfg["hidden_size"], "heads": cfg["num_attention_heads"],
            "kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"],
            "intermediate": cfg["intermediate_size"], "vocab": cfg["vocab_size"],
            "tied_embeddings": cfg["tie_word_embeddings"],
            "rope": f"theta 5e5, llama3 x{cfg['rope_scaling']['factor']:g} (1, 4, 8192)",
            "rms_eps": cfg["rms_norm_eps"], "page_size": page,
            "l2": f"inputs larger than L2 (weights {parameter_gb:.1f} GB per step)",
            "peaks": pk["source"]},
        "e2e": {"value": round(e2e["tokens_per_s"], 1), "unit": "tokens/s",
                "h2d_bytes_per_step": e2e["h2d_bytes_per_step"],
                "d2h_bytes_per_step": e2e["d2h_bytes_per_step"],
                "ms_per_step": round(e2e["ms_per_step"], 4),
                "ms_per_step_min": round(e2e["ms_min"], 4),
                "ms_per_step_max": round(e2e["ms_max"], 4)},
        "gpu_launches": head["launches"],
        "clocks": clocks.summary(),
        "prefill": {"value": round(pre["tokens_per_s"], 1), "tokens": PROMPT_LEN,
                    "ms": round(pre["ms"], 3),
                    "frac": round(pre["flops"] / (pre["ms"] / 1e3) / (pk["bf16_tflops"] * 1e12), 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"],
                     "unit": "GB/s", "frac": round(achieved / pk["hbm_gbs"], 4)},
        "points": points,
        "libraries": sorted(lib.loaded_libraries()),
    }
    print(json.dumps(record))
    return 0


if __name__ == "__main__":
    sys.exit(main())
