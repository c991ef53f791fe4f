#!/usr/bin/env python3
"""The reference arm of bench.py: t-avil/mstar's own engine on the benchmark's workload.

Runs the unmodified reference, installed under ``baseline/_ref`` (see the repository's
design notes for the pip command), through the code its server runs for the Orpheus
language model, and nothing of mstar_b200:

* ``OrpheusForCausalLM`` built as ``OrpheusModel._create_llm_submodule`` builds it
  (mstar/model/orpheus/orpheus_model.py:440-466: on the meta device, cast to bfloat16,
  ``to_empty`` on the GPU), random weights under the checkpoint's tensor names loaded
  through its own ``load_weights`` (mstar/model/orpheus/components/language_model.py:110-115),
  wrapped in its ``OrpheusLLMSubmodule``;
* its ``KVCacheEngine`` (mstar/engine/kv_cache_engine.py): ``load_model`` makes the paged
  cache, the allocation manager and the sampler, ``warmup`` captures its CUDA graphs,
  ``execute_batch`` runs prefill and decode batches through its dispatch (captured graph,
  else batched eager) with its FlashInfer wrappers and its sampler.

What stands in for the rest of the server (HTTP front end, conductor, worker processes,
tokenizer, SNAC codec, checkpoint download: they need the network and packages that are not
installed) is this loop: it admits B requests, prefills their 2,048-token prompts, and
feeds every sampled token back as the next input, as the reference's worker does
(mstar/worker/worker.py:1552-1595).

Prints one JSON line: the bench contract's keys with ``"impl": "reference"``, or
``{"impl": "reference", "unavailable": "<the exception>"}``.
"""
from __future__ import annotations

import argparse
import json
import statistics
import sys
import time
import traceback
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
REF = ROOT / "baseline" / "_ref"
PROMPT_LEN = 2048
CONTEXT = 4096


def log(msg: str) -> None:
    print(f"[reference] {msg}", file=sys.stderr, flush=True)


def random_weights(cfg, torch, device):
    """(name, tensor) pairs under the checkpoint's names, N(0, 0.02) in bfloat16, norm weights
    one; the head gets the embedding's values (the checkpoint ties them; the reference has a
    parameter of its own for it)."""
    g = torch.Generator(device=device).manual_seed(0)
    H, I, V = cfg.hidden_size, cfg.intermediate_size, cfg.vocab_size
    q, kv = cfg.num_attention_heads * cfg.head_dim, cfg.num_key_value_heads * cfg.head_dim

    def mat(rows, cols):
        return (0.02 * torch.randn(rows, cols, generator=g, device=device)).to(torch.bfloat16)

    embed = mat(V, H)
    yield "model.embed_tokens.weight", embed
    yield "lm_head.weight", embed
    yield "model.norm.weight", torch.ones(H, dtype=torch.bfloat16, device=device)
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}"
        yield f"{p}.self_attn.q_proj.weight", mat(q, H)
        yield f"{p}.self_attn.k_proj.weight", mat(kv, H)
        yield f"{p}.self_attn.v_proj.weight", mat(kv, H)
        yield f"{p}.self_attn.o_proj.weight", mat(H, q)
        yield f"{p}.mlp.gate_proj.weight", mat(I, H)
        yield f"{p}.mlp.up_proj.weight", mat(I, H)
        yield f"{p}.mlp.down_proj.weight", mat(H, I)
        yield f"{p}.input_layernorm.weight", torch.ones(H, dtype=torch.bfloat16, device=device)
        yield f"{p}.post_attention_layernorm.weight", torch.ones(H, dtype=torch.bfloat16,
                                                                 device=device)


def run(args) -> dict:
    sys.path.insert(0, str(REF))
    import torch

    from mstar.communication.tensors import LocalTransferEngine
    from mstar.conductor.request_info import CurrentForwardPassInfo
    from mstar.distributed.communication import TPCommGroup, WorkerTPGroups
    from mstar.engine.base import NodeBatch
    from mstar.engine.kv_cache_engine import KVCacheEngine
    from mstar.engine.kv_store import KVCacheConfig, TransferEngineInfo
    from mstar.model.orpheus.components.language_model import OrpheusForCausalLM
    from mstar.model.orpheus.config import OrpheusModelConfig
    from mstar.model.orpheus.submodules import OrpheusLLMSubmodule
    from mstar.utils.sampling import SamplingConfig

    device = torch.device("cuda:0")
    torch.cuda.set_device(0)
    cfg = OrpheusModelConfig()
    full_layers = cfg.num_hidden_layers
    if args.layers:
        cfg.num_hidden_layers = args.layers
    batch, steps, warmup = args.batch, args.steps, max(args.warmup, 3)

    log("building OrpheusForCausalLM (bfloat16, random weights) ...")
    tp = TPCommGroup.trivial()
    with torch.device("meta"):
        lm = OrpheusForCausalLM(cfg, comm_group=tp)
    lm = lm.to(torch.bfloat16)
    lm.to_empty(device=device)
    loaded = lm.load_weights(random_weights(cfg, torch, device))
    missing = {n for n, _ in lm.named_parameters()} - set(loaded)
    if missing:
        raise RuntimeError(f"the reference's loader left parameters unset: {sorted(missing)[:4]}")
    lm.eval()
    submodule = OrpheusLLMSubmodule(language_model=lm, config=cfg)

    pages_per_request = -(-CONTEXT // args.page_size)
    kv_cfg = KVCacheConfig(
        num_layers=cfg.num_hidden_layers, num_kv_heads=cfg.num_key_value_heads,
        head_dim=cfg.head_dim, max_seq_len=cfg.max_position_embeddings,
        max_num_pages=(batch + 64 + 2) * pages_per_request, page_size=args.page_size,
        num_qo_heads=cfg.num_attention_heads)
    # the reference's own generation defaults for this model are a temperature with top-p and
    # a repetition penalty (mstar/model/orpheus/config.py:44-48); the benchmark samples
    # greedily on both arms unless --sampling defaults
    if args.sampling == "greedy":
        sampling = SamplingConfig(vocab_size=cfg.vocab_size, temperature=0.0, ignore_eos=True)
    else:
        sampling = SamplingConfig(vocab_size=cfg.vocab_size, temperature=cfg.temperature,
                                  top_p=cfg.top_p, repetition_penalty=cfg.repetition_penalty,
                                  ignore_eos=True)
    engine = KVCacheEngine(autocast_dtype=torch.bfloat16)
    engine.load_model(
        submodules={"LLM": submodule},
        tp_groups=WorkerTPGroups(num_workers=1, global_rank=0),
        kv_cache_config=[kv_cfg], device=device,
        transfer_engine_info=TransferEngineInfo(
            my_entity_id="bench", my_session_id="localhost",
            transfer_engine=LocalTransferEngine("localhost")),
        default_sampling_config={"LLM": sampling})
    graphs = "off (--no-graphs)"
    if not args.no_graphs:
        log("engine.warmup(): capturing the reference's CUDA graphs ...")
        t0 = time.time()
        engine.warmup()
        runner = engine.submodule_management["LLM"].cuda_graph_runner
        graphs = f"{len(runner.graphs)} captured" if runner is not None else "none captured"
        log(f"warm-up took {time.time() - t0:.0f} s; graphs: {graphs}")

    g = torch.Generator().manual_seed(batch)
    prompts = torch.randint(0, cfg.vocab_size, (batch, PROMPT_LEN), generator=g)

    def info(rid: str, walk: str, index: int) -> CurrentForwardPassInfo:
        return CurrentForwardPassInfo(request_id=rid, graph_walk=walk, requires_cfg=False,
                                      fwd_index=index, random_seed=1, max_tokens=CONTEXT,
                                      sampling_config={"LLM": sampling})

    def execute(walk: str, rids: list, inputs: dict, index: int) -> dict:
        nb = NodeBatch(node_name="LLM", graph_walk=walk, request_ids=list(rids),
                       per_request_input_tensors={r: {"text_inputs": [inputs[r]]} for r in rids},
                       per_request_info={r: info(r, walk, index) for r in rids})
        try:
            out = engine.execute_batch(nb)
        finally:
            engine.finalize_batch(nb)
        if out.allocation_failed:
            raise RuntimeError("the reference's engine reported allocation_failed")
        return {r: out.per_request_output_tensors[r]["new_token"][0] for r in rids}

    def start(prefix: str) -> tuple:
        rids = [f"{prefix}{i}" for i in range(batch)]
        for r in rids:
            engine.add_request(r)
        tokens = {}
        # whole prompts, one request per prefill batch (the reference never cuts a prompt)
        for i, r in enumerate(rids):
            tokens.update(execute("prefill", [r], {r: prompts[i].to(device)}, 0))
        return rids, tokens

    def finish(rids: list) -> None:
        for r in rids:
            engine.remove_request(r)

    # ---- prefill of one 2,048-token prompt
    log("prefill ...")
    times = []
    for k in range(5):
        rid = f"p{k}"
        engine.add_request(rid)
        ids = torch.randint(0, cfg.vocab_size, (PROMPT_LEN,), generator=g).to(device)
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        execute("prefill", [rid], {rid: ids}, 0)
        b.record()
        torch.cuda.synchronize()
        engine.remove_request(rid)
        if k >= 2:
            times.append(a.elapsed_time(b))
    prefill_ms = statistics.median(times)

    # ---- decode, timed on the device
    log("decode ...")
    rids, tokens = start("d")
    index = 1
    for _ in range(warmup):
        tokens = execute("decode", rids, tokens, index)
        index += 1
    rounds = []
    for _ in range(args.rounds):
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(steps):
            tokens = execute("decode", rids, tokens, index)
            index += 1
        b.record()
        torch.cuda.synchronize()
        rounds.append(a.elapsed_time(b) / steps)
    finish(rids)
    ms = statistics.median(rounds)

    # ---- end to end: token ids leave for the host and come back from it every step
    log("end to end ...")
    rids, tokens = start("e")
    host = torch.stack([tokens[r].reshape(()) for r in rids]).cpu()
    pinned = torch.empty(batch, dtype=torch.long, pin_memory=True)
    e2e_rounds = []
    index = 1
    for rnd in range(args.rounds + 1):
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(steps if rnd else warmup):
            pinned.copy_(host)
            dev = pinned.to(device, non_blocking=True)
            tokens = execute("decode", rids, {r: dev[i:i + 1] for i, r in enumerate(rids)}, index)
            index += 1
            host = torch.stack([tokens[r].reshape(()) for r in rids]).cpu()
        torch.cuda.synchronize()
        if rnd:
            e2e_rounds.append((time.perf_counter() - t0) / steps * 1e3)
    finish(rids)
    e2e_ms = statistics.median(e2e_rounds)

    return {
        "impl": "reference",
        "metric": f"decode tok/s at batch {batch} (Orpheus 3B bf16, 2,048-token cached prompts)",
        "value": round(batch / (ms / 1e3), 1), "unit": "tokens/s", "n_gpus": 1,
        "steps": steps, "warmup": warmup, "ms_per_step": round(ms, 4),
        "ms_per_step_min": round(min(rounds), 4), "ms_per_step_max": round(max(rounds), 4),
        "rounds": len(rounds), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic token ids, random-init weights N(0, 0.02)",
        "config": {"model": "Orpheus 3B / Llama 3.2 3B", "global_batch": batch,
                   "seq_len": CONTEXT, "prompt_len": PROMPT_LEN, "parallelism": "single GPU",
                   "layers": cfg.num_hidden_layers, "layers_of_model": full_layers,
                   "page_size": args.page_size, "sampling": args.sampling,
                   "cuda_graphs": graphs,
                   "path": "KVCacheEngine.execute_batch, OrpheusLLMSubmodule, FlashInfer"},
        "e2e": {"value": round(batch / (e2e_ms / 1e3), 1), "unit": "tokens/s",
                "h2d_bytes_per_step": 8 * batch, "d2h_bytes_per_step": 8 * batch,
                "ms_per_step": round(e2e_ms, 4)},
        "prefill": {"value": round(PROMPT_LEN / (prefill_ms / 1e3), 1), "tokens": PROMPT_LEN,
                    "ms": round(prefill_ms, 3)},
    }


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--rounds", type=int, default=5)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--page-size", type=int, default=16)
    ap.add_argument("--layers", type=int, default=None)
    ap.add_argument("--sampling", default="greedy", choices=["greedy", "defaults"])
    ap.add_argument("--no-graphs", action="store_true",
                    help="skip engine.warmup(): batched eager instead of captured graphs")
    args = ap.parse_args()
    if not (REF / "mstar").is_dir():
        print(json.dumps({"impl": "reference", "unavailable":
                          "baseline/_ref holds no install of t-avil/mstar (pip install --no-index "
                          "--no-deps --target baseline/_ref <the reference's source tree>)"}))
        return 0
    try:
        record = run(args)
    except BaseException as exc:                      # whatever the reference raises is the answer
        traceback.print_exc(file=sys.stderr)
        last = traceback.extract_tb(exc.__traceback__)[-1]
        where = f"{Path(last.filename).name}:{last.lineno}"
        print(json.dumps({"impl": "reference", "unavailable":
                          f"{type(exc).__name__}: {str(exc)[:300]} (at {where})"}))
        return 0
    print(json.dumps(record))
    return 0


if __name__ == "__main__":
    sys.exit(main())
