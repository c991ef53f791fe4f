"""The ``mstar`` command of this engine.

    mstar generate MODEL_DIR --prompt-ids 128259,791,1917,128009 --temperature 0
    mstar generate MODEL_DIR --prompt-file prompts.jsonl --max-output-tokens 64
    mstar random-model CONFIG_JSON OUT_DIR --seed 0
    mstar replay --model DIR --dtype float32 --out DIR --max-tokens N < trace.jsonl

Options keep the reference CLI's names and meanings where it has them
(mstar/cli/main.py:138-167: positional model, --gpus, --config, --log-level,
--log-stats, --log-stats-file); the deployment file given with --config carries, as in
the reference's YAML (docs/serving.rst:161-238), ``max_concurrent_requests``,
``autocast_dtype`` and a ``kv_cache:`` section with ``page_size`` and ``max_num_pages``.
Sampling options are the fields of the reference's SamplingConfig
(mstar/utils/sampling.py:207-226).  ``serve`` (an HTTP server) is not part of this
engine; prompts are token ids because tokenisation lives in the reference's API server.
"""
from __future__ import annotations

import argparse
import json
import logging
import os
import sys
import time
from pathlib import Path


def _read_deployment(path: str | None) -> dict:
    if not path:
        return {}
    p = Path(path)
    if not p.exists():
        sys.exit(f"error: --config path not found: {path}")
    text = p.read_text()
    if p.suffix in (".yaml", ".yml"):
        import yaml

        return yaml.safe_load(text) or {}
    return json.loads(text)


def _prompts(args) -> list:
    prompts = []
    if args.prompt_ids:
        for item in args.prompt_ids:
            prompts.append([int(t) for t in item.replace(" ", "").split(",") if t])
    if args.prompt_file:
        for line in Path(args.prompt_file).read_text().splitlines():
            line = line.strip()
            if line:
                obj = json.loads(line)
                prompts.append(obj["prompt_token_ids"] if isinstance(obj, dict) else obj)
    if not prompts:
        sys.exit("error: give --prompt-ids or --prompt-file")
    return prompts


def _generate(args) -> None:
    if args.gpus is not None:
        os.environ["CUDA_VISIBLE_DEVICES"] = args.gpus
    logging.basicConfig(level=getattr(logging, args.log_level))
    deploy = _read_deployment(args.config)
    kv = deploy.get("kv_cache") or {}

    from mstar_b200 import LLM, SamplingParams
    from mstar_b200.config.base import GenerationDefaults

    dtype = args.dtype or deploy.get("autocast_dtype") or "bfloat16"
    llm = LLM(args.model, dtype=dtype,
              page_size=args.page_size or kv.get("page_size", 64),
              max_num_pages=args.max_num_pages or kv.get("max_num_pages"),
              max_num_batched_tokens=args.max_num_batched_tokens,
              max_concurrent_requests=args.max_concurrent_requests
              or deploy.get("max_concurrent_requests", 64),
              log_stats=args.log_stats or bool(args.log_stats_file))
    d = GenerationDefaults.from_folder(args.model)

    def pick(value, default):
        return default if value is None else value

    params = SamplingParams(
        temperature=pick(args.temperature, d.temperature), top_k=pick(args.top_k, d.top_k),
        top_p=pick(args.top_p, d.top_p),
        repetition_penalty=pick(args.repetition_penalty, d.repetition_penalty),
        ignore_eos=args.ignore_eos or d.ignore_eos,
        max_output_tokens=pick(args.max_output_tokens, d.max_new_tokens), seed=args.seed)
    prompts = _prompts(args)
    t0 = time.perf_counter()
    results = llm.generate(prompts, params)
    elapsed = time.perf_counter() - t0
    for r in results:
        print(json.dumps({"request_id": r.request_id, "token_ids": r.token_ids,
                          "finish_reason": r.finish_reason}))
    if args.log_stats or args.log_stats_file:
        s = llm.stats
        report = (f"requests={len(results)} steps={s.steps} prompt_tokens={s.prompt_tokens} "
                  f"generated_tokens={s.generated_tokens} preemptions={s.preemptions} "
                  f"seconds={elapsed:.3f} tokens_per_second={s.generated_tokens / elapsed:.1f}")
        print(report, file=sys.stderr)
        if args.log_stats_file:
            with open(args.log_stats_file, "a") as f:
                f.write(report + "\n")


def _random_model(args) -> None:
    from mstar_b200.config.registry import config_from_dict
    from mstar_b200.weights.random_init import write_model_folder

    raw = json.loads(Path(args.config_json).read_text())
    cfg = config_from_dict(raw)
    out = write_model_folder(args.out_dir, cfg, args.seed, std=args.std,
                             norm_noise=args.norm_noise)
    print(out)


def _replay(args) -> None:
    from mstar_b200.engine.replay import main as replay_main

    sys.exit(replay_main(args.rest))


def build_parser() -> argparse.ArgumentParser:
    parser = argparse.ArgumentParser(prog="mstar", description="mstar_b200 inference CLI")
    sub = parser.add_subparsers(dest="command", required=True)

    gen = sub.add_parser("generate", help="generate tokens for token-id prompts")
    gen.add_argument("model", help="model folder (config.json + model.safetensors)")
    gen.add_argument("--gpus", default=None, help="CUDA_VISIBLE_DEVICES, e.g. '0'")
    gen.add_argument("--config", default=None, help="deployment file (YAML or JSON)")
    gen.add_argument("--dtype", default=None, choices=["bfloat16", "float32"])
    gen.add_argument("--prompt-ids", action="append",
                     help="comma-separated token ids; may be given several times")
    gen.add_argument("--prompt-file", default=None,
                     help="JSON lines: a list of token ids, or {\"prompt_token_ids\": [...]}")
    gen.add_argument("--temperature", type=float, default=None)
    gen.add_argument("--top-k", type=int, default=None)
    gen.add_argument("--top-p", type=float, default=None)
    gen.add_argument("--repetition-penalty", type=float, default=None)
    gen.add_argument("--ignore-eos", action="store_true")
    gen.add_argument("--max-output-tokens", type=int, default=None)
    gen.add_argument("--seed", type=int, default=None)
    gen.add_argument("--page-size", type=int, default=None)
    gen.add_argument("--max-num-pages", type=int, default=None)
    gen.add_argument("--max-num-batched-tokens", type=int, default=2048)
    gen.add_argument("--max-concurrent-requests", type=int, default=None)
    gen.add_argument("--log-level", default="INFO",
                     choices=["DEBUG", "INFO", "WARNING", "ERROR"])
    gen.add_argument("--log-stats", action="store_true",
                     help="print engine statistics when generation ends")
    gen.add_argument("--log-stats-file", default=None,
                     help="append engine statistics to this file (implies --log-stats)")
    gen.set_defaults(func=_generate)

    rnd = sub.add_parser("random-model", help="write a random-weight model folder")
    rnd.add_argument("config_json", help="a config.json of a known architecture")
    rnd.add_argument("out_dir")
    rnd.add_argument("--seed", type=int, default=0)
    rnd.add_argument("--std", type=float, default=0.02)
    rnd.add_argument("--norm-noise", type=float, default=0.0)
    rnd.set_defaults(func=_random_model)

    rep = sub.add_parser("replay", help="trace replay (same options as bin/trace_run)")
    rep.add_argument("rest", nargs=argparse.REMAINDER)
    rep.set_defaults(func=_replay)
    return parser


def main(argv: list[str] | None = None) -> None:
    parser = build_parser()
    args = parser.parse_args(argv)
    args.func(args)


if __name__ == "__main__":
    main()
