"""Trace replay: feed given token ids through a model step by step and write logits.

    trace_run --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N

Steps are read from standard input, one JSON object per line:

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

All entries of a step form one batch for the engine's own step function (the one
generation uses); nothing is sampled.  For a step that wants something, the float32
logits [wanted, vocab] are written little-endian to ``<out>/<step>.f32``.  After
every step ``done <step>`` is printed and flushed.  Requests named in ``end`` give
back what they hold after the step.  The cache pool is sized for ``--max-tokens``
tokens held by live requests, each request's count rounded up to whole pages, so
that pages are reused.

The reference has no such program; its closest facility is reading back static
logits in a CUDA-graph parity test (test/integration/test_prefill_cuda_graph.py:17-21).
"""
from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

PAGE_SIZE = 16
MAX_LIVE_REQUESTS = 64


def build_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    p.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    p.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    p.add_argument("--out", required=True, help="folder for <step>.f32 files")
    p.add_argument("--max-tokens", type=int, required=True,
                   help="most tokens that live requests hold at any time")
    p.add_argument("--page-size", type=int, default=PAGE_SIZE)
    p.add_argument("--device", default="cuda:0")
    return p


def main(argv=None) -> int:
    args = build_parser().parse_args(argv)
    import numpy as np
    import torch

    from .. import ops
    from .model import load_model
    from .step import StepEntry, make_stepper

    out_dir = Path(args.out)
    out_dir.mkdir(parents=True, exist_ok=True)
    print(f"[trace_run] loading {args.model} as {args.dtype}", file=sys.stderr, flush=True)
    model = load_model(args.model, dtype=args.dtype, device=args.device)
    # one spare page per live request covers a request's last, partly filled page
    pages = -(-args.max_tokens // args.page_size) + 0
    stepper = make_stepper(model, page_size=args.page_size, num_pages=max(pages, 1),
                           num_slots=MAX_LIVE_REQUESTS)
    print(f"[trace_run] ready: {pages} pages of {args.page_size} tokens", file=sys.stderr,
          flush=True)

    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        record = json.loads(line)
        step_id = record["step"]
        entries = []
        for e in record.get("entries", []):
            if not stepper.has_request(e["id"]):
                stepper.add_request(e["id"])
            entries.append(StepEntry(e["id"], e["tokens"], e.get("want", [])))
        logits = stepper.step(entries)
        host = None
        if logits.shape[0] > 0:
            host = logits.to("cpu", torch.float32).contiguous().numpy().astype("<f4", copy=False)
        # a kernel whose bounded wait ran out has left partial output: fail, do not write on
        ops.check_error_word(model.runtime.device)
        if host is not None:
            host.tofile(out_dir / f"{step_id}.f32")
        for rid in record.get("end", []):
            if stepper.has_request(rid):
                stepper.free_request(rid)
        print(f"done {step_id}", flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
