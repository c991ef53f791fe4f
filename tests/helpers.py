"""Helpers of the GPU tests: build replay schedules, run them through the engine's
step function (in process, or through bin/trace_run), compare with the plain model."""
from __future__ import annotations

import json
import subprocess
import sys
from pathlib import Path

import numpy as np
import torch

import plain_llama as P

ROOT = Path(__file__).resolve().parent.parent

# Tolerances on logits (absolute; logits of the tiny models are of order 1, largest
# about 2.5).  float32: the plain model evaluated in float32 instead of float64 differs
# from itself by up to 4.4e-6 on these models, so 2e-5 is a few times plain float
# rounding.  bfloat16: activations are rounded to 8 bits of mantissa between parts
# (sums, softmax and the residual stay float); scaled from the float figure by the
# ratio of the roundings this predicts worst errors of 2e-2 to 3e-2.
TOL = {"float32": 2e-5, "bfloat16": 6e-2}
MEAN_TOL = {"float32": 2e-6, "bfloat16": 1.2e-2}


def request_tokens(vocab: int, length: int, seed: int) -> list:
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (length,), generator=g).tolist()


def whole(reqs: dict) -> list:
    """Each request alone and whole, one step each, every position wanted."""
    steps = []
    for rid, toks in reqs.items():
        steps.append({"entries": [{"id": rid, "tokens": toks, "want": list(range(len(toks)))}],
                      "end": [rid]})
    return steps


def prefill_then_decode(reqs: dict, tail: int = 32) -> list:
    """Most of each request in one step, its last ``tail`` tokens one by one."""
    steps = []
    for rid, toks in reqs.items():
        cut = max(len(toks) - tail, 1)
        steps.append({"entries": [{"id": rid, "tokens": toks[:cut],
                                   "want": list(range(cut))}], "end": []})
        for i in range(cut, len(toks)):
            steps.append({"entries": [{"id": rid, "tokens": [toks[i]], "want": [0]}],
                          "end": [rid] if i == len(toks) - 1 else []})
        if cut == len(toks):
            steps[-1]["end"] = [rid]
    return steps


def portions(reqs: dict, sizes=(7, 2, 13, 3, 2, 29, 5, 2, 64, 11)) -> list:
    """Portions of changing size, down to two tokens."""
    steps = []
    for rid, toks in reqs.items():
        pos, k = 0, 0
        while pos < len(toks):
            n = min(sizes[k % len(sizes)], len(toks) - pos)
            k += 1
            last = pos + n == len(toks)
            steps.append({"entries": [{"id": rid, "tokens": toks[pos:pos + n],
                                       "want": list(range(n))}], "end": [rid] if last else []})
            pos += n
    return steps


def mixed(reqs: dict, seed: int = 0, max_live: int = 4, prompt_frac: float = 0.6,
          sizes=(5, 2, 9, 17, 3, 2, 31)) -> list:
    """Up to ``max_live`` requests at a time: portions of the prompts of some beside
    single decoded tokens of others; a request may sit out a step; finished requests
    leave so that their pages are taken by the next."""
    rng = np.random.default_rng(seed)
    pending = list(reqs.items())
    live: dict = {}
    steps = []
    while pending or live:
        while pending and len(live) < max_live:
            rid, toks = pending.pop(0)
            live[rid] = {"toks": toks, "pos": 0, "prompt": max(int(len(toks) * prompt_frac), 1)}
        entries, end = [], []
        for rid, st in list(live.items()):
            if len(live) > 1 and rng.random() < 0.2:
                continue                      # left out of this step
            toks, pos = st["toks"], st["pos"]
            if pos < st["prompt"]:
                n = min(int(sizes[rng.integers(len(sizes))]), st["prompt"] - pos)
            else:
                n = 1
            entries.append({"id": rid, "tokens": toks[pos:pos + n], "want": list(range(n))})
            st["pos"] = pos + n
            if st["pos"] == len(toks):
                end.append(rid)
                del live[rid]
        if entries:
            steps.append({"entries": entries, "end": end})
    return steps


def serving(reqs: dict, prompt_len: dict, max_live: int, budget: int, order=None) -> list:
    """The steps a continuous-batching server would run: requests are admitted in order
    while fewer than ``max_live`` are live; every live request whose prompt is in brings one
    token, then prompt portions fill what is left of ``budget`` tokens (cut anywhere, down
    to one token); a request leaves after its last token, and its pages go to whoever
    comes next.  ``prompt_len[rid]`` tokens of a request are prompt, the rest are fed one
    by one as if they had been sampled."""
    pending = list(order or reqs)
    live: dict = {}
    steps = []
    while pending or live:
        while pending and len(live) < max_live:
            rid = pending.pop(0)
            live[rid] = 0
        left = budget
        entries, end = [], []
        for phase in ("decode", "prompt"):
            for rid in list(live):
                toks, pos = reqs[rid], live[rid]
                decoding = pos >= prompt_len[rid]
                if decoding != (phase == "decode") or left <= 0:
                    continue
                n = 1 if decoding else min(prompt_len[rid] - pos, left)
                entries.append({"id": rid, "tokens": toks[pos:pos + n],
                                "want": list(range(n))})
                left -= n
                live[rid] = pos + n
        for rid in list(live):
            if live[rid] == len(reqs[rid]):
                end.append(rid)
                del live[rid]
        assert entries, "budget too small for any progress"
        steps.append({"entries": entries, "end": end})
    return steps


def max_tokens_of(steps: list, page: int = 64) -> int:
    """The --max-tokens a trace needs: the most tokens live requests hold at any time,
    each request's count rounded up to a multiple of ``page``."""
    held: dict = {}
    worst = 0
    for st in steps:
        for e in st["entries"]:
            held[e["id"]] = held.get(e["id"], 0) + len(e["tokens"])
        worst = max(worst, sum(-(-n // page) * page for n in held.values()))
        for rid in st["end"]:
            held.pop(rid, None)
    return worst


def run_steps_in_process(stepper, steps: list, device_fed_seed=None, keep=None) -> dict:
    """Feed ``steps`` to a Stepper; returns {(request, position): logits row (cpu, f32)}.
    ``device_fed_seed``: about half of the single tokens (chosen by this seed) are not
    given to the step as values but left on the device, in a tensor that also holds other
    numbers, as the engine feeds the tokens a step sampled to the step after it.
    ``keep``: a set of (request, position); the engine still computes every wanted row,
    but only these are brought back."""
    from mstar_b200.engine.step import StepEntry

    out = {}
    pos = {}
    rng = None if device_fed_seed is None else np.random.default_rng(device_fed_seed)
    vocab = stepper.model.vocab_size
    for st in steps:
        entries, pending, fed = [], {}, []
        for e in st["entries"]:
            if not stepper.has_request(e["id"]):
                stepper.add_request(e["id"])
            tokens = e["tokens"]
            if rng is not None and len(tokens) == 1 and rng.random() < 0.5:
                pending[len(entries)] = len(fed)
                fed.append(tokens[0])
                tokens = [(tokens[0] + 1) % vocab]          # a wrong value: it must not be used
            entries.append(StepEntry(e["id"], tokens, e["want"]))
        if pending:
            perm = rng.permutation(len(fed) + 3)              # shuffled, among strangers
            place = {j: int(perm[j]) for j in range(len(fed))}
            values = [0] * (len(fed) + 3)
            for j, tok in enumerate(fed):
                values[place[j]] = tok
            dev_tokens = torch.tensor(values, dtype=torch.int32, device=stepper.device)
            logits = stepper.step(entries, {i: place[j] for i, j in pending.items()}, dev_tokens)
        else:
            logits = stepper.step(entries)
        keys = []
        for e in st["entries"]:
            base = pos.get(e["id"], 0)
            keys.extend((e["id"], base + w) for w in e["want"])
            pos[e["id"]] = base + len(e["tokens"])
        assert len(keys) == logits.shape[0]
        rows = [i for i, k in enumerate(keys) if keep is None or k in keep]
        if rows:
            if len(rows) < len(keys):
                logits = logits[torch.tensor(rows, device=logits.device)]
            host = logits.float().cpu()
            for j, i in enumerate(rows):
                out[keys[i]] = host[j]
        for rid in st["end"]:
            stepper.free_request(rid)
            pos.pop(rid, None)
    return out


def run_steps_with_trace_run(model_dir, dtype: str, steps: list, out_dir, vocab: int,
                             max_tokens: int) -> dict:
    """Drive bin/trace_run as a user would: one JSON line per step on stdin, wait for
    ``done <step>`` before the next."""
    cmd = [sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(model_dir),
           "--dtype", dtype, "--out", str(out_dir), "--max-tokens", str(max_tokens)]
    proc = subprocess.Popen(cmd, stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True)
    try:
        for i, st in enumerate(steps):
            proc.stdin.write(json.dumps({"step": i, **st}) + "\n")
            proc.stdin.flush()
            line = proc.stdout.readline().strip()
            assert line == f"done {i}", f"trace_run answered {line!r} to step {i}"
        proc.stdin.close()
        assert proc.wait(timeout=120) == 0
    finally:
        if proc.poll() is None:
            proc.kill()
    out, pos = {}, {}
    for i, st in enumerate(steps):
        n_want = sum(len(e["want"]) for e in st["entries"])
        f = Path(out_dir) / f"{i}.f32"
        if n_want == 0:
            assert not f.exists()
        else:
            arr = np.fromfile(f, dtype="<f4").reshape(n_want, vocab)
        row = 0
        for e in st["entries"]:
            base = pos.get(e["id"], 0)
            for w in e["want"]:
                out[(e["id"], base + w)] = torch.from_numpy(arr[row].copy())
                row += 1
            pos[e["id"]] = base + len(e["tokens"])
        for rid in st["end"]:
            pos.pop(rid, None)
    return out


def spread(a: dict, b: dict) -> tuple:
    """(largest, mean over rows of the mean) absolute difference of two sets of rows."""
    worst, total = 0.0, 0.0
    for key, row in a.items():
        err = (row.double() - b[key].double()).abs()
        worst = max(worst, err.max().item())
        total += err.mean().item()
    return worst, total / len(a)


def in_float32(fn):
    """``fn()`` with the plain model's sums in float32 (its roundings stay where they are)."""
    P.DT = torch.float32
    try:
        return fn()
    finally:
        P.DT = torch.float64


def kernel_rounding_yardstick(tensors: dict, raw_cfg: dict, reqs: dict) -> tuple:
    """How far the logits move through what a bfloat16 kernel does differently from the
    plain model beyond rounding its stored activations: the plain model with activations
    rounded to bfloat16 (``act=P.round_bf16``) against the same with its products summed in
    float32 and its attention probabilities rounded to bfloat16 before they multiply V.
    Nothing the engine computes enters.  Returns (max, mean) over all positions of
    ``reqs``."""
    a, b = {}, {}
    for rid, toks in reqs.items():
        x = P.plain_logits(tensors, raw_cfg, toks, act=P.round_bf16)
        y = in_float32(lambda: P.plain_logits(tensors, raw_cfg, toks, act=P.round_bf16,
                                              round_probs=P.round_bf16))
        for i in range(len(toks)):
            a[(rid, i)], b[(rid, i)] = x[i], y[i].double()
    return spread(a, b)


def plain_rows(tensors: dict, raw_cfg: dict, reqs: dict) -> dict:
    out = {}
    for rid, toks in reqs.items():
        logits = P.plain_logits(tensors, raw_cfg, toks)
        for i in range(len(toks)):
            out[(rid, i)] = logits[i]
    return out


def compare(got: dict, want: dict, dtype: str, what: str, tol=None, mean_tol=None) -> float:
    """Every wanted row within tolerance; on failure name the first wrong token.  ``tol``
    and ``mean_tol`` replace the tiny models' tolerances for models of another size."""
    assert got, f"{what}: no logits came back"
    tol = TOL[dtype] if tol is None else tol
    mean_tol = MEAN_TOL[dtype] if mean_tol is None else mean_tol
    worst, total, count = 0.0, 0.0, 0
    first_bad = None
    for key in sorted(got, key=lambda k: (str(k[0]), k[1])):
        err = (got[key].double() - want[key]).abs()
        m = err.max().item()
        total += err.mean().item()
        count += 1
        if m > tol and first_bad is None:
            first_bad = (key, m)
        worst = max(worst, m)
    assert first_bad is None, (f"{what} [{dtype}]: first wrong token is request "
                               f"{first_bad[0][0]!r} position {first_bad[0][1]} "
                               f"(max abs error {first_bad[1]:.3e}, tolerance {tol:.1e}; "
                               f"worst over all {worst:.3e})")
    assert total / count <= mean_tol, (f"{what} [{dtype}]: mean abs error "
                                       f"{total / count:.3e} > {mean_tol:.1e}")
    return worst
