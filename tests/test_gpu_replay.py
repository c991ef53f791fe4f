"""The engine's step function against the plain model under every way of cutting the
work, in float32 and in bfloat16, on both tiny configurations."""
import pytest
import torch

import helpers as H

pytestmark = pytest.mark.gpu

PAGE = {"tiny_a": 4, "tiny_b": 8}
LENGTHS = {"tiny_a": [5, 9, 17, 70, 133], "tiny_b": [1, 7, 33, 40, 101, 150]}

_models: dict = {}
_plain: dict = {}


def get_model(model_folders, name, dtype):
    from mstar_b200.engine.model import load_model

    key = (name, dtype)
    if key not in _models:
        folder, _, _ = model_folders[name]
        _models[key] = load_model(folder, dtype=dtype, device="cuda:0")
    return _models[key]


def get_requests(model_folders, name):
    _, raw, tensors = model_folders[name]
    reqs = {f"r{i}": H.request_tokens(raw["vocab_size"], n, seed=100 + i)
            for i, n in enumerate(LENGTHS[name])}
    if name not in _plain:
        _plain[name] = H.plain_rows(tensors, raw, reqs)
    return reqs, _plain[name]


def run(model_folders, name, dtype, steps, what, page=None, slack_pages=0):
    from mstar_b200.engine.step import make_stepper

    model = get_model(model_folders, name, dtype)
    page = page or PAGE[name]
    pages = H.max_tokens_of(steps, page) // page + slack_pages
    stepper = make_stepper(model, page_size=page, num_pages=pages, num_slots=8)
    reqs, want = get_requests(model_folders, name)
    got = H.run_steps_in_process(stepper, steps)
    assert stepper.manager.check() == 0
    assert stepper.manager.num_requests() == 0
    assert stepper.manager.free_pages(0) == pages
    return H.compare(got, want, dtype, what)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["tiny_a", "tiny_b"])
class TestCuttings:
    def test_whole(self, model_folders, name, dtype):
        reqs, _ = get_requests(model_folders, name)
        run(model_folders, name, dtype, H.whole(reqs), "whole prompts")

    def test_prefill_then_last_32_one_by_one(self, model_folders, name, dtype):
        reqs, _ = get_requests(model_folders, name)
        run(model_folders, name, dtype, H.prefill_then_decode(reqs, 32), "prefill + decode")

    def test_portions_of_changing_size(self, model_folders, name, dtype):
        reqs, _ = get_requests(model_folders, name)
        run(model_folders, name, dtype, H.portions(reqs), "portions")

    def test_mixed_batches_with_page_reuse(self, model_folders, name, dtype):
        reqs, _ = get_requests(model_folders, name)
        for seed in (0, 1):
            steps = H.mixed(reqs, seed=seed)
            assert max(len(s["entries"]) for s in steps) >= 3
            # the pool is the minimum the trace needs, so freed pages are taken again
            total_pages = sum(-(-len(t) // PAGE[name]) for t in reqs.values())
            assert H.max_tokens_of(steps, PAGE[name]) // PAGE[name] < total_pages
            run(model_folders, name, dtype, steps, f"mixed batches (seed {seed})")

    def test_long_decoding(self, model_folders, name, dtype):
        reqs, _ = get_requests(model_folders, name)
        rid = max(reqs, key=lambda r: len(reqs[r]))
        one = {rid: reqs[rid]}
        run(model_folders, name, dtype, H.prefill_then_decode(one, len(reqs[rid]) - 3),
            "long decoding")

    def test_first_tokens(self, model_folders, name, dtype):
        reqs, _ = get_requests(model_folders, name)
        rid = max(reqs, key=lambda r: len(reqs[r]))
        toks = reqs[rid][:4]
        steps = [{"entries": [{"id": rid, "tokens": [t], "want": [0]}],
                  "end": [rid] if i == 3 else []} for i, t in enumerate(toks)]
        run(model_folders, name, dtype, steps, "first tokens")

    def test_other_page_size(self, model_folders, name, dtype):
        reqs, _ = get_requests(model_folders, name)
        run(model_folders, name, dtype, H.mixed(reqs, seed=5), "mixed, page 16", page=16)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_cuttings_agree_with_each_other(model_folders, dtype):
    """Beyond agreeing with the plain model, different cuttings agree with each other:
    in float32 to 1e-6, the same row going through the same arithmetic; in bfloat16, where
    a portion and a single token go through different attention kernels, within what such
    kernel-internal differences (the order of float sums, probabilities held in bfloat16)
    move the plain model's own logits on these requests (``kernel_rounding_yardstick``)."""
    from mstar_b200.engine.step import make_stepper

    name = "tiny_b"
    model = get_model(model_folders, name, dtype)
    reqs, _ = get_requests(model_folders, name)
    outs = []
    for steps in (H.whole(reqs), H.portions(reqs), H.mixed(reqs, seed=3)):
        stepper = make_stepper(model, page_size=8, num_pages=200, num_slots=8)
        outs.append(H.run_steps_in_process(stepper, steps))
    if dtype == "float32":
        tol = 1e-6
    else:
        _, raw, tensors = model_folders[name]
        tol = H.kernel_rounding_yardstick(tensors, raw, reqs)[0]
    worst = 0.0
    for other in outs[1:]:
        for key, row in outs[0].items():
            worst = max(worst, (row - other[key]).abs().max().item())
            assert worst <= tol, (key, worst, tol)
    print(f"cuttings differ from each other by {worst:.3e} at most [{dtype}] (allowed {tol:.3e})")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_program(model_folders, dtype, tmp_path):
    """bin/trace_run as a user drives it, mixed batches with a minimal pool."""
    name = "tiny_b"
    folder, raw, _ = model_folders[name]
    reqs, want = get_requests(model_folders, name)
    steps = H.mixed(reqs, seed=7)
    steps.insert(2, {"entries": [{"id": "quiet", "tokens": [1, 2, 3], "want": []}],
                     "end": ["quiet"]})     # a step that wants nothing writes no file
    got = H.run_steps_with_trace_run(folder, dtype, steps, tmp_path, raw["vocab_size"],
                                     H.max_tokens_of(steps, 64))
    H.compare(got, want, dtype, "trace_run")


def test_cache_exhaustion_leaves_state_unchanged(model_folders):
    from mstar_b200.cache import CacheExhausted
    from mstar_b200.engine.step import StepEntry, make_stepper

    model = get_model(model_folders, "tiny_a", "float32")
    stepper = make_stepper(model, page_size=4, num_pages=3, num_slots=2)
    stepper.add_request("a")
    stepper.step([StepEntry("a", [1, 2, 3, 4, 5], [4])])
    stepper.add_request("b")
    with pytest.raises(CacheExhausted):
        stepper.step([StepEntry("a", [6], [0]), StepEntry("b", [1, 2, 3, 4, 5, 6], [])])
    assert stepper.manager.length("a") == 5 and stepper.manager.length("b") == 0
    assert stepper.manager.free_pages(0) == 1 and stepper.manager.check() == 0
    stepper.step([StepEntry("a", [6], [0]), StepEntry("b", [1, 2], [])])   # this fits
    assert stepper.manager.length("a") == 6 and stepper.manager.length("b") == 2


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_decode_steps_replay_cuda_graphs_with_the_same_logits(model_folders, dtype):
    """Single-token batches run as replays of captured graphs (padded to a captured
    batch size, block tables padded to a fixed width); the logits must be the ones the
    eager path gives, for every batch size from 1 to 5 and across a width change."""
    from mstar_b200.engine.step import make_stepper

    name = "tiny_b"
    model = get_model(model_folders, name, dtype)
    reqs, want = get_requests(model_folders, name)
    reqs = {k: v for k, v in reqs.items() if len(v) > 1}
    steps = H.prefill_then_decode(reqs, 32)                 # one request at a time
    # and all requests decoding together: lengths differ, requests drop out one by one
    together = [{"entries": [{"id": r, "tokens": t[:1], "want": [0]} for r, t in reqs.items()],
                 "end": []}]
    longest = max(len(t) for t in reqs.values())
    for pos in range(1, longest):
        entries = [{"id": r, "tokens": [t[pos]], "want": [0]} for r, t in reqs.items()
                   if pos < len(t)]
        end = [r for r, t in reqs.items() if pos == len(t) - 1]
        together.append({"entries": entries, "end": end})
    for trace, what in ((steps, "graphs, one request"), (together, "graphs, batch")):
        outs = {}
        for graphs in (True, False):
            stepper = make_stepper(model, page_size=8, num_pages=200, num_slots=8,
                                   cuda_graphs=graphs)
            outs[graphs] = H.run_steps_in_process(stepper, trace)
            assert (stepper.graph_replays > 0) == graphs
            assert stepper.manager.check() == 0 and stepper.manager.free_pages(0) == 200
        H.compare(outs[True], want, dtype, what)
        # a replayed step runs the kernels of the eager step; only the number of key
        # splits may differ with the padded batch (bfloat16: sums in another order)
        tol = 1e-6 if dtype == "float32" else 4e-3
        for key, row in outs[False].items():
            assert (row - outs[True][key]).abs().max().item() <= tol, key


@pytest.mark.parametrize("switch", [("MSTAR_FUSED_ROPE", "0"), ("MSTAR_SKINNY", "1"),
                                    ("MSTAR_DECODE_ATTENTION", "per_item")])
@pytest.mark.parametrize("name", ["tiny_a", "tiny_b"])
def test_other_kernels_of_a_measurement_switch_give_the_same_model(model_folders, name, switch,
                                                                  monkeypatch):
    """The kernels that the measurement switches select instead of the default ones run the
    same requests within the same tolerances: decode steps (single tokens, where the
    small-M products, the fused first product and the decode attention are chosen) and a
    mixed batch, in bfloat16."""
    monkeypatch.setenv(*switch)
    reqs, _ = get_requests(model_folders, name)
    run(model_folders, name, "bfloat16", H.prefill_then_decode(reqs, 32), f"{switch[0]}: decode")
    run(model_folders, name, "bfloat16", H.mixed(reqs, seed=0), f"{switch[0]}: mixed")
