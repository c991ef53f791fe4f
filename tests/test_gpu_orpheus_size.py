"""The benchmark model's layer sizes (Orpheus 3B / Llama 3.2 3B: width 3072, 24 query and
8 key/value heads of 128, feed-forward 8192, vocabulary 156,940, tied head, llama3 rotary
scaling x32) with two layers, against the plain model: whole prompt, portions, and a
mixed batch.  At these sizes the product path runs the kernels serving runs: the
tcgen05 gate/up and LM-head products, the small-M products, the tensor-core attention.
The same at the layer sizes of Llama 3.2 1B (width 2048, 32 query heads of 64) and of
Llama 3.1 8B (width 4096, feed-forward 14336, a head of its own, scaling x8)."""
import pytest
import torch

import helpers as H
import plain_llama as P

pytestmark = pytest.mark.gpu

CFG = dict(
    architectures=["LlamaForCausalLM"], num_hidden_layers=2, hidden_size=3072,
    num_attention_heads=24, num_key_value_heads=8, head_dim=128, intermediate_size=8192,
    vocab_size=156940, tie_word_embeddings=True, rope_theta=500000.0,
    rope_scaling={"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0,
                  "high_freq_factor": 4.0, "original_max_position_embeddings": 8192},
    rms_norm_eps=1e-5, max_position_embeddings=131072, hidden_act="silu",
)
SIZES = {
    "3b": CFG,
    "1b": dict(CFG, hidden_size=2048, num_attention_heads=32, head_dim=64, vocab_size=128256),
    "8b": dict(CFG, hidden_size=4096, num_attention_heads=32, intermediate_size=14336,
               vocab_size=128256, tie_word_embeddings=False,
               rope_scaling=dict(CFG["rope_scaling"], factor=8.0)),
}
LENGTHS = [150, 37]
# Tolerances at this size, derived as for the tiny models (tests/helpers.py): the plain
# model evaluated in float32 instead of float64 differs from itself by 2.9e-5 (max) and
# 2.8e-6 (mean) here, against 4.4e-6 on the tiny models whose float32 tolerance is 2e-5:
# the same factor gives 1.3e-4 / 1.3e-5.  bfloat16: the plain model with its activations
# rounded to bfloat16 at the places where the engine stores bfloat16 (normed rows, q, k,
# v, attention output, projections, gate, up, their product) differs from float64 by
# 0.18 (max) and 0.018 (mean) on these requests, logits being as large as 5.5; the
# tolerance is 1.5 times that rounding noise.  The other sizes by the same two rules
# from their own noise: 1B 1.4e-5 / 1.5e-6 in float32 and 0.086 / 0.0105 in bfloat16,
# 8B 2.7e-5 / 3.0e-6 and 0.20 / 0.020.
TOLS = {"3b": {"float32": (1.3e-4, 1.3e-5), "bfloat16": (0.27, 0.027)},
        "1b": {"float32": (6.2e-5, 6.9e-6), "bfloat16": (0.13, 0.0158)},
        "8b": {"float32": (1.2e-4, 1.37e-5), "bfloat16": (0.305, 0.030)}}


ROUNDED: dict = {}     # size -> (logits of the rounded plain model, tolerance against them)


@pytest.fixture(scope="module", params=["3b", "1b", "8b"])
def big(request):
    from mstar_b200.config.registry import config_from_dict
    from mstar_b200.weights.random_init import random_checkpoint

    size = request.param
    CFG = SIZES[size]
    cfg = config_from_dict(CFG)
    tensors = random_checkpoint(cfg, seed=3, std=0.02, device="cuda:0")
    for key in tensors:                       # sharper attention, as in the tiny models
        if key.endswith("q_proj.weight") or key.endswith("k_proj.weight"):
            tensors[key] = (tensors[key].float() * 2.0).to(torch.bfloat16)
    reqs = {f"o{i}": H.request_tokens(CFG["vocab_size"], n, seed=70 + i)
            for i, n in enumerate(LENGTHS)}
    # the plain model's float64 products run where the weights are, on the GPU.  Beside the
    # float64 logits, the second bfloat16 oracle (activations rounded where the engine
    # stores bfloat16) and the yardstick for what remains between it and a bfloat16 kernel
    # (tests/helpers.py kernel_rounding_yardstick, here on the compared rows only)
    want, rounded, rounded32 = {}, {}, {}
    head = tensors["model.embed_tokens.weight" if CFG["tie_word_embeddings"]
                   else "lm_head.weight"].double()
    for rid, toks in reqs.items():
        rows = sorted({0, 1, 15, 16, 17, len(toks) // 2, len(toks) - 2, len(toks) - 1})
        logits = (P.plain_hidden_states(tensors, CFG, toks)[rows] @ head.T).cpu()
        bf = (P.plain_hidden_states(tensors, CFG, toks, act=P.round_bf16)[rows] @ head.T).cpu()
        bf32 = (H.in_float32(lambda: P.plain_hidden_states(
            tensors, CFG, toks, act=P.round_bf16, round_probs=P.round_bf16))[rows].double()
            @ head.T).cpu()
        for i, r in enumerate(rows):
            want[(rid, r)], rounded[(rid, r)], rounded32[(rid, r)] = logits[i], bf[i], bf32[i]
    del head
    pushes = H.spread(rounded32, rounded)
    ROUNDED[size] = (rounded, (2 * pushes[0], 2 * pushes[1]))
    return size, cfg, tensors, reqs, want


def only_wanted(steps, want):
    """Keep `want` only at the positions the plain logits were computed for."""
    pos = {}
    for st in steps:
        for e in st["entries"]:
            base = pos.get(e["id"], 0)
            e["want"] = [w for w in e["want"] if (e["id"], base + w) in want]
            pos[e["id"]] = base + len(e["tokens"])
    return steps


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_orpheus_sized_layers_match_the_plain_model(big, dtype):
    from mstar_b200.engine.model import load_model
    from mstar_b200.engine.step import make_stepper

    size, cfg, tensors, reqs, want = big
    tol, mean_tol = TOLS[size][dtype]
    model = load_model(None, dtype=dtype, device="cuda:0", config=cfg, tensors=tensors)
    for steps, what in ((H.whole(reqs), f"{size}-sized layers, whole"),
                        (H.portions(reqs, sizes=(64, 2, 30, 17)), f"{size}-sized layers, portions"),
                        (H.mixed(reqs, seed=1, prompt_frac=0.8), f"{size}-sized layers, mixed")):
        steps = only_wanted(steps, want)
        pages = H.max_tokens_of(steps, 16) // 16
        stepper = make_stepper(model, page_size=16, num_pages=pages, num_slots=4)
        got = H.run_steps_in_process(stepper, steps)
        assert set(got) == set(want)
        worst = H.compare(got, want, dtype, what, tol=tol, mean_tol=mean_tol)
        print(f"{what} [{dtype}]: worst abs error {worst:.3e}")
        if dtype == "bfloat16":
            rounded, (rtol, rmean) = ROUNDED[size]
            worst = H.compare(got, rounded, dtype, what + ", against the rounded plain model",
                              tol=rtol, mean_tol=rmean)
            print(f"{what} [rounded plain model]: worst abs error {worst:.3e} of {rtol:.3e}")
    del model
    torch.cuda.empty_cache()


# A request of 2,500 tokens at the 3B layer sizes: prompt portions of 1,024 (the second and
# third attend to keys that earlier steps cached, over several key tiles and pages), then the
# last 8 tokens one by one (decode kernels with their keys split).  Places checked: the
# first token, both sides of the portion edges, the decoded tail.  Tolerances by the rules
# above from this request's own noise (float32 3.7e-5 / 4.6e-6, bfloat16 0.19 / 0.025).
LONG = 2500
LONG_ROWS = [0, 1023, 1024, 1025, 2047, 2048, 2300, 2491, 2492, 2495, 2498, 2499]
LONG_TOLS = {"float32": (1.7e-4, 2.1e-5), "bfloat16": (0.29, 0.037)}


@pytest.fixture(scope="module")
def long_request():
    from mstar_b200.config.registry import config_from_dict
    from mstar_b200.weights.random_init import random_checkpoint

    cfg = config_from_dict(CFG)
    tensors = random_checkpoint(cfg, seed=3, std=0.02, device="cuda:0")
    for key in tensors:
        if key.endswith("q_proj.weight") or key.endswith("k_proj.weight"):
            tensors[key] = (tensors[key].float() * 2.0).to(torch.bfloat16)
    toks = H.request_tokens(CFG["vocab_size"], LONG, seed=90)
    cpu = {k: v.cpu() for k, v in tensors.items()}
    hidden = P.plain_hidden_states(cpu, CFG, toks)
    logits = hidden[LONG_ROWS] @ cpu["model.embed_tokens.weight"].double().T
    want = {("long", r): logits[i] for i, r in enumerate(LONG_ROWS)}
    return cfg, tensors, toks, want


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_request_in_portions_then_decoded(long_request, dtype):
    from mstar_b200.engine.model import load_model
    from mstar_b200.engine.step import make_stepper

    cfg, tensors, toks, want = long_request
    model = load_model(None, dtype=dtype, device="cuda:0", config=cfg, tensors=tensors)
    steps, pos = [], 0
    cuts = [1024, 1024, LONG - 2048 - 8] + [1] * 8
    for n in cuts:
        steps.append({"step": len(steps), "entries": [
            {"id": "long", "tokens": toks[pos:pos + n], "want": list(range(n))}], "end": []})
        pos += n
    assert pos == LONG
    steps[-1]["end"] = ["long"]
    steps = only_wanted(steps, want)
    stepper = make_stepper(model, page_size=64, num_pages=-(-LONG // 64), num_slots=2)
    got = H.run_steps_in_process(stepper, steps)
    assert set(got) == set(want)
    tol, mean_tol = LONG_TOLS[dtype]
    worst = H.compare(got, want, dtype, "a long request in portions", tol=tol, mean_tol=mean_tol)
    print(f"long request [{dtype}]: worst abs error {worst:.3e}")
    del model
    torch.cuda.empty_cache()


@pytest.mark.parametrize("switch", [("MSTAR_FUSED_ROPE", "0"), ("MSTAR_SKINNY", "1"),
                                    ("MSTAR_DECODE_ATTENTION", "per_item")])
def test_measurement_switches_at_these_sizes(big, switch, monkeypatch):
    """The kernels a measurement switch selects instead of the default ones (the first product
    and the rotary kernel apart, decode attention with one CTA per item), on the mixed trace
    in bfloat16, within the same tolerances."""
    from mstar_b200.engine.model import load_model
    from mstar_b200.engine.step import make_stepper

    monkeypatch.setenv(*switch)
    size, cfg, tensors, reqs, want = big
    tol, mean_tol = TOLS[size]["bfloat16"]
    model = load_model(None, dtype="bfloat16", device="cuda:0", config=cfg, tensors=tensors)
    steps = only_wanted(H.mixed(reqs, seed=1, prompt_frac=0.8), want)
    pages = H.max_tokens_of(steps, 16) // 16
    stepper = make_stepper(model, page_size=16, num_pages=pages, num_slots=4)
    got = H.run_steps_in_process(stepper, steps)
    assert set(got) == set(want)
    H.compare(got, want, "bfloat16", f"{size}-sized layers, {switch[0]}", tol=tol, mean_tol=mean_tol)
    del model
    torch.cuda.empty_cache()
