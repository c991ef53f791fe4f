"""Generation through the Python entry point and the command line."""
import json
import subprocess
import sys

import pytest
import torch

import helpers as H
import plain_llama as P

pytestmark = pytest.mark.gpu


def check_greedy_chain(prompt, token_ids, tensors, raw, dtype):
    """Every token is the plain model's greedy choice after the tokens before it; only a
    near-tie may be decided differently, and only in bfloat16."""
    ids = list(prompt)
    for k, tok in enumerate(token_ids):
        logits = P.plain_logits(tensors, raw, ids)[-1]
        best = int(logits.argmax())
        if tok != best:
            assert dtype == "bfloat16", (prompt, k, tok, best)
            assert (logits[best] - logits[tok]).item() < 2 * H.TOL["bfloat16"], (k, tok, best)
        ids.append(tok)


def check_greedy(results, prompts, tensors, raw, dtype, n_new):
    for prompt, res in zip(prompts, results):
        assert res.finish_reason == "length" and len(res.token_ids) == n_new
        check_greedy_chain(prompt, res.token_ids, tensors, raw, dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["tiny_a", "tiny_b"])
def test_greedy_generation_matches_the_plain_model(model_folders, name, dtype):
    from mstar_b200 import LLM, SamplingParams

    folder, raw, tensors = model_folders[name]
    lengths = [5, 9, 17] if name == "tiny_a" else [1, 7, 33, 40]
    prompts = [H.request_tokens(raw["vocab_size"], n, seed=200 + n) for n in lengths]
    # portions of 16 tokens at most, small pages: prompts are cut and mixed with decoding
    llm = LLM(folder, dtype=dtype, page_size=4 if name == "tiny_a" else 8, max_num_pages=64,
              max_num_batched_tokens=16)
    params = SamplingParams(temperature=0.0, max_output_tokens=8, ignore_eos=True)
    results = llm.generate(prompts, params)
    check_greedy(results, prompts, tensors, raw, dtype, 8)
    assert llm.stepper.manager.num_requests() == 0 and llm.stepper.manager.check() == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_preemption_does_not_change_greedy_tokens(model_folders, dtype):
    """A pre-empted request computes its prompt and what it had generated again, as one
    prompt; in float32 the tokens are those of a run with room for everyone, in bfloat16
    (where the second computation goes through other kernels than the first) they are the
    plain model's greedy tokens up to near-ties."""
    from mstar_b200 import LLM, SamplingParams

    folder, raw, tensors = model_folders["tiny_b"]
    prompts = [H.request_tokens(raw["vocab_size"], n, seed=300 + n) for n in (20, 22, 24)]
    params = SamplingParams(temperature=0.0, max_output_tokens=24, ignore_eos=True)
    roomy = LLM(folder, dtype=dtype, page_size=8, max_num_pages=64).generate(prompts, params)
    tight_llm = LLM(folder, dtype=dtype, page_size=8, max_num_pages=12)
    tight = tight_llm.generate(prompts, params)
    assert tight_llm.stats.preemptions > 0
    if dtype == "float32":
        assert [r.token_ids for r in tight] == [r.token_ids for r in roomy]
    check_greedy(tight, prompts, tensors, raw, dtype, 24)
    assert sum(r.preemptions for r in tight) == tight_llm.stats.preemptions
    assert tight_llm.stepper.manager.num_requests() == 0 and tight_llm.stepper.manager.check() == 0


def test_sampling_options_through_the_entry_point(model_folders):
    from mstar_b200 import LLM, SamplingParams

    folder, raw, tensors = model_folders["tiny_a"]
    llm = LLM(folder, dtype="float32", page_size=4, max_num_pages=64)
    prompt = H.request_tokens(raw["vocab_size"], 9, seed=1)

    def gen(**kw):
        opts = dict(temperature=0.8, max_output_tokens=12, ignore_eos=True)
        opts.update(kw)
        return llm.generate(prompt, SamplingParams(**opts), request_ids=None).token_ids

    a, b, c = gen(seed=5), gen(seed=5), gen(seed=6)
    assert a == b and a != c                               # the seed decides the draw
    r1 = llm.generate(prompt, SamplingParams(temperature=0.8, max_output_tokens=6,
                                             ignore_eos=True), request_ids=None)
    assert len(r1.token_ids) == 6
    # top_k=1 is greedy whatever the temperature
    greedy = gen(temperature=0.0)
    assert gen(top_k=1, seed=9) == greedy
    # every sampled token lies in the top-k set of the plain distribution
    toks = gen(top_k=3, top_p=0.9, seed=11)
    ids = list(prompt)
    for tok in toks:
        p = P.plain_sampling_distribution(P.plain_logits(tensors, raw, ids)[-1], 0.8, top_k=3,
                                          top_p=0.9)
        assert p[tok] > 0
        ids.append(tok)
    # a strong repetition penalty forbids repeating a generated token under greedy decoding
    rep = gen(temperature=0.0, repetition_penalty=50.0, max_output_tokens=20)
    assert len(set(rep)) == len(rep)


def test_stop_token_ends_a_request(model_folders, tmp_path):
    from mstar_b200 import LLM, SamplingParams
    from mstar_b200.config.registry import config_from_dict
    from mstar_b200.weights.random_init import write_model_folder

    folder, raw, tensors = model_folders["tiny_a"]
    prompt = H.request_tokens(raw["vocab_size"], 9, seed=1)
    greedy = P.plain_greedy(tensors, raw, prompt, 6)
    raw2 = {**raw, "eos_token_id": greedy[3]}
    write_model_folder(tmp_path, config_from_dict(raw2), 0, tensors=tensors)
    llm = LLM(tmp_path, dtype="float32", page_size=4, max_num_pages=32)
    res = llm.generate(prompt, SamplingParams(temperature=0.0, max_output_tokens=6))
    first = greedy.index(greedy[3])
    assert res.token_ids == greedy[:first + 1] and res.finish_reason == "stop"
    res = llm.generate(prompt, SamplingParams(temperature=0.0, max_output_tokens=6,
                                              ignore_eos=True))
    assert res.token_ids == greedy and res.finish_reason == "length"


def test_command_line(model_folders):
    folder, raw, tensors = model_folders["tiny_a"]
    prompt = H.request_tokens(raw["vocab_size"], 9, seed=1)
    cmd = [sys.executable, str(H.ROOT / "bin" / "mstar"), "generate", str(folder), "--dtype",
           "float32", "--prompt-ids", ",".join(map(str, prompt)), "--temperature", "0",
           "--max-output-tokens", "5", "--ignore-eos", "--max-num-pages", "32", "--log-stats"]
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stderr
    record = json.loads(out.stdout.strip().splitlines()[-1])
    assert record["token_ids"] == P.plain_greedy(tensors, raw, prompt, 5)
    assert "generated_tokens=5" in out.stderr


@pytest.mark.parametrize("graphs", [True, False])
def test_tokens_taken_from_the_device_give_the_same_logits(model_folders, graphs):
    """A step may bring tokens that only the device holds (what the step before sampled):
    decode-only batches (a graph replay) and batches mixed with a prompt portion give the
    logits they give with the same tokens passed from the host."""
    from mstar_b200.engine.model import load_model
    from mstar_b200.engine.step import StepEntry, make_stepper

    folder, raw, _ = model_folders["tiny_a"]
    model = load_model(folder, dtype="float32")
    vocab = raw["vocab_size"]
    prompts = [H.request_tokens(vocab, n, seed=500 + n) for n in (6, 11, 3)]
    late = H.request_tokens(vocab, 9, seed=77)
    nxt = [5, 17, 3]

    def run(from_device: bool):
        st = make_stepper(model, page_size=4, num_pages=64, cuda_graphs=graphs)
        for i in range(3):
            st.add_request(i)
        st.add_request("late")
        st.step([StepEntry(i, prompts[i], ()) for i in range(3)])
        on_device = torch.tensor([nxt[2], 999 % vocab, nxt[0], nxt[1]], dtype=torch.int32,
                                 device="cuda:0")          # in another order, with a stranger
        where = {0: 2, 1: 3, 2: 0}
        outs = []
        for mixed in (False, True):
            entries = [StepEntry(i, [0 if from_device else nxt[i]], (0,)) for i in range(3)]
            if mixed:
                entries.insert(1, StepEntry("late", late, (len(late) - 1,)))
            pending = None
            if from_device:
                pending = {k: where[e.request] for k, e in enumerate(entries)
                           if e.request != "late"}
            outs.append(st.step(entries, pending, on_device if from_device else None).clone())
        return outs

    for a, b in zip(run(False), run(True)):
        assert torch.equal(a, b)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_stop_and_length_through_the_pipelined_entry_point(model_folders, tmp_path, dtype):
    """Steps are launched before the tokens of the step before are read: a request that
    stops is cut at its stop token although one more token was computed for it, and the
    other requests of the batch are not disturbed."""
    from mstar_b200 import LLM, SamplingParams

    folder, raw, tensors = model_folders["tiny_a"]
    prompts = [H.request_tokens(raw["vocab_size"], n, seed=600 + n) for n in (4, 9, 13, 6)]
    free = SamplingParams(temperature=0.0, max_output_tokens=12, ignore_eos=True)
    ref = LLM(folder, dtype=dtype, page_size=4, max_num_pages=64).generate(prompts, free)
    for prompt, r in zip(prompts, ref):
        check_greedy_chain(prompt, r.token_ids, tensors, raw, dtype)
    # declare the 5th token of request 1 a stop token: config.json's eos_token_id
    stop = ref[1].token_ids[4]
    from mstar_b200.config.registry import config_from_dict
    from mstar_b200.weights.random_init import write_model_folder

    alt = tmp_path / "with_stop"
    write_model_folder(alt, config_from_dict({**raw, "eos_token_id": int(stop)}), 0, tensors=tensors)
    llm = LLM(alt, dtype=dtype, page_size=4, max_num_pages=64)
    got = llm.generate(prompts, SamplingParams(temperature=0.0, max_output_tokens=12))
    for r, g in zip(ref, got):
        cut = r.token_ids.index(stop) + 1 if stop in r.token_ids else len(r.token_ids)
        assert g.token_ids == r.token_ids[:cut]
        assert g.finish_reason == ("stop" if stop in r.token_ids else "length")
    assert llm.pipelined_steps > 0
    assert llm.stepper.manager.num_requests() == 0 and llm.stepper.manager.check() == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_abort_through_the_entry_point(model_folders, dtype):
    from mstar_b200 import LLM, SamplingParams

    folder, raw, tensors = model_folders["tiny_a"]
    prompts = [H.request_tokens(raw["vocab_size"], n, seed=700 + n) for n in (5, 8, 11)]
    params = SamplingParams(temperature=0.0, max_output_tokens=10, ignore_eos=True)
    ref = LLM(folder, dtype=dtype, page_size=4, max_num_pages=64).generate(prompts, params)
    for prompt, r in zip(prompts, ref):
        check_greedy_chain(prompt, r.token_ids, tensors, raw, dtype)
    llm = LLM(folder, dtype=dtype, page_size=4, max_num_pages=64)
    ids = [llm.add_request(p, params) for p in prompts]
    done = {}
    for _ in range(4):                                  # a few steps, one always under way
        for r in llm.step():
            done[r.request_id] = r
    assert llm.abort(ids[1]) and not llm.abort("nobody")
    while llm.has_unfinished():
        for r in llm.step():
            done[r.request_id] = r
    assert done[ids[1]].finish_reason == "abort" and None not in done[ids[1]].output
    assert done[ids[1]].output == ref[1].token_ids[:len(done[ids[1]].output)]
    for k in (0, 2):                                    # the others are not disturbed
        assert done[ids[k]].output == ref[k].token_ids and done[ids[k]].finish_reason == "length"
    assert llm.stepper.manager.num_requests() == 0 and llm.stepper.manager.check() == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_temperature_beside_greedy_with_portions_of_16(model_folders, dtype):
    """Four requests with prompts of 1, 7, 33 and 40 tokens, two greedy and two at
    temperature 0.8, prompts cut into portions of 16 at most, pages of 8: the greedy ones
    follow the plain model; every token drawn at a temperature is the inverse-CDF draw of the
    plain distribution for that request's seed and step (within what the dtype's logit
    error moves the CDF's steps)."""
    from mstar_b200 import LLM, SamplingParams

    folder, raw, tensors = model_folders["tiny_b"]
    lengths = [1, 7, 33, 40]
    prompts = [H.request_tokens(raw["vocab_size"], n, seed=900 + n) for n in lengths]
    n_new = 10
    params = [SamplingParams(temperature=0.0, max_output_tokens=n_new, ignore_eos=True),
              SamplingParams(temperature=0.8, max_output_tokens=n_new, ignore_eos=True, seed=41),
              SamplingParams(temperature=0.0, max_output_tokens=n_new, ignore_eos=True),
              SamplingParams(temperature=0.8, max_output_tokens=n_new, ignore_eos=True, seed=42)]
    llm = LLM(folder, dtype=dtype, page_size=8, max_num_pages=64, max_num_batched_tokens=16)
    results = llm.generate(prompts, params)
    assert llm.stats.steps > n_new + 2                  # the prompts did not fit one step
    # how far a logit error of the dtype's tolerance can move a cumulative probability:
    # d(softmax)/d(logit) <= 1/4 per unit of logit/temperature, summed over a CDF at most 1
    slack = {"float32": 1e-4, "bfloat16": H.TOL["bfloat16"] / 0.8}[dtype]
    for prompt, sp, res in zip(prompts, params, results):
        assert res.finish_reason == "length" and len(res.token_ids) == n_new
        if sp.temperature == 0:
            check_greedy_chain(prompt, res.token_ids, tensors, raw, dtype)
            continue
        ids = list(prompt)
        for step, tok in enumerate(res.token_ids):
            p = P.plain_sampling_distribution(P.plain_logits(tensors, raw, ids)[-1], 0.8)
            cdf = torch.cumsum(p, 0)
            u = P.plain_uniform(sp.seed, step)
            lo = cdf[tok - 1].item() if tok else 0.0
            assert lo - slack <= u <= cdf[tok].item() + slack, (lengths, step, tok, u)
            ids.append(tok)
    assert llm.stepper.manager.num_requests() == 0 and llm.stepper.manager.check() == 0


def test_a_wait_that_ran_out_stops_the_entry_point(model_folders):
    """Kernels with bounded waits report into a device word and return with partial
    output; the entry point reads that word with every step's tokens and raises instead
    of handing tokens out.  The word is set by hand here: no kernel is made to hang."""
    from mstar_b200 import LLM, SamplingParams, ops

    folder, raw, _ = model_folders["tiny_a"]
    llm = LLM(folder, dtype="bfloat16", page_size=4, max_num_pages=32)
    llm.add_request(H.request_tokens(raw["vocab_size"], 6, seed=1),
                    SamplingParams(temperature=0.0, max_output_tokens=8, ignore_eos=True))
    llm.step()
    llm.step()
    ops.tcgen05_error_word(llm.device).fill_(4)
    with pytest.raises(ops.KernelError, match="code 4"):
        for _ in range(3):
            llm.step()
    assert int(ops.tcgen05_error_word(llm.device).item()) == 0     # cleared for what follows
    with pytest.raises(ops.KernelError):
        ops.tcgen05_error_word(llm.device).fill_(13)
        ops.check_error_word(llm.device)
    ops.check_error_word(llm.device)                               # zero again: silent
