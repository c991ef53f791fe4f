"""The scheduler's decisions (CPU): admission, portions under a token budget, decode
first, finishing, and pre-emption by recomputation when pages run out."""
import pytest

from mstar_b200.cache import CacheManager, GroupConfig
from mstar_b200.engine.scheduler import Request, Scheduler, SchedulerConfig
from mstar_b200.sampling import SamplingParams


def make(pages=100, page=4, slots=8, budget=16, cap=None, batch=64, stops=(99,)):
    cm = CacheManager([GroupConfig(page, pages)], num_slots=slots)
    sch = Scheduler(SchedulerConfig(max_num_batched_tokens=budget, max_concurrent_requests=cap,
                                    max_batch_size=batch), cm, stops)
    return cm, sch


def req(rid, n, max_out=4, **kw):
    return Request(rid, list(range(1, n + 1)), SamplingParams(temperature=0.0,
                                                              max_output_tokens=max_out, **kw))


def run_step(cm, sch, token=7):
    """What the engine does around one plan: reserve + commit, then report tokens."""
    plan = sch.schedule()
    ids = [e.request.request_id for e in plan.entries]
    counts = [len(e.tokens) for e in plan.entries]
    cm.reserve(ids, counts)
    for i, c in zip(ids, counts):
        cm.commit(i, c)
    sampled = {e.request.request_id: (token(e.request) if callable(token) else token)
               for e in plan.entries if e.samples}
    done = sch.update(plan, sampled)
    assert cm.check() == 0
    return plan, done


def test_prompt_is_cut_into_portions_under_the_budget():
    cm, sch = make(budget=16)
    sch.add(req("a", 40))
    sizes = []
    for _ in range(3):
        plan, _ = run_step(cm, sch)
        sizes.append([len(e.tokens) for e in plan.entries])
        assert plan.num_tokens() <= 16
    assert sizes == [[16], [16], [8]]
    assert plan.entries[0].samples                     # the last portion samples
    assert plan.entries[0].tokens == list(range(33, 41))
    plan, _ = run_step(cm, sch)
    assert [len(e.tokens) for e in plan.entries] == [1] and plan.entries[0].tokens == [7]


def test_decoding_goes_first_and_prompts_fill_the_rest():
    cm, sch = make(budget=16)
    sch.add(req("a", 5, max_out=10))
    run_step(cm, sch)                                  # a: whole prompt, now decoding
    sch.add(req("b", 40))
    plan, _ = run_step(cm, sch)
    assert [(e.request.request_id, len(e.tokens)) for e in plan.entries] == [("a", 1), ("b", 15)]
    plan, _ = run_step(cm, sch)
    assert [(e.request.request_id, len(e.tokens)) for e in plan.entries] == [("a", 1), ("b", 15)]
    assert not plan.entries[1].samples


def test_admission_cap_and_first_come_order():
    cm, sch = make(budget=64, cap=2)
    for rid in "abc":
        sch.add(req(rid, 3, max_out=2))
    plan, _ = run_step(cm, sch)
    assert [r.request_id for r in plan.admitted] == ["a", "b"]
    plan, done = run_step(cm, sch)                     # a and b reach max_output_tokens
    assert {r.request_id for r in done} == {"a", "b"} and all(r.finish_reason == "length"
                                                             for r in done)
    plan, _ = run_step(cm, sch)
    assert [r.request_id for r in plan.admitted] == ["c"]
    assert cm.num_requests() == 1


def test_slots_limit_admission():
    cm, sch = make(slots=1, budget=64)
    sch.add(req("a", 3))
    sch.add(req("b", 3))
    plan, _ = run_step(cm, sch)
    assert [r.request_id for r in plan.admitted] == ["a"] and len(sch.waiting) == 1


def test_finishing_on_stop_token_and_ignore_eos():
    cm, sch = make()
    sch.add(req("a", 3, max_out=10))
    sch.add(req("b", 3, max_out=3, ignore_eos=True))
    plan, done = run_step(cm, sch, token=99)
    assert [(r.request_id, r.finish_reason, r.output) for r in done] == [("a", "stop", [99])]
    _, done = run_step(cm, sch, token=99)
    assert done == []
    _, done = run_step(cm, sch, token=99)
    assert [(r.request_id, r.finish_reason, r.output) for r in done] == [
        ("b", "length", [99, 99, 99])]
    assert not sch.has_work() and cm.num_requests() == 0 and cm.free_pages() == 100


def test_pages_run_out_the_newest_request_is_recomputed():
    cm, sch = make(pages=6, page=4, budget=64)         # 24 tokens in all
    sch.add(req("old", 8, max_out=12))
    sch.add(req("new", 8, max_out=12))
    plan, _ = run_step(cm, sch)                        # both prompts: 2 + 2 pages
    assert len(plan.entries) == 2 and cm.free_pages() == 2
    seen_preemption = None
    for step in range(12):
        plan, _ = run_step(cm, sch, token=lambda r: 50 + len(r.output))
        if plan.preempted:
            seen_preemption = step
            break
    assert seen_preemption is not None
    victim = plan.preempted[0]
    assert victim.request_id == "new" and victim.status == "waiting" and victim.num_computed == 0
    assert sch.waiting[0] is victim and not cm.has("new")
    assert [e.request.request_id for e in plan.entries] == ["old"]   # the older one went on
    kept = list(victim.output)
    # "new" comes back only when its prompt and what it generated fit again (here: when
    # "old" has ended), and recomputes all of it in one portion
    entry = None
    while entry is None:
        old_running = any(r.request_id == "old" for r in sch.running)
        plan, _ = run_step(cm, sch, token=lambda r: 50 + len(r.output))
        hits = [e for e in plan.entries if e.request.request_id == "new"]
        entry = hits[0] if hits else None
    assert not old_running
    assert entry.tokens == victim.prompt + kept and entry.samples
    assert victim.preemptions == 1
    while sch.has_work():
        run_step(cm, sch, token=lambda r: 50 + len(r.output))
    assert [len(r.output) for r in sch.finished] == [12, 12] and cm.free_pages() == 6


def test_prompts_never_take_the_pages_decoding_needs():
    cm, sch = make(pages=4, page=4, budget=64)
    sch.add(req("a", 7, max_out=8))
    run_step(cm, sch)                                  # a holds 2 pages, 7 tokens
    sch.add(req("b", 12))                              # would need 3 pages, 2 are free
    plan, _ = run_step(cm, sch)
    # a decodes (its 8th token fits its second page); b gets what is left: 2 pages = 8 tokens
    assert [(e.request.request_id, len(e.tokens)) for e in plan.entries] == [("a", 1), ("b", 8)]


def test_a_request_larger_than_the_pool_is_finished_not_starved():
    cm, sch = make(pages=3, page=4, budget=64)
    sch.add(req("huge", 30))
    sch.add(req("ok", 4, max_out=1))
    plan, done = run_step(cm, sch)
    assert [(r.request_id, r.finish_reason) for r in plan.finished] == [("huge", "cache_exhausted")]
    assert [r.request_id for r in done] == ["ok"]
    # one that fits at first but outgrows the pool while decoding alone
    sch.add(req("grow", 10, max_out=50))
    reasons = []
    for _ in range(10):
        plan, done = run_step(cm, sch)
        reasons += [r.finish_reason for r in plan.finished + done]
        if not sch.has_work():
            break
    assert reasons == ["cache_exhausted"] and cm.free_pages() == 3 and cm.check() == 0


def test_two_prompts_that_block_each_other():
    cm, sch = make(pages=4, page=4, budget=6)          # each prompt needs 3 pages
    sch.add(req("a", 12, max_out=1))
    sch.add(req("b", 12, max_out=1))
    finished = []
    for _ in range(20):
        plan, done = run_step(cm, sch)
        finished += [r.request_id for r in done]
        if not sch.has_work():
            break
    assert finished == ["a", "b"]                      # both complete, the older first


def test_abort():
    cm, sch = make()
    sch.add(req("a", 3))
    sch.add(req("b", 3))
    run_step(cm, sch)
    sch.add(req("c", 3))
    assert sch.abort("c") and sch.abort("a") and not sch.abort("zzz")
    assert [r.request_id for r in sch.running] == ["b"] and cm.num_requests() == 1
    assert {r.request_id: r.finish_reason for r in sch.finished} == {"c": "abort", "a": "abort"}


def test_batch_size_cap():
    cm, sch = make(budget=64, batch=2)
    for rid in "abc":
        sch.add(req(rid, 2, max_out=5))
    plan, _ = run_step(cm, sch)
    assert len(plan.entries) == 2
    plan, _ = run_step(cm, sch)
    assert len(plan.entries) == 2


def test_may_admit_tells_whether_a_waiting_request_could_enter():
    """The engine launches the next decode step ahead only while no waiting request could
    be admitted: behind a full cap, a full batch or no free slot."""
    cm, sch = make(cap=2, slots=8, budget=64)
    assert not sch.may_admit()                        # nobody waits
    for i in range(3):
        sch.add(req(f"r{i}", 4, max_out=3))
    assert sch.may_admit()
    run_step(cm, sch)                                 # r0 and r1 enter, r2 waits behind the cap
    assert [r.request_id for r in sch.running] == ["r0", "r1"] and len(sch.waiting) == 1
    assert not sch.may_admit()
    while len(sch.running) == 2:
        run_step(cm, sch)
    assert sch.may_admit()                            # one finished: r2 can enter now
    cm2, sch2 = make(slots=1, budget=64)
    sch2.add(req("a", 4)), sch2.add(req("b", 4))
    run_step(cm2, sch2)
    assert not sch2.may_admit()                       # the only state slot is taken
    cm3, sch3 = make(batch=1, budget=64)
    sch3.add(req("a", 4)), sch3.add(req("b", 4))
    run_step(cm3, sch3)
    assert not sch3.may_admit()                       # the batch is full


def test_scheduling_cost_does_not_grow_with_the_square_of_the_batch():
    """One cache-manager query per request and decision: a step with 64 decoding requests
    asks for page needs about 64 times, not 64 * 64."""
    cm, sch = make(pages=4000, slots=80, budget=4096, batch=64)
    for i in range(64):
        sch.add(req(f"r{i}", 8, max_out=50))
    run_step(cm, sch)
    calls = []
    orig = cm.pages_needed
    cm.pages_needed = lambda ids, counts: (calls.append(len(ids)), orig(ids, counts))[1]
    plan, _ = run_step(cm, sch)
    assert len(plan.entries) == 64
    assert len(calls) <= 70 and max(calls) == 1


def launch_then_read(cm, sch, pending, token):
    """One engine step the pipelined way: plan and launch the next batch (``advance``),
    then read the batch before (``resolve``).  ``pending``: the plan in flight or None.
    Returns (the new plan in flight, requests reported as finished by the resolve)."""
    plan = sch.schedule()
    ids = [e.request.request_id for e in plan.entries]
    counts = [len(e.tokens) for e in plan.entries]
    cm.reserve(ids, counts)
    for i, c in zip(ids, counts):
        cm.commit(i, c)
    sch.advance(plan)
    done = []
    if pending is not None:
        sampled = {e.request.request_id: token(e.request) for e in pending.entries if e.samples}
        done = sch.resolve(pending, sampled)
    assert cm.check() == 0
    return plan, done


def test_advance_then_resolve_a_stop_takes_effect_one_step_late():
    """The next step is planned before the last one's tokens are known: places (None) stand
    for them; a request that stopped has one token computed in vain, which is dropped."""
    cm, sch = make(budget=64)
    sch.add(req("a", 4, max_out=10))
    sch.add(req("b", 4, max_out=10))
    count = {"a": 0, "b": 0}

    def token(r):                       # a stops with its second token, b never
        count[r.request_id] += 1
        return 99 if (r.request_id == "a" and count["a"] == 2) else 7

    p0, _ = launch_then_read(cm, sch, None, token)            # prompts; samples pending
    a, b = p0.entries[0].request, p0.entries[1].request
    assert a.output == [None] and b.output == [None]
    p1, done = launch_then_read(cm, sch, p0, token)           # decode 1 launched, p0 read
    assert p1.entries[0].tokens == [None] and a.output == [7, None] and not done
    p2, done = launch_then_read(cm, sch, p1, token)           # decode 2 launched, p1 read: a stopped
    assert [r.request_id for r in done] == ["a"] and a.finish_reason == "stop"
    assert a.output == [7, 99]                                # the place of decode 2 is gone
    assert a.status == "finished" and [r.request_id for r in sch.running] == ["b"]
    p3, done = launch_then_read(cm, sch, p2, token)           # a's token of decode 2 is ignored
    assert not done and a.output == [7, 99] and b.output == [7, 7, 7, None]
    assert all(e.request is b for e in p3.entries)


def test_advance_foresees_the_length_and_resolve_reports_it_complete():
    cm, sch = make(budget=64)
    sch.add(req("a", 4, max_out=2))
    p0, _ = launch_then_read(cm, sch, None, lambda r: 7)
    a = p0.entries[0].request
    p1, done = launch_then_read(cm, sch, p0, lambda r: 7)
    assert a.status == "finished" and a.finish_reason == "length"     # foreseen at the launch
    assert not done and a.output == [7, None]                         # ... but not complete
    p2, done = launch_then_read(cm, sch, p1, lambda r: 5)
    assert not p2.entries and [r.request_id for r in done] == ["a"] and a.output == [7, 5]
    # the last allowed token is a stop token: the reason says so
    sch.add(req("b", 4, max_out=1))
    p0, _ = launch_then_read(cm, sch, None, lambda r: 99)
    b = p0.entries[0].request
    assert b.finish_reason == "length"
    _, done = launch_then_read(cm, sch, p0, lambda r: 99)
    assert [r.request_id for r in done] == ["b"] and b.finish_reason == "stop" and b.output == [99]


def test_a_preempted_request_keeps_the_place_of_its_token_in_flight():
    cm, sch = make(pages=6, page=4, budget=64)
    sch.add(req("old", 7, max_out=20))
    sch.add(req("new", 7, max_out=20))
    inflight, _ = launch_then_read(cm, sch, None, lambda r: 7)
    victim = None
    for _ in range(12):
        plan = sch.schedule()
        if plan.preempted:
            victim = plan.preempted[0]
            assert victim.request_id == "new" and victim.output[-1] is None
            ids = [e.request.request_id for e in plan.entries]
            cm.reserve(ids, [1] * len(ids))
            for i in ids:
                cm.commit(i, 1)
            sch.advance(plan)
            sch.resolve(inflight, {e.request.request_id: 7 for e in inflight.entries if e.samples})
            break
        ids = [e.request.request_id for e in plan.entries]
        counts = [len(e.tokens) for e in plan.entries]
        cm.reserve(ids, counts)
        for i, c in zip(ids, counts):
            cm.commit(i, c)
        sch.advance(plan)
        sch.resolve(inflight, {e.request.request_id: 7 for e in inflight.entries if e.samples})
        inflight = plan
    assert victim is not None and None not in victim.output     # the value arrived all the same
    assert victim.status == "waiting" and victim.num_computed == 0


def test_abort_while_a_step_is_under_way():
    cm, sch = make(budget=64)
    sch.add(req("a", 4, max_out=10))
    sch.add(req("b", 4, max_out=10))
    p0, _ = launch_then_read(cm, sch, None, lambda r: 7)
    p1, _ = launch_then_read(cm, sch, p0, lambda r: 7)        # decode 1 under way
    a = p1.entries[0].request
    assert sch.abort("a") and a.status == "finished" and a.finish_reason == "abort"
    assert cm.num_requests() == 1                             # its pages and slot are back
    p2, done = launch_then_read(cm, sch, p1, lambda r: 99 if r.request_id == "a" else 7)
    # a's token (a stop token, even) arrives and is dropped
    assert not done and a.finish_reason == "abort" and None not in a.output
    assert [e.request.request_id for e in p2.entries] == ["b"]
    assert not sch.abort("a") and not sch.abort("nobody")


def test_sequences_end_where_the_models_positions_end():
    """max_seq_len (the model's max_position_embeddings; the reference's max_seq_len,
    mstar/model/orpheus/orpheus_model.py:88-95): a prompt that fills it is refused, and
    generation finishes with "length" where the positions end, whatever max_output_tokens
    says."""
    cm = CacheManager([GroupConfig(4, 100)], num_slots=4)
    cm.set_max_positions(12)
    sch = Scheduler(SchedulerConfig(max_num_batched_tokens=64, max_seq_len=12), cm, (99,))
    with pytest.raises(ValueError, match="sequences of up to 12"):
        sch.add(req("long", 12))
    with pytest.raises(ValueError):
        sch.add(req("longer", 30))
    sch.add(req("a", 9, max_out=50))                   # 9 + 3 = 12: three tokens, no more
    sch.add(req("b", 3, max_out=2))                    # its own limit is the smaller one
    outputs = {}
    for _ in range(8):
        if not sch.has_work():
            break
        _, done = run_step(cm, sch)
        for r in done:
            outputs[r.request_id] = (len(r.output), r.finish_reason)
    assert outputs == {"a": (3, "length"), "b": (2, "length")}
    assert cm.num_requests() == 0 and cm.check() == 0


def test_the_manager_refuses_a_step_beyond_the_positions():
    from mstar_b200.cache import SequenceTooLong

    cm = CacheManager([GroupConfig(4, 100)], num_slots=2)
    cm.set_max_positions(10)
    cm.add_request("a")
    cm.add_request("b")
    cm.reserve(["a"], [10])                            # positions 0..9: allowed
    cm.commit("a", 10)
    free = cm.free_pages()
    with pytest.raises(SequenceTooLong, match="'a'"):
        cm.reserve(["b", "a"], [4, 1])                 # a would get position 10
    assert cm.free_pages() == free and cm.block_table("b") == [] and cm.check() == 0
    cm.set_max_positions(None)
    cm.reserve(["b", "a"], [4, 1])
