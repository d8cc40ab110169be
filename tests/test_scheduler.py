"""The scheduler's decisions, with a scripted stand-in for the model (no GPU).

The stand-in produces the next token as a function of all tokens so far, as a real model
does, so a request that is preempted and recomputed must produce the same output
(the reference tests its generation loop the same way with a FakeRunner,
tests/runtime/scheduler_test.cpp:108-333)."""
import random

import pytest
import torch

from poor_mans_mamba_b200.cache import CacheManager
from poor_mans_mamba_b200.engine.scheduler import SamplingParams, Scheduler
from poor_mans_mamba_b200.parts.base import StateSpec

SPECS = {0: [("a.kv", StateSpec.paged("kv", 2, 4)), ("m.s", StateSpec.fixed("s", (2,), "float32"))]}


def make(num_pages=8, num_slots=4, page_size=4, budget=16, max_seqs=4):
    cache = CacheManager(SPECS, page_size=page_size, num_pages=num_pages, num_slots=num_slots,
                         dtype=torch.float32, device="cpu")
    return cache, Scheduler(cache, max_batched_tokens=budget, max_seqs=max_seqs)


def next_token(tokens):
    return (sum(tokens) * 31 + len(tokens) * 7) % 97 + 3


def run(sched, cache, max_steps=10000, log=None):
    """Drive the scheduler like the engine does, checking the plan against the cache."""
    steps = 0
    while sched.has_work():
        plan = sched.plan()
        sampled = []
        for e in plan.entries:
            assert e.count >= 1 and e.start == e.req.n_computed
            cache.grow(e.req.id, e.start + e.count)  # must fit: the plan promised it
            cache.advance(e.req.id, e.count)
            if e.samples:
                assert e.start + e.count == len(e.req.tokens)
                sampled.append(next_token(e.req.tokens))
        assert plan.n_tokens <= sched.max_batched_tokens
        if log is not None:
            log.append(plan)
        sched.complete(plan, sampled)
        cache.check()
        steps += 1
        assert steps < max_steps
    return steps


def expected(prompt, n, eos=-1):
    seq, out = list(prompt), []
    for _ in range(n):
        t = next_token(seq)
        out.append(t)
        seq.append(t)
        if t == eos:
            break
    return out


def test_prompt_is_cut_to_the_budget_then_decoded():
    cache, s = make(num_pages=16, budget=5)
    r = s.add("a", list(range(1, 13)), SamplingParams(max_new_tokens=3))
    log = []
    run(s, cache, log=log)
    assert [p.entries[0].count for p in log] == [5, 5, 2, 1, 1]
    assert [p.entries[0].samples for p in log] == [False, False, True, True, True]
    assert r.output == expected(r.prompt, 3) and r.status == "done"
    assert cache.min_free_pages() == 16 and cache.free_slots == 4
    assert s.counters["prefill_tokens"] == 12 and s.counters["decode_tokens"] == 2


def test_decodes_go_first_and_prompts_share_the_rest():
    cache, s = make(num_pages=32, budget=8)
    a = s.add("a", [1, 2, 3], SamplingParams(max_new_tokens=4))
    log = []
    plan = s.plan()
    cache.grow("a", 3), cache.advance("a", 3)
    s.complete(plan, [next_token(a.tokens)])
    b = s.add("b", list(range(1, 21)), SamplingParams(max_new_tokens=2))
    plan = s.plan()
    assert [(e.req.id, e.count) for e in plan.entries] == [("a", 1), ("b", 7)]  # 1 + 7 = budget


def test_fifo_admission_and_sequence_cap():
    cache, s = make(num_pages=32, budget=64, max_seqs=2)
    for i in range(4):
        s.add(i, [5 + i, 6, 7], SamplingParams(max_new_tokens=2))
    plan = s.plan()
    assert [e.req.id for e in plan.entries] == [0, 1] and [r.id for r in s.waiting] == [2, 3]
    run(s, cache)
    assert all(s.requests[i].output == expected(s.requests[i].prompt, 2) for i in range(4))


def test_eos_is_kept_and_ends_the_request():
    cache, s = make(num_pages=16)
    prompt = [4, 9]
    eos = expected(prompt, 3)[2]
    r = s.add("a", prompt, SamplingParams(max_new_tokens=10, eos_id=eos))
    run(s, cache)
    assert r.output == expected(prompt, 10, eos) and r.output[-1] == eos and len(r.output) <= 3 and r.status == "done"


def test_preemption_when_pages_run_out_gives_the_same_tokens():
    prompts = [[3, 1, 4, 1, 5], [9, 2, 6], [5, 3, 5, 8, 9, 7]]
    n_new = 14
    cache, s = make(num_pages=64)
    for i, p in enumerate(prompts):
        s.add(i, p, SamplingParams(max_new_tokens=n_new))
    run(s, cache)
    calm = [s.requests[i].output for i in range(3)]
    assert s.counters["preemptions"] == 0 and calm == [expected(p, n_new) for p in prompts]

    cache, s = make(num_pages=9)  # 36 tokens of cache for 3 requests that grow to 19, 17 and 20
    for i, p in enumerate(prompts):
        s.add(i, p, SamplingParams(max_new_tokens=n_new))
    log = []
    run(s, cache, log=log)
    assert s.counters["preemptions"] > 0
    assert [s.requests[i].output for i in range(3)] == calm
    assert all(r.status == "done" for r in s.requests.values())
    first = next(p for p in log if p.preempted)
    assert first.preempted[0] == 2  # the most recently admitted request gives way
    assert cache.min_free_pages() == 9 and cache.free_slots == 4


def test_request_that_can_never_fit_fails_at_once_and_others_go_on():
    cache, s = make(num_pages=4)  # 16 tokens
    big = s.add("big", list(range(1, 30)), SamplingParams(max_new_tokens=2))
    ok = s.add("ok", [1, 2, 3], SamplingParams(max_new_tokens=2))
    run(s, cache)
    assert big.status == "oom" and big.output == [] and s.counters["rejects"] == 1
    assert ok.status == "done" and ok.output == expected(ok.prompt, 2)


def test_lone_request_that_outgrows_the_pool_ends_with_what_it_has():
    cache, s = make(num_pages=3)  # 12 tokens
    r = s.add("a", [1, 2, 3, 4, 5], SamplingParams(max_new_tokens=50))
    run(s, cache)
    assert r.status == "cache_full" and r.output == expected(r.prompt, 50)[:len(r.output)]
    assert len(r.prompt) + len(r.output) == 13  # 12 tokens cached + the one just sampled
    assert cache.min_free_pages() == 3 and s.counters["cache_full"] == 1


def test_bad_submissions():
    cache, s = make()
    with pytest.raises(ValueError):
        s.add("a", [], SamplingParams())
    with pytest.raises(ValueError):
        s.add("a", [1], SamplingParams(max_new_tokens=0))
    s.add("a", [1], SamplingParams())
    with pytest.raises(ValueError):
        s.add("a", [1], SamplingParams())


@pytest.mark.parametrize("seed", range(5))
def test_random_traffic(seed):
    rng = random.Random(seed)
    cache, s = make(num_pages=rng.choice([6, 10, 20]), num_slots=3, budget=rng.choice([4, 9, 32]), max_seqs=3)
    want = {}
    for i in range(12):
        p = [rng.randrange(1, 90) for _ in range(rng.choice([1, 2, 5, 11, 17]))]
        n = rng.choice([1, 3, 8])
        s.add(i, p, SamplingParams(max_new_tokens=n))
        want[i] = expected(p, n)
    run(s, cache)
    for i, r in s.requests.items():
        if r.status == "done":
            assert r.output == want[i]
        else:
            assert r.status in ("oom", "cache_full") and r.output == want[i][:len(r.output)]
    assert cache.free_slots == 3 and cache.min_free_pages() == cache.groups[(2, 4, 0)].num_pages


def run_one_step_ahead(sched, cache, max_steps=10000):
    """Drives the scheduler the way the engine's decode path does: a decode-only step whose
    requests equal the previous step's is 'launched' (its tokens computed from what the device
    knows) before the previous step's ids are handed to the scheduler."""
    truth = {}      # request id -> every token the device has seen or produced (never PENDING)
    inflight = None  # (ids, slots, sampled)
    steps = 0

    def settle():
        nonlocal inflight
        if inflight is not None:
            _, slots, sampled = inflight
            inflight = None
            sched.resolve(slots, sampled)

    while sched.has_work() or inflight is not None:
        plan = sched.plan()
        if not plan.entries:
            settle()
            plan = sched.plan()
            if not plan.entries:
                continue
        pure = all(e.count == 1 and e.samples for e in plan.entries)
        ids = [e.req.id for e in plan.entries]
        ahead = pure and inflight is not None and inflight[0] == ids
        if inflight is not None and not ahead:
            settle()
            plan.entries = [e for e in plan.entries if not e.req.finished]
            if not plan.entries:
                continue
        sampled = []
        for e in plan.entries:
            r = e.req
            cache.grow(r.id, e.start + e.count)
            cache.advance(r.id, e.count)
            if not ahead:  # the host feeds these tokens: none of them may be a placeholder
                fed = r.tokens[e.start:e.start + e.count]
                assert Scheduler.PENDING not in fed
                truth[r.id] = r.tokens[:e.start + e.count]
            if e.samples:
                tok = next_token(truth[r.id])
                truth[r.id] = truth[r.id] + [tok]
                sampled.append(tok)
        if pure:
            slots = sched.advance(plan)
            if ahead:
                settle()
            inflight = ([e.req.id for e in plan.entries], slots, sampled)
        else:
            sched.complete(plan, sampled)
        cache.check()
        steps += 1
        assert steps < max_steps
    return steps


@pytest.mark.parametrize("seed", range(8))
def test_one_step_ahead_gives_the_same_outputs(seed):
    """Stop tokens seen one step late, requests ending by length, preemption and admission while
    a step is in flight: outputs equal the step-by-step ones, nothing stays held."""
    rng = random.Random(100 + seed)
    cache, s = make(num_pages=rng.choice([6, 10, 20]), num_slots=3, budget=rng.choice([4, 9, 32]), max_seqs=3)
    want = {}
    for i in range(12):
        p = [rng.randrange(1, 90) for _ in range(rng.choice([1, 2, 5, 11, 17]))]
        n = rng.choice([1, 3, 8, 14])
        free_run = expected(p, n)
        eos = rng.choice([-1, -1, free_run[len(free_run) // 2], free_run[-1]])  # in the middle, at the end, never
        s.add(i, p, SamplingParams(max_new_tokens=n, eos_id=eos))
        want[i] = expected(p, n, eos)
    run_one_step_ahead(s, cache)
    for i, r in s.requests.items():
        assert Scheduler.PENDING not in r.output
        if r.status == "done":
            assert r.output == want[i], (i, r.output, want[i])
        else:
            assert r.status in ("oom", "cache_full") and r.output == want[i][:len(r.output)]
    assert cache.free_slots == 3 and cache.min_free_pages() == cache.groups[(2, 4, 0)].num_pages
    assert not s.running and not s.waiting


def test_request_ends_with_partial_output_when_it_reaches_max_seq_len():
    """Reference: KV overflow on decode ends the session as done with what it has
    (src/runtime/cluster_scheduler.cpp:645-651)."""
    cache = CacheManager(SPECS, page_size=4, num_pages=16, num_slots=4, dtype=torch.float32, device="cpu")
    s = Scheduler(cache, max_batched_tokens=16, max_seqs=4, max_seq_len=10)
    a = s.add("a", list(range(1, 8)), SamplingParams(max_new_tokens=50))      # 7 + 3 fed tokens fill 10 places
    b = s.add("b", [5, 6], SamplingParams(max_new_tokens=4))                   # ends by length first
    c = s.add("c", list(range(1, 12)), SamplingParams(max_new_tokens=4))       # prompt alone is too long
    run(s, cache)
    # positions 0..9 are computed; the token sampled at position 9 is still handed out
    assert a.status == "max_seq" and a.output == expected(a.prompt, 4) and a.n_computed == 10
    assert b.status == "done" and b.output == expected(b.prompt, 4)
    assert c.status == "max_seq" and c.output == []
    assert cache.min_free_pages() == 16 and cache.free_slots == 4


def test_max_seq_len_with_late_results():
    """The two-halves digestion (advance / resolve) ends a request at max_seq_len too."""
    cache = CacheManager(SPECS, page_size=4, num_pages=16, num_slots=4, dtype=torch.float32, device="cpu")
    s = Scheduler(cache, max_batched_tokens=16, max_seqs=4, max_seq_len=6)
    a = s.add("a", [1, 2, 3, 4], SamplingParams(max_new_tokens=50))
    pending = None
    while s.has_work():
        plan = s.plan()
        toks = []
        for e in plan.entries:
            cache.grow(e.req.id, e.start + e.count), cache.advance(e.req.id, e.count)
            known = [t for t in e.req.tokens if t != Scheduler.PENDING]
            toks.append(next_token(known + ([pending[1][0]] if pending else [])))
        slots = s.advance(plan)
        if pending is not None:
            s.resolve(*pending)
        pending = (slots, toks)
    s.resolve(*pending)
    assert a.status == "max_seq" and a.output == expected(a.prompt, 3) and a.n_computed == 6


def test_requests_are_given_back_through_the_release_callback():
    cache = CacheManager(SPECS, page_size=4, num_pages=3, num_slots=4, dtype=torch.float32, device="cpu")
    released = []

    def release(rid):
        released.append(rid)
        cache.release(rid)

    s = Scheduler(cache, max_batched_tokens=16, max_seqs=4, release=release)
    s.add("a", [1, 2, 3, 4, 5], SamplingParams(max_new_tokens=6))
    s.add("b", [1, 2, 3], SamplingParams(max_new_tokens=6))
    run(s, cache)
    assert s.counters["preemptions"] >= 1           # 3 pages cannot hold both to the end
    assert sorted(set(released)) == ["a", "b"] and len(released) == 2 + s.counters["preemptions"]
    assert cache.min_free_pages() == 3
