"""The scheduler's decisions, on the host, against a fake engine with the real
cache manager."""
import random

import numpy as np
import pytest

from fakes import FakeEngine, FakeSampler, fake_logits
from sglang_c_b200.engine.scheduler import Scheduler
from sglang_c_b200.sampling import SamplingParams, request_stream, uniform


def sched(**kw):
    opts = {k: kw.pop(k) for k in ("seed", "prefill_chunk", "token_budget") if k in kw}
    eng = FakeEngine(**kw)
    return Scheduler(eng, sampler=FakeSampler(), **opts), eng


def serial(prompt, max_new, vocab, sp=None, seed=0, rid=1, eos=None):
    """What a request generates when it runs alone."""
    sp = sp or SamplingParams()
    rng = request_stream(seed ^ sp.seed, rid)
    toks, out = list(prompt), []
    for _ in range(max_new):
        row = fake_logits(toks, vocab)
        if sp.temperature <= 0:
            u = 0.0
        else:
            rng, u = uniform(rng)
        t = FakeSampler().sample([row], [sp], [u])[0]
        if t == eos and eos is not None and not sp.ignore_eos:
            break
        if sp.is_stop(t):
            break
        out.append(t)
        toks.append(t)
    return out


def drain(s):
    out = {}
    while True:
        g = s.poll()
        if g is None:
            return out
        out[g[0]] = g[1]


def test_prompt_is_cut_under_the_budget_and_decode_goes_first():
    s, eng = sched(max_step_tokens=8, prefill_chunk=6, n_pages=32, max_positions=128)
    a = s.submit_ids(list(range(10)), max_new=3)
    s.step()
    assert eng.steps[-1] == [(a, 6, False)]                   # a portion of the chunk size, nothing wanted
    b = s.submit_ids(list(range(20)), max_new=2)
    s.step()
    assert eng.steps[-1] == [(a, 4, True), (b, 4, False)]     # budget 8: rest of a, then b fills it
    s.step()
    assert eng.steps[-1][0] == (a, 1, True)                   # a decodes first
    assert eng.steps[-1][1] == (b, 6, False)                  # b's portion is capped by the chunk
    s.run_until_done()
    got = drain(s)
    assert got[a] == serial(list(range(10)), 3, 50, rid=a)
    assert got[b] == serial(list(range(20)), 2, 50, rid=b)
    st = s.get_stats()
    assert st.prefill_tokens == 30 and st.decode_tokens == 5 and st.n_finished == 2
    assert st.pool_free == st.pool_pages and st.n_running == 0 and st.n_waiting == 0


def test_first_come_first_served_and_slots():
    s, eng = sched(max_requests=2, n_pages=32, max_step_tokens=64)
    ids = [s.submit_ids([1, 2, 3], max_new=4) for _ in range(4)]
    s.step()
    assert [e[0] for e in eng.steps[-1]] == ids[:2]           # two slots: the first two arrivals
    s.run_until_done()
    order = [r.id for r in s.done]
    assert order == ids


def test_requests_that_can_never_run_are_refused():
    s, eng = sched(n_pages=4, page_size=4, max_positions=64, vocab=50)
    assert s.submit_ids([], 4) == -1
    assert s.submit_ids([1, 99], 4) == -1                     # id outside the vocabulary
    assert s.submit_ids(list(range(10)), 10) == -1            # 20 tokens never fit 16 cache positions
    assert s.submit_ids([1] * 64, 1) == -1                    # prompt fills every position
    assert s.submit_ids(list(range(10)), 6) > 0
    s2, _ = sched(n_pages=8, page_size=4)
    r = s2.submit_ids([1, 2], 0)                              # max_new <= 0 means 16, as in the reference
    assert r > 0 and s2.requests[r].max_new == 16


def test_finishing_rules():
    vocab = 50
    # eos: not appended
    base = serial([5, 6, 7], 12, vocab)
    eos = base[4]
    first = base.index(eos)
    s, _ = sched(eos_token_id=eos)
    r = s.submit_ids([5, 6, 7], 12)
    s.run_until_done()
    assert drain(s)[r] == base[:first] and s.requests[r].finish_reason == "eos"
    # ignore_eos runs on
    s, _ = sched(eos_token_id=eos)
    r = s.submit_ids([5, 6, 7], 12, SamplingParams(ignore_eos=True))
    s.run_until_done()
    assert drain(s)[r] == base
    # a stop id ends without being appended
    s, _ = sched()
    r = s.submit_ids([5, 6, 7], 12, SamplingParams(stop_ids=[base[2]]))
    s.run_until_done()
    assert drain(s)[r] == base[:base.index(base[2])] and s.requests[r].finish_reason == "stop"
    # the model's positions end a request
    s, _ = sched(max_positions=8, n_pages=8)
    r = s.submit_ids([1, 2, 3, 4, 5], 50)
    s.run_until_done()
    assert s.requests[r].finish_reason == "context"
    assert len(s.requests[r].gen) + 5 <= 8


def test_when_pages_run_out_the_latest_arrival_is_preempted_and_recomputed():
    # 6 pages of 4 positions; three requests of 6 prompt tokens that each grow to 14
    s, eng = sched(n_pages=6, page_size=4, max_positions=64, max_step_tokens=32, max_requests=4)
    prompts = [[1, 2, 3, 4, 5, 6], [7, 8, 9, 10, 11, 12], [13, 14, 15, 16, 17, 18]]
    ids = [s.submit_ids(p, 8) for p in prompts]
    s.run_until_done(max_steps=500)
    assert s.nactive() == 0
    st = s.get_stats()
    assert st.n_preempt >= 1 and st.recomputed_tokens > 0
    got = drain(s)
    for rid, p in zip(ids, prompts):
        assert got[rid] == serial(p, 8, 50, rid=rid), "preemption changed the output"
    # the first arrival was never the victim
    assert s.requests[ids[0]].n_preempted == 0
    assert s.requests[ids[2]].n_preempted >= 1
    assert st.pool_free == st.pool_pages
    eng.cache.check()


def test_preemption_keeps_the_random_stream():
    sp = SamplingParams(temperature=0.9, seed=5)
    s, eng = sched(n_pages=6, page_size=4, max_positions=64, seed=3)
    prompts = [[1, 2, 3, 4, 5, 6], [7, 8, 9, 10, 11, 12], [13, 14, 15, 16, 17, 18]]
    ids = [s.submit_ids(p, 8, sp) for p in prompts]
    s.run_until_done(max_steps=500)
    assert s.get_stats().n_preempt >= 1
    got = drain(s)
    for rid, p in zip(ids, prompts):
        assert got[rid] == serial(p, 8, 50, sp=sp, seed=3, rid=rid)


def test_the_seed_is_honoured():
    outs = []
    for seed in (1, 2):
        s, _ = sched(seed=seed)
        r = s.submit_ids([3, 4, 5], 10, SamplingParams(temperature=1.0))
        s.run_until_done()
        outs.append(drain(s)[r])
    assert outs[0] != outs[1]


def test_abort_frees_pages_in_any_state():
    s, eng = sched(n_pages=16, max_requests=1)
    a = s.submit_ids([1, 2, 3, 4, 5], 10)
    b = s.submit_ids([1, 2, 3], 10)
    s.step()
    assert s.abort(b) == 0                                    # waiting
    assert s.abort(a) == 0                                    # running
    assert s.abort(a) == -1 and s.abort(12345) == -1
    assert s.nactive() == 0 and eng.cache.n_free_pages() == 16
    assert s.requests[a].finish_reason == "abort"


@pytest.mark.parametrize("seed", range(4))
def test_random_arrivals_match_serial_runs(seed):
    rng = random.Random(seed)
    s, eng = sched(n_pages=10, page_size=4, max_positions=40, max_step_tokens=12, prefill_chunk=5,
                   max_requests=3, seed=seed)
    want = {}
    pending = [([rng.randrange(50) for _ in range(rng.randrange(1, 14))], rng.randrange(1, 9))
               for _ in range(12)]
    steps = 0
    while (pending or s.nactive()) and steps < 3000:
        if pending and rng.random() < 0.4:
            p, n = pending.pop()
            rid = s.submit_ids(p, n)
            assert rid > 0
            want[rid] = serial(p, n, 50, seed=seed, rid=rid)
        s.step()
        eng.cache.check()
        steps += 1
    assert s.nactive() == 0
    assert drain(s) == want
    assert eng.cache.n_free_pages() == 10
