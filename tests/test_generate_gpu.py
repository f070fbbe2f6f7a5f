"""Generation through the entry points: greedy and sampled, one request and many, with and
without page pressure, against the plain implementation."""
import os
import subprocess
import sys

import numpy as np
import pytest

import plain_gpt2
import traces
from conftest import PAGE_SIZE, ROOT, TINY

pytestmark = pytest.mark.gpu
STORE = {"float32": "float32", "bfloat16": "bfloat16"}
# a different token than the plain implementation's is accepted only where the plain logits
# of the two are this close (a near tie that rounding may flip)
TIE = {"float32": 1e-4, "bfloat16": 2e-2}


def check_greedy(model_dir, prompt, got, dtype):
    cfg, w = plain_gpt2.read_model_dir(model_dir)
    seq = list(prompt)
    for t in got:
        lg = plain_gpt2.forward(cfg, w, seq)[-1]
        best = int(np.argmax(lg))
        assert t == best or lg[best] - lg[t] < TIE[dtype], (t, best, float(lg[best] - lg[t]))
        seq.append(t)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_greedy_generation_matches_plain(model_dirs, name, dtype):
    from sglang_c_b200.engine import generate, sched_new
    from sglang_c_b200.sampling import SamplingParams
    d = model_dirs(name, STORE[dtype])
    V = TINY[name]["vocab_size"]
    lens = [5, 17, 32] if name == "A" else [1, 9, 40, 63, 100]
    prompts = [traces.random_tokens(70 + i, n, V) for i, n in enumerate(lens)]
    s = sched_new(d, dtype=dtype, page_size=PAGE_SIZE[name], max_tokens=1024, max_requests=8,
                  max_step_tokens=64, prefill_chunk=24)
    seen = []
    got = generate(s, prompts, SamplingParams(temperature=0.0), max_new=16,
                   on_token=lambda i, t: seen.append((i, t)))
    for p, g in zip(prompts, got):
        assert len(g) == 16
        check_greedy(d, p, g, dtype)
    assert sorted(t for i, t in seen if i == 0) == sorted(got[0])
    st = s.get_stats()
    assert st.n_finished == len(prompts) and st.pool_free == st.pool_pages
    # one prompt alone gives the same tokens as in the batch
    s2 = sched_new(d, dtype=dtype, page_size=PAGE_SIZE[name], max_tokens=256, max_requests=2,
                   max_step_tokens=128)
    alone = generate(s2, prompts[1], SamplingParams(temperature=0.0), max_new=16)
    if dtype == "float32":
        assert alone == got[1]
    else:
        check_greedy(d, prompts[1], alone, dtype)


def _mix64(x):
    m = (1 << 64) - 1
    x &= m
    x ^= x >> 33
    x = (x * 0xFF51AFD7ED558CCD) & m
    x ^= x >> 33
    x = (x * 0xC4CEB9FE1A85EC53) & m
    x ^= x >> 33
    return x


def _stream(seed, rid):
    m = (1 << 64) - 1
    return _mix64((seed & m) ^ _mix64((rid * 0x9E3779B97F4A7C15 + 1) & m)) or 0x9E3779B97F4A7C15


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_temperature_sampling_follows_the_plain_distribution(model_dirs, dtype):
    """With the request's own random stream restated here, every sampled token must be the
    one whose interval of the plain implementation's CDF (in index order) holds the draw."""
    from sglang_c_b200.engine import sched_new
    from sglang_c_b200.sampling import SamplingParams
    name = "B"
    d = model_dirs(name, STORE[dtype])
    V = TINY[name]["vocab_size"]
    cfg, w = plain_gpt2.read_model_dir(d)
    prompts = [traces.random_tokens(90 + i, n, V) for i, n in enumerate([1, 9, 40, 63, 100])]
    seed, T = 7, 0.8
    s = sched_new(d, seed=seed, dtype=dtype, page_size=PAGE_SIZE[name], max_tokens=2048, max_requests=8,
                  max_step_tokens=64, prefill_chunk=24)
    ids = [s.submit_ids(p, 24, SamplingParams(temperature=T, seed=3)) for p in prompts]
    s.run_until_done()
    out = {}
    while True:
        g = s.poll()
        if g is None:
            break
        out[g[0]] = g[1]
    slack = 1e-5 if dtype == "float32" else 2e-2
    for rid, p in zip(ids, prompts):
        state = _stream(seed ^ 3, rid)
        seq = list(p)
        assert len(out[rid]) == 24
        for t in out[rid]:
            state, u = plain_gpt2.uniform(state)
            cdf = np.cumsum(plain_gpt2.temperature_probs(plain_gpt2.forward(cfg, w, seq)[-1], T))
            lo = cdf[t - 1] if t > 0 else 0.0
            assert lo - slack <= u <= cdf[t] + slack, (rid, t, u, lo, cdf[t])
            seq.append(t)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_page_pressure_preempts_and_output_stays(model_dirs, dtype):
    from sglang_c_b200.engine import generate, sched_new
    from sglang_c_b200.sampling import SamplingParams
    name = "A"
    d = model_dirs(name, STORE[dtype])
    V = TINY[name]["vocab_size"]
    prompts = [traces.random_tokens(30 + i, n, V) for i, n in enumerate([40, 33, 50, 21, 45, 38])]
    sp = SamplingParams(temperature=0.0)
    roomy = sched_new(d, dtype=dtype, page_size=16, max_tokens=2048, max_requests=8, max_step_tokens=64)
    want = generate(roomy, prompts, sp, max_new=30)
    tight = sched_new(d, dtype=dtype, page_size=16, n_pages=14, max_requests=8, max_step_tokens=64)
    got = generate(tight, prompts, sp, max_new=30)
    st = tight.get_stats()
    assert st.n_preempt >= 1, "the pool was meant to be too small for all requests at once"
    assert st.pool_free == st.pool_pages
    tight.engine.cache.check()
    if dtype == "float32":
        assert got == want
    else:
        for p, g in zip(prompts, got):
            check_greedy(d, p, g, dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_steps_prepared_ahead_change_nothing(model_dirs, dtype):
    """The scheduler queues the next step of single tokens behind the one in flight (ids pass on
    the device) and reads a step's ids one call later; it falls back to wait-plan-launch when a
    request ends, is aborted or arrives.  With requests that end at different times (lengths, a
    stop id, the model's positions), an arrival and an abort in between, the tokens are those
    of a scheduler that reads every step's ids at once, and no page is lost."""
    from sglang_c_b200.engine import sched_new
    from sglang_c_b200.sampling import SamplingParams
    name = "B"
    d = model_dirs(name, STORE[dtype])
    V = TINY[name]["vocab_size"]
    prompts = [traces.random_tokens(50 + i, n, V) for i, n in enumerate([7, 30, 15, 44, 3])]
    max_new = [40, 9, 25, 33, 40]

    def run(ahead, stop_ids):
        s = sched_new(d, dtype=dtype, page_size=PAGE_SIZE[name], max_tokens=1024, max_requests=8,
                      max_step_tokens=64, prefill_chunk=24)
        s.lagging = ahead
        ids = [s.submit_ids(p, m, SamplingParams(temperature=0.9 if i == 2 else 0.0, top_k=40 if i == 2 else 0,
                                                 stop_ids=list(stop_ids) if i == 0 else []))
               for i, (p, m) in enumerate(zip(prompts[:4], max_new[:4]))]
        steps = 0
        while s.nactive() > 0:
            s.step()
            steps += 1
            if steps == 12:
                ids.append(s.submit_ids(prompts[4], max_new[4], SamplingParams(temperature=0.0)))
            if steps == 20:
                s.abort(ids[3])
        out = [list(s.requests[i].gen) for i in ids]
        st = s.get_stats()
        assert st.pool_free == st.pool_pages
        s.engine.cache.check()
        return out, s.engine.graph_replays

    plain, _ = run(False, [])
    # request 0 ends on a stop id in the middle of steady decoding (the first id from place 8 on
    # that it has not produced before), while a step with it is already queued
    j = next(j for j in range(8, len(plain[0])) if plain[0][j] not in plain[0][:j])
    stop = [plain[0][j]]
    want, _ = run(False, stop)
    got, _ = run(True, stop)
    assert len(want[0]) == j and len(want[1]) == 9
    # the aborted request has read one step less when the abort comes after the same number
    # of calls; what it has is the same
    assert got[3] == want[3][:len(got[3])] and 0 <= len(want[3]) - len(got[3]) <= 1
    assert got[:3] + got[4:] == want[:3] + want[4:]


def test_command_line_with_random_weights(tmp_path):
    import json
    cfg = tmp_path / "config.json"
    cfg.write_text(json.dumps(TINY["A"]))
    cmd = [sys.executable, os.path.join(ROOT, "bin", "sglc"), "--random-weights", "5", "--config", str(cfg),
           "--save-model", str(tmp_path / "m"), "--prompt", "3, 1, 4, 1, 5", "--max-new", "6",
           "--temperature", "0", "--dtype", "fp32", "--verbose"]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr
    ids = [int(t) for t in r.stdout.split()]
    assert ids[:5] == [3, 1, 4, 1, 5] and len(ids) == 11
    assert "generated 6 tokens" in r.stderr and "tok/s" in r.stderr
    check_greedy(str(tmp_path / "m"), ids[:5], ids[5:], "float32")
    # the same folder through --model, sampled with the reference's default options
    r2 = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "sglc"), "--model", str(tmp_path / "m"),
                         "--prompt-ids", "3 1 4", "--max-new", "4", "--seed", "2"],
                        capture_output=True, text=True, timeout=300)
    assert r2.returncode == 0, r2.stderr
    assert len(r2.stdout.split()) == 7
