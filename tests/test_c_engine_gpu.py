"""The native engine behind the C interface on the device: greedy generation against the plain
implementation, and everything it generates (greedy and sampled, penalties, stop ids, few pages
so that requests are preempted and recomputed) against the Python scheduler on the same model:
both launch the same kernels, so the ids are equal."""
import numpy as np
import pytest

import plain_gpt2
import traces
from conftest import PAGE_SIZE, TINY

pytestmark = pytest.mark.gpu
STORE = {"float32": "float32", "bfloat16": "bfloat16"}
TIE = {"float32": 1e-4, "bfloat16": 2e-2}


def drain(s):
    out = {}
    while True:
        g = s.poll()
        if g is None:
            return out
        out[g[0]] = g[1]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_greedy_generation_matches_plain(model_dirs, name, dtype):
    from sglang_c_b200.engine.c_api import CEngine
    d = model_dirs(name, STORE[dtype])
    V = TINY[name]["vocab_size"]
    lens = [5, 17, 32] if name == "A" else [1, 9, 40, 63, 100]
    prompts = [traces.random_tokens(70 + i, n, V) for i, n in enumerate(lens)]
    e = CEngine(d, dtype=dtype, page_size=PAGE_SIZE[name], max_tokens=1024, max_requests=8, max_step_tokens=64,
                prefill_chunk=24)
    ids = [e.submit_ids(p, 16) for p in prompts]
    e.run_until_done()
    got = drain(e)
    cfg, w = plain_gpt2.read_model_dir(d)
    for rid, p in zip(ids, prompts):
        assert len(got[rid]) == 16
        seq = list(p)
        for t in got[rid]:
            lg = plain_gpt2.forward(cfg, w, seq)[-1]
            best = int(np.argmax(lg))
            assert t == best or lg[best] - lg[t] < TIE[dtype], (t, best, float(lg[best] - lg[t]))
            seq.append(t)
    st = e.get_stats()
    assert st.n_finished == len(prompts) and st.pool_free == st.pool_pages and st.graph_replays > 0
    assert e.check()
    e.close()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name,n_pages", [("A", 9), ("B", 40), ("C", 64)])
def test_everything_it_generates_equals_the_python_engines(model_dirs, name, n_pages, dtype):
    """Mixed sampling options, arrivals over time and a pool so small that requests are preempted:
    the same ids, finish reasons, log-probabilities and counters from both engines."""
    from sglang_c_b200.engine import sched_new
    from sglang_c_b200.engine.c_api import CEngine
    from sglang_c_b200.sampling import SamplingParams
    d = model_dirs(name, STORE[dtype])
    V = TINY[name]["vocab_size"]
    kw = dict(dtype=dtype, page_size=PAGE_SIZE[name], n_pages=n_pages, max_requests=4, max_step_tokens=48,
              prefill_chunk=20, seed=11, want_logprobs=True)
    py = sched_new(d, **kw)
    ce = CEngine(d, **kw)
    sps = [SamplingParams(), SamplingParams(temperature=0.9, seed=3), SamplingParams(temperature=1.3, top_k=20, top_p=0.9),
           SamplingParams(temperature=0.7, repetition_penalty=1.3, frequency_penalty=0.2, presence_penalty=0.1),
           SamplingParams(temperature=1.0, min_p=0.05, stop_ids=[3, 5, 7]), SamplingParams(ignore_eos=True)]
    # A: short prompts that grow long, so that the running requests outgrow the pool
    lens = {"A": [10, 5, 14, 8, 3, 12], "B": [33, 5, 61, 18, 2, 47, 29, 70], "C": [300, 40, 5, 180, 77, 260]}[name]
    new = (lambda i: 50) if name == "A" else (lambda i: 6 + 3 * (i % 4))
    arrivals = [(traces.random_tokens(500 + i, n, V), new(i), sps[i % len(sps)]) for i, n in enumerate(lens)]
    steps = 0
    while (arrivals or py.nactive()) and steps < 2000:
        if arrivals and steps % 3 == 0:
            p, n, sp = arrivals.pop(0)
            a, b = py.submit_ids(p, n, sp), ce.submit_ids(p, n, sp)
            assert a == b > 0
        py.step()
        ce.step()
        assert ce.check()
        steps += 1
    while py.nactive():          # (the Python scheduler reads a step's ids one call later)
        py.step()
    assert ce.nactive() == 0
    got_py = {}
    while True:
        g = py.poll()
        if g is None:
            break
        got_py[g[0]] = (g[1], py.requests[g[0]].finish_reason, py.poll_logprobs(g[0]))
    got_c = {}
    while True:
        g = ce.poll()
        if g is None:
            break
        got_c[g[0]] = (g[1], ce.last_finish, ce.last_logprobs)
    assert set(got_c) == set(got_py)
    for rid in got_py:
        assert got_c[rid][0] == got_py[rid][0], rid
        assert got_c[rid][1] == got_py[rid][1], rid
        np.testing.assert_allclose(got_c[rid][2], got_py[rid][2], rtol=0, atol=1e-6)
    cs, st = ce.get_stats(), py.get_stats()
    for k in ("prefill_tokens", "decode_tokens", "n_finished", "n_preempt", "recomputed_tokens", "pool_free"):
        assert getattr(cs, k) == getattr(st, k), k
    if name == "A":
        assert cs.n_preempt >= 1
    ce.close()


def test_it_refuses_to_start_without_its_kernel_libraries(model_dirs, tmp_path):
    from sglang_c_b200.engine.c_api import CEngine, CEngineError, COptions
    import ctypes as C
    e = CEngine(model_dirs("A"), dry_run=True)
    o = COptions()
    e.lib.sglc_engine_options_default(C.byref(o))
    o.library_dir = str(tmp_path).encode()
    err = C.create_string_buffer(4096)
    assert not e.lib.sglc_engine_new(model_dirs("A").encode(), C.byref(o), err, len(err))
    assert b"cannot be loaded" in err.value and b"no CPU path" in err.value


def test_the_c_program_generates_what_the_python_entry_point_generates(model_dirs):
    import os
    import subprocess
    from conftest import ROOT
    from sglang_c_b200.engine import generate, sched_new
    from sglang_c_b200.sampling import SamplingParams
    d = model_dirs("B", "bfloat16")
    prompt = traces.random_tokens(3, 21, TINY["B"]["vocab_size"])
    r = subprocess.run([os.path.join(ROOT, "bin", "sglc_native"), "--model", d, "--prompt-ids",
                        " ".join(map(str, prompt)), "--max-new", "12", "--temperature", "0.9", "--seed", "4",
                        "--page-size", "8", "--verbose"], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr
    got = [int(t) for t in r.stdout.split()]
    s = sched_new(d, seed=4, dtype="bfloat16", page_size=8, max_tokens=128, max_requests=4)
    want = generate(s, prompt, SamplingParams(temperature=0.9, top_k=50, top_p=0.95, seed=4), 12)
    assert got == prompt + want
    assert "generated" in r.stderr and "MB of weights" in r.stderr


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_equals_the_python_engines(model_dirs, dtype):
    """Two requests that decode for hundreds of steps side by side (steps queued ahead, a new
    graph each time the context bound moves, pages taken one by one), a third that arrives in
    between and stops at a stop id: the same ids from both engines."""
    from sglang_c_b200.engine import sched_new
    from sglang_c_b200.engine.c_api import CEngine
    from sglang_c_b200.sampling import SamplingParams
    d = model_dirs("C", STORE[dtype])
    V = TINY["C"]["vocab_size"]
    kw = dict(dtype=dtype, page_size=16, n_pages=140, max_requests=4, max_step_tokens=64, prefill_chunk=32, seed=2)
    py, ce = sched_new(d, **kw), CEngine(d, **kw)
    jobs = [(traces.random_tokens(1, 9, V), 700, SamplingParams(temperature=0.8, ignore_eos=True)),
            (traces.random_tokens(2, 40, V), 650, SamplingParams(ignore_eos=True))]
    for p, n, sp in jobs:
        assert py.submit_ids(p, n, sp) == ce.submit_ids(p, n, sp) > 0
    for s in (py, ce):
        for _ in range(300):
            s.step()
    late = (traces.random_tokens(3, 21, V), 200, SamplingParams(temperature=1.1, stop_ids=[1, 2, 3, 4, 5, 6, 7, 8]))
    assert py.submit_ids(*late) == ce.submit_ids(*late) > 0
    py.run_until_done()
    ce.run_until_done()
    got_py, got_c = drain(py), drain(ce)
    assert got_c == got_py
    assert len(got_c[1]) == 700 and len(got_c[2]) == 650
    st = ce.get_stats()
    assert st.steps_ahead > 500 and st.graph_replays > 600 and st.pool_free == st.pool_pages
    assert ce.check()
    ce.close()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_half_and_double_precision_files_load_alike(model_dirs, tmp_path, dtype):
    """A file with float16 matrices and float64 vectors: the native loader converts as the Python
    loader does (float16 and float64 to 32-bit exactly / by rounding, then to the runtime's
    precision), so both engines generate the same ids."""
    import json
    import os
    import torch
    from sglang_c_b200.engine import generate, sched_new
    from sglang_c_b200.engine.c_api import CEngine
    from sglang_c_b200.sampling import SamplingParams
    from sglang_c_b200.weights.safetensors_io import SafetensorsFile, write_safetensors
    src = model_dirs("B")
    d = str(tmp_path / "mixed_precisions")
    os.makedirs(d)
    with open(os.path.join(src, "config.json")) as f, open(os.path.join(d, "config.json"), "w") as g:
        json.dump(json.load(f), g)
    f = SafetensorsFile(os.path.join(src, "model.safetensors"))
    tensors = {n: (f.tensor(n).to(torch.float16) if f.tensor(n).dim() == 2 else f.tensor(n).to(torch.float64))
               for n in f.names()}
    f.close()
    write_safetensors(os.path.join(d, "model.safetensors"), tensors)
    prompts = [traces.random_tokens(9, 30, TINY["B"]["vocab_size"]), traces.random_tokens(10, 7, TINY["B"]["vocab_size"])]
    sp = SamplingParams(temperature=0.9, seed=1)
    kw = dict(dtype=dtype, page_size=8, max_tokens=512, max_requests=4, seed=6)
    want = generate(sched_new(d, **kw), prompts, sp, 20)
    ce = CEngine(d, **kw)
    ids = [ce.submit_ids(p, 20, sp) for p in prompts]
    ce.run_until_done()
    got = drain(ce)
    assert [got[i] for i in ids] == want
    ce.close()


def test_the_python_entry_points_run_on_the_native_engine(model_dirs, capsys):
    """sched_new(native=True) gives the same entry points on the native engine: `generate` with
    its per-token callback, and the command line's --native, give the ids of the Python engine."""
    from sglang_c_b200 import cli
    from sglang_c_b200.engine import generate, sched_new
    from sglang_c_b200.sampling import SamplingParams
    d = model_dirs("A", "bfloat16")
    prompts = [traces.random_tokens(5, 12, TINY["A"]["vocab_size"]), traces.random_tokens(6, 3, TINY["A"]["vocab_size"])]
    sp = SamplingParams(temperature=0.8, top_k=50, top_p=0.95, seed=3)
    kw = dict(seed=3, dtype="bfloat16", page_size=16, max_tokens=256, max_requests=4)
    want = generate(sched_new(d, **kw), prompts, sp, 10)
    seen = []
    got = generate(sched_new(d, native=True, **kw), prompts, sp, 10, on_token=lambda i, t: seen.append((i, t)))
    assert got == want
    assert [t for i, t in seen if i == 0] == want[0] and [t for i, t in seen if i == 1] == want[1]
    ids = " ".join(map(str, prompts[0]))
    outs = []
    for extra in ([], ["--native"]):
        assert cli.main(["--model", d, "--prompt-ids", ids, "--max-new", "10", "--seed", "3", "--verbose"] + extra) == 0
        outs.append(capsys.readouterr().out.split())
    assert outs[0] == outs[1] and len(outs[0]) == len(prompts[0]) + 10
