"""The native engine behind the C interface, without a device (its dry-run mode): configuration
and tensor checks, the page tables' invariants and the scheduler's decisions, the last compared
step by step with the Python scheduler on the same arrivals."""
import json
import os
import random

import pytest
import torch

from fakes import FakeEngine
from sglang_c_b200.config import resolve_architecture
from sglang_c_b200.engine.c_api import CEngine, CEngineError
from sglang_c_b200.engine.scheduler import Scheduler
from sglang_c_b200.sampling import SamplingParams
from sglang_c_b200.weights import write_random_model
from sglang_c_b200.weights.safetensors_io import SafetensorsFile, write_safetensors

CFG = dict(architectures=["GPT2LMHeadModel"], model_type="gpt2", n_layer=2, n_embd=24, n_head=3, n_inner=40,
           vocab_size=50, n_positions=40, layer_norm_epsilon=1e-5, activation_function="gelu_new")


def model_dir(tmp_path, cfg=CFG, name="m"):
    arch = resolve_architecture(cfg)
    return write_random_model(str(tmp_path / name), arch, arch.config_class.from_dict(cfg), 7, store_dtype="float32")


def formula(rid, new_len, vocab):
    """The dry run's stand-in for a sampled token."""
    return (rid * 7919 + new_len * 104729) % vocab


class FormulaEngine(FakeEngine):
    """A fake engine whose 'logits' are (request, length after the step) pairs."""

    def step(self, entries):
        wants = [(e.req, self.cache.length(e.req) + len(e.tokens)) for e in entries]
        assert self.cache.can_extend_all(wants)
        rows = []
        for e, (req, new_len) in zip(entries, wants):
            assert self.cache.extend(req, new_len)
            if e.want:
                rows.append((req, new_len))
        self.cache.check()
        self.steps.append([(e.req, len(e.tokens), bool(e.want)) for e in entries])
        return rows


class FormulaSampler:
    def __init__(self, vocab):
        self.vocab = vocab

    def sample(self, logits, params, uniforms, histories=None, want_logprobs=False):
        return [formula(r, n, self.vocab) for r, n in logits]


def drain(s):
    out = {}
    while True:
        g = s.poll()
        if g is None:
            return out
        out[g[0]] = g[1]


def test_the_interface_generates_and_reports(tmp_path):
    d = model_dir(tmp_path)
    e = CEngine(d, dry_run=True, run_ahead=False, page_size=4, n_pages=16, max_requests=4, max_step_tokens=8,
                prefill_chunk=6)
    assert e.vocab_size == 50 and e.max_positions == 40 and e.eos_token_id is None
    a = e.submit_ids(list(range(10)), max_new=3)
    assert a == 1
    assert e.step() == 0 and e.last_step() == [(a, 6, False)]          # a portion of the chunk size
    b = e.submit_ids(list(range(20)), max_new=2)
    e.step()
    assert e.last_step() == [(a, 4, True), (b, 4, False)]              # budget 8: rest of a, then b fills it
    e.step()
    assert e.last_step() == [(a, 1, True), (b, 6, False)]              # a decodes first; b capped by the chunk
    e.run_until_done()
    got = drain(e)
    assert got[a] == [formula(a, 10 + i, 50) for i in range(3)]
    assert got[b] == [formula(b, 20 + i, 50) for i in range(2)]
    st = e.get_stats()
    assert st.prefill_tokens == 30 and st.decode_tokens == 5 and st.n_finished == 2
    assert st.pool_free == st.pool_pages == 16 and st.n_running == 0 and st.n_waiting == 0
    assert e.check()
    e.close()


def test_requests_that_can_never_run_are_refused(tmp_path):
    e = CEngine(model_dir(tmp_path), dry_run=True, page_size=4, n_pages=4)
    assert e.submit_ids([], 4) == -1
    assert e.submit_ids([1, 99], 4) == -1                     # id outside the vocabulary
    assert e.submit_ids(list(range(10)), 10) == -1            # 20 tokens never fit 16 cache positions
    assert e.submit_ids([1] * 40, 1) == -1                    # prompt fills every position
    assert e.submit_ids(list(range(10)), 6) > 0


def test_finishing_rules(tmp_path):
    d = model_dir(tmp_path)
    base = [formula(1, 3 + i, 50) for i in range(12)]
    eos = base[4]
    e = CEngine(d, dry_run=True, eos_token_id=eos)
    r = e.submit_ids([5, 6, 7], 12)
    e.run_until_done()
    assert drain(e)[r] == base[:base.index(eos)] and e.last_finish == "eos"      # eos: not appended
    e = CEngine(d, dry_run=True, eos_token_id=eos)
    r = e.submit_ids([5, 6, 7], 12, SamplingParams(ignore_eos=True))
    e.run_until_done()
    assert drain(e)[r] == base and e.last_finish == "length"
    e = CEngine(d, dry_run=True)
    r = e.submit_ids([5, 6, 7], 12, SamplingParams(stop_ids=[base[2]]))
    e.run_until_done()
    assert drain(e)[r] == base[:base.index(base[2])] and e.last_finish == "stop"
    e = CEngine(d, dry_run=True, page_size=4, n_pages=16)
    r = e.submit_ids(list(range(36)), 50)                     # the model's 40 positions end it
    e.run_until_done()
    got = drain(e)[r]
    assert e.last_finish == "context" and len(got) + 36 <= 40
    e = CEngine(d, dry_run=True, run_ahead=False, max_requests=1)
    a, b = e.submit_ids([1, 2, 3, 4, 5], 10), e.submit_ids([1, 2, 3], 10)
    e.step()
    assert e.abort(b) == 0 and e.abort(a) == 0 and e.abort(a) == -1 and e.abort(12345) == -1
    assert e.nactive() == 0 and e.get_stats().pool_free == e.get_stats().pool_pages
    assert drain(e) == {a: [formula(a, 5, 50)], b: []} and e.check()


@pytest.mark.parametrize("seed", range(6))
def test_decisions_equal_the_python_schedulers_under_random_arrivals(tmp_path, seed):
    """Same arrivals, same step-by-step plans (who runs, how many tokens, who is sampled), same
    preemptions, same output: few pages, so that requests are preempted and recomputed."""
    rng = random.Random(seed)
    kw = dict(page_size=4, n_pages=10, max_requests=3, max_step_tokens=12)
    ce = CEngine(model_dir(tmp_path), dry_run=True, run_ahead=False, prefill_chunk=5, seed=seed, **kw)
    fe = FormulaEngine(vocab=50, max_positions=40, **kw)
    ps = Scheduler(fe, seed=seed, prefill_chunk=5, sampler=FormulaSampler(50))
    pending = [([rng.randrange(50) for _ in range(rng.randrange(1, 14))], rng.randrange(1, 9)) for _ in range(14)]
    steps = 0
    while (pending or ps.nactive()) and steps < 3000:
        if pending and rng.random() < 0.4:
            p, n = pending.pop()
            assert ce.submit_ids(p, n) == ps.submit_ids(p, n) > 0
        n_before = len(fe.steps)
        assert ce.step() == ps.step()
        assert ce.last_step() == (fe.steps[-1] if len(fe.steps) > n_before else [])
        assert ce.check()
        assert ce.nactive() == ps.nactive()
        steps += 1
    assert ce.nactive() == 0
    assert drain(ce) == drain(ps)
    cs, st = ce.get_stats(), ps.get_stats()
    for k in ("prefill_tokens", "decode_tokens", "n_finished", "n_preempt", "recomputed_tokens", "n_steps", "pool_free"):
        assert getattr(cs, k) == getattr(st, k), k
    assert cs.pool_free == 10


def test_when_pages_run_out_the_latest_arrival_is_preempted_and_recomputed(tmp_path):
    # 6 pages of 4 positions; three requests of 6 prompt tokens that each grow to 14
    e = CEngine(model_dir(tmp_path), dry_run=True, run_ahead=False, page_size=4, n_pages=6, max_step_tokens=32,
                max_requests=4)
    prompts = [[1, 2, 3, 4, 5, 6], [7, 8, 9, 10, 11, 12], [13, 14, 15, 16, 17, 18]]
    ids = [e.submit_ids(p, 8) for p in prompts]
    preempted = set()
    running = set()
    for _ in range(500):
        if not e.nactive():
            break
        e.step()
        now = {r for r, _, _ in e.last_step()}
        preempted |= running - now - set(drain_ids(e))
        running = now
        assert e.check()
    assert e.nactive() == 0
    st = e.get_stats()
    assert st.n_preempt >= 1 and st.recomputed_tokens > 0 and st.pool_free == st.pool_pages
    assert ids[0] not in preempted                          # the first arrival was never the victim
    for rid in ids:                                         # the output is what an undisturbed run gives
        assert DONE[rid] == [formula(rid, 6 + i, 50) for i in range(8)]


DONE = {}


def drain_ids(e):
    while True:
        g = e.poll()
        if g is None:
            return list(DONE)
        DONE[g[0]] = g[1]


@pytest.mark.parametrize("seed", range(4))
def test_steps_queued_ahead_change_no_output(tmp_path, seed):
    """run_ahead reads a step's ids one call later and queues the next step of single tokens
    before it has seen them: the same output, request by request, as reading every step at once;
    requests that end by eos, a stop id, their length or the model's positions while a step with
    them is queued have that step's id dropped; aborts in between; few pages."""
    d = model_dir(tmp_path)
    outs = []
    for ahead in (False, True):
        rng = random.Random(seed)
        e = CEngine(d, dry_run=True, run_ahead=ahead, page_size=4, n_pages=12, max_requests=3, max_step_tokens=12,
                    prefill_chunk=5, seed=seed, eos_token_id=7)
        pending = [([rng.randrange(50) for _ in range(rng.randrange(1, 14))], rng.randrange(1, 25),
                    SamplingParams(stop_ids=[rng.randrange(50)], ignore_eos=rng.random() < 0.3)) for _ in range(16)]
        submitted, reasons, steps = [], {}, 0
        while (pending or e.nactive()) and steps < 4000:
            if pending and rng.random() < 0.3:
                p, n, sp = pending.pop()
                submitted.append(e.submit_ids(p, n, sp))
                if len(submitted) == 5:
                    # (aborted before it has run a step: whatever is in flight, it generated nothing)
                    assert e.abort(submitted[-1]) == 0
            e.step()
            assert e.check()
            steps += 1
        assert e.nactive() == 0
        # two more that arrive together and decode side by side with nobody waiting
        for p in ([1, 2, 3], [4, 5, 6, 7]):
            assert e.submit_ids(p, 12, SamplingParams(ignore_eos=True)) > 0
        e.run_until_done()
        got = {}
        while True:
            g = e.poll()
            if g is None:
                break
            got[g[0]] = (g[1], e.last_finish)
        st = e.get_stats()
        assert st.pool_free == st.pool_pages == 12
        assert (st.steps_ahead > 0) == ahead
        outs.append(got)
    assert outs[0] == outs[1]
    assert {r for _, r in outs[1].values()} >= {"length", "abort"}


def test_configuration_errors_name_the_key(tmp_path):
    d = model_dir(tmp_path)
    def with_cfg(**kw):
        c = dict(CFG, **kw)
        c = {k: v for k, v in c.items() if v is not ...}
        with open(os.path.join(d, "config.json"), "w") as f:
            json.dump(c, f)
    with_cfg(n_head=5)
    with pytest.raises(CEngineError, match=r"n_embd \(24\) is not a multiple of n_head \(5\)"):
        CEngine(d, dry_run=True)
    with_cfg(n_layer=...)
    with pytest.raises(CEngineError, match="key 'n_layer' is required"):
        CEngine(d, dry_run=True)
    with_cfg(activation_function="swish")
    with pytest.raises(CEngineError, match="activation_function.*known values"):
        CEngine(d, dry_run=True)
    with_cfg(architectures=["LlamaForCausalLM"], model_type="llama")
    with pytest.raises(CEngineError, match="known architectures: GPT2LMHeadModel"):
        CEngine(d, dry_run=True)
    with open(os.path.join(d, "config.json"), "w") as f:
        f.write("{not json")
    with pytest.raises(CEngineError, match="not valid JSON"):
        CEngine(d, dry_run=True)


def test_weight_errors_come_as_one_message(tmp_path):
    d = model_dir(tmp_path)
    path = os.path.join(d, "model.safetensors")
    f = SafetensorsFile(path)
    tensors = {n: f.tensor(n) for n in f.names()}
    f.close()
    del tensors["h.1.ln_2.bias"]
    tensors["h.0.mlp.c_fc.weight"] = torch.zeros(40, 24)          # transposed
    tensors["extra.weight"] = torch.zeros(3)
    tensors["lm_head.weight"] = torch.zeros(50, 24)               # ignorable
    write_safetensors(path, tensors)
    with pytest.raises(CEngineError) as ei:
        CEngine(d, dry_run=True)
    msg = str(ei.value)
    assert "missing tensors (1): h.1.ln_2.bias" in msg
    assert "unexpected tensors (1): extra.weight" in msg
    assert "h.0.mlp.c_fc.weight: file has [40, 24], model needs [24, 40]" in msg
    assert "lm_head" not in msg


def test_sharded_checkpoints_and_prefixed_names(tmp_path):
    d = model_dir(tmp_path)
    path = os.path.join(d, "model.safetensors")
    f = SafetensorsFile(path)
    tensors = {"transformer." + n: f.tensor(n) for n in f.names()}
    f.close()
    os.remove(path)
    names = sorted(tensors)
    half = len(names) // 2
    write_safetensors(os.path.join(d, "a.safetensors"), {n: tensors[n] for n in names[:half]})
    write_safetensors(os.path.join(d, "b.safetensors"), {n: tensors[n] for n in names[half:]})
    wmap = {n: ("a.safetensors" if i < half else "b.safetensors") for i, n in enumerate(names)}
    with open(os.path.join(d, "model.safetensors.index.json"), "w") as fh:
        json.dump({"weight_map": wmap}, fh)
    e = CEngine(d, dry_run=True)
    assert e.submit_ids([1, 2, 3], 2) == 1
    e.run_until_done()
    wmap[names[0]] = "b.safetensors"
    with open(os.path.join(d, "model.safetensors.index.json"), "w") as fh:
        json.dump({"weight_map": wmap}, fh)
    with pytest.raises(CEngineError, match="tensors not found in the shard it names"):
        CEngine(d, dry_run=True)


def test_a_c_program_on_the_interface_generates(tmp_path):
    """csrc/apps/sglc.c, compiled with the system's C compiler and linked against the engine's
    library, run without a device."""
    import subprocess
    from sglang_c_b200.csrc import build
    exe = build.build_app("sglc")
    d = model_dir(tmp_path)
    r = subprocess.run([exe, "--model", d, "--prompt-ids", "5, 6 7", "--max-new", "5", "--dry-run", "--verbose"],
                       capture_output=True, text=True, timeout=60)
    assert r.returncode == 0, r.stderr
    assert r.stdout.split() == [str(t) for t in [5, 6, 7] + [formula(1, 3 + i, 50) for i in range(5)]]
    assert "generated 5 tokens" in r.stderr and "finish reason 3" in r.stderr
    r = subprocess.run([exe, "--model", d, "--prompt-ids", "5 99", "--dry-run"], capture_output=True, text=True)
    assert r.returncode == 2 and "refused" in r.stderr
    r = subprocess.run([exe, "--model", str(tmp_path / "nothing"), "--prompt-ids", "5", "--dry-run"],
                       capture_output=True, text=True)
    assert r.returncode == 2 and "no config.json" in r.stderr


@pytest.mark.parametrize("seed", range(5))
def test_page_tables_under_random_orders(seed):
    """The native page tables alone: requests arrive, grow by portions of any size, are cut back
    and end in random order, in a group with all keys and a group with a window; no page lost,
    held twice or freed twice, no visible page given back (checked inside the library)."""
    import ctypes as C
    from sglang_c_b200.csrc import build
    lib = build.load("host_engine")
    err = C.create_string_buffer(512)
    for page_size, n_pages, window in ((4, 24, 9), (16, 12, 40), (1, 64, 5)):
        rc = lib.sglc_pages_selftest(page_size, n_pages, 5, window, seed, 4000, err, len(err))
        assert rc == 0, err.value.decode()
