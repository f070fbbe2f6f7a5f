"""Decode and prefill throughput of the engine on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

The default run has the layer sizes of GPT-2 small (n_layer 12, n_embd 768,
n_head 12, n_inner 3072, vocab 50257, positions 1024) with random weights in
bfloat16, a batch of 8 requests decoding at a context of 512 tokens, pages of
16.  A "step" is one decode step of the whole batch.  One JSON line is printed:
`value` is decoded tokens a second with the steps timed on the device (CUDA events
on the stream the steps run on, around chunks of K steps of the native engine's
scheduler, each step's sampled ids feeding the next; the median of five regions of
at least 50 ms each; a step reads more than L2 holds, so nothing is flushed;
`points.decode_b8_python_engine` is the same for the Python engine's loop); `e2e` is the same through the Python entry point (`sched_new(...,
native=True)`: scheduler and step in C++, host token ids in and out every step;
`points.e2e_python_scheduler_b8` is the Python scheduler); `prefill` is one step of 2,048 prompt tokens (2 x 1,024);
`roofline` is the decode step's bytes (every weight once, the cache of the live
requests) over its time, against the measured copy bandwidth; `points` has decode
at batch 1 and 64, the true 32-bit path and the prefill through the C interface;
`kernels` says where a decode and a
prefill step's time goes, kernel by kernel.  `--full` adds medium and XL layer
sizes and the mixed workload to `points`.
"""
import argparse
import atexit
import json
import os
import shutil
import statistics
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

SMALL = dict(architectures=["GPT2LMHeadModel"], model_type="gpt2", n_layer=12, n_embd=768, n_head=12,
             n_inner=3072, vocab_size=50257, n_positions=1024, layer_norm_epsilon=1e-5,
             activation_function="gelu_new")
MEDIUM = dict(SMALL, n_layer=24, n_embd=1024, n_head=16, n_inner=4096)
XL = dict(SMALL, n_layer=48, n_embd=1600, n_head=25, n_inner=6400)
MODELS = {"small": SMALL, "medium": MEDIUM, "xl": XL}
CONTEXT = 512
BATCH = 8
PAGE = 16
PREFILL_TOKENS = 2048


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            d = json.load(f)
        return dict(hbm_gbs=d["hbm_gbs"], bf16_tflops=d["bf16_tflops"], source="measured")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, source="fallback")


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.rows = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            if len(r) < 6:
                continue
            try:
                sm.append(float(r[0]))
                mx.append(float(r[1]))
            except ValueError:
                continue
            for n, v in zip(names, r[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def model_bytes_flops(cfg, batch, context, elem=2, kv_elem=None):
    """Bytes a decode step has to read (every weight it uses once, the cache of
    the live requests) and the flops of a prefill of T tokens as n prompts."""
    E, I, L, V, H = cfg["n_embd"], cfg["n_inner"], cfg["n_layer"], cfg["vocab_size"], cfg["n_head"]
    mats = L * (E * 3 * E + E * E + E * I + I * E)
    vecs = L * (3 * E + E + I + E + 4 * E) + 2 * E
    weights = (mats + V * E) * elem + vecs * 4 + batch * E * elem      # + the position rows used
    kv = batch * context * L * 2 * E * (kv_elem or elem)
    return weights + kv


def prefill_flops(cfg, n_prompts, prompt_len):
    E, I, L, V = cfg["n_embd"], cfg["n_inner"], cfg["n_layer"], cfg["vocab_size"]
    T = n_prompts * prompt_len
    gemm = 2 * T * L * (E * 3 * E + E * E + 2 * E * I)
    attn = n_prompts * L * 4 * E * (prompt_len * (prompt_len + 1) // 2)
    head = 2 * n_prompts * V * E
    return gemm + attn + head


def make_model(tmp, cfg_d, n_layer=None):
    from sglang_c_b200.config import resolve_architecture
    from sglang_c_b200.weights import write_random_model
    d = dict(cfg_d)
    if n_layer is not None:
        d["n_layer"] = n_layer
    arch = resolve_architecture(d)
    cfg = arch.config_class.from_dict(d)
    return write_random_model(os.path.join(tmp, "model"), arch, cfg, 1234, scheme="standard",
                              store_dtype="bfloat16")


REGION_MS = 50.0       # a timed region lasts at least this long
N_REGIONS = 5          # a point is the median of this many regions


def time_decode(eng, batch, context, steps, warmup):
    """Decode steps of `batch` requests that hold `context` tokens each, timed on the device.
    A chunk is `steps` steps in a row between one pair of CUDA events, real decoding (each step's
    sampled ids are the next step's input, on the device) queued one ahead as the scheduler does;
    after a chunk the requests are rewound to `context` (host bookkeeping only, untimed) and one
    untimed step re-primes the repeat path.  A region is as many chunks as it takes to reach
    REGION_MS of device time; the result is the median region's ms per step over N_REGIONS, with
    the launches of one chunk.  L2 is not flushed: a step reads more than L2 holds (every weight
    and the cache of the live requests)."""
    import numpy as np
    import torch
    from sglang_c_b200.csrc import ops
    from sglang_c_b200.engine import StepEntry
    from sglang_c_b200.sampling import Sampler
    V = eng.plan.vocab_size
    rng = np.random.default_rng(batch)
    reqs = [f"b{batch}_{i}" for i in range(batch)]
    for r in reqs:
        eng.add_request(r)
    todo = {r: [int(t) for t in rng.integers(0, V, size=context)] for r in reqs}
    done = 0
    while done < context:
        n = min(eng.max_step_tokens // batch, context - done)
        eng.step([StepEntry(r, todo[r][done:done + n], []) for r in reqs])
        done += n
    sampler = Sampler(eng.rt.device, max(batch, 1))
    toks = [int(t) for t in rng.integers(0, V, size=batch)]

    def one_step(first):
        if first or not eng.prepare_repeat(reqs):
            logits = eng.step([StepEntry(r, [t], [0]) for r, t in zip(reqs, toks)])
        else:
            logits = eng.run_prepared(device_tokens=sampler.d_out)
        ops.sample(logits, sampler.d_params[:batch], sampler.d_hist_tok, sampler.d_hist_cnt,
                   sampler.d_out[:batch])

    def chunk(n):
        for r in reqs:
            eng.truncate(r, context)
        one_step(True)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        l0 = ops.LAUNCHES
        e0.record()
        for _ in range(n):
            one_step(False)
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1), ops.LAUNCHES - l0

    chunk(max(warmup, 3))
    regions, launches = [], 0
    for _ in range(N_REGIONS):
        ms, n = 0.0, 0
        while ms < REGION_MS:
            t, launches = chunk(steps)
            ms += t
            n += steps
        regions.append(ms / n)
    for r in reqs:
        eng.end_request(r)
    return statistics.median(regions), launches, regions


def time_decode_native(model_dir, batch, context, steps, warmup, dtype="bfloat16"):
    """time_decode on the native engine (`sched_new(..., native=True)`): the requests are brought to
    `context` tokens through the scheduler, then chunks of `steps` decode steps are timed on the
    device between two marks on the stream the steps run on (sglc_engine_mark: CUDA events; the
    stream is synchronised before the first, the second is waited for).  The steps are the
    scheduler's own: each queued behind the one in flight, its ids taken from the sampler on the
    device, arrays up and ids down on side streams, the sampler inside the step's graph.  After a
    chunk the requests are rewound to their first generated token (host bookkeeping, untimed) and
    one untimed step re-primes the queue.  Median region's ms per step, launches of a chunk,
    the regions."""
    import numpy as np
    from sglang_c_b200.engine import sched_new
    from sglang_c_b200.sampling import SamplingParams
    e = sched_new(model_dir, seed=0, dtype=dtype, page_size=PAGE, max_tokens=batch * (context + steps + warmup + 96),
                  max_requests=max(batch, 1), max_step_tokens=PREFILL_TOKENS, prefill_chunk=512, native=True)
    rng = np.random.default_rng(batch)
    sp = SamplingParams(temperature=0.0, ignore_eos=True)
    ids = [e.submit_ids([int(t) for t in rng.integers(0, e.vocab_size, size=context)], warmup + steps + 64, sp)
           for _ in range(batch)]
    while True:                                    # prompts done; every request decodes from here
        e.step()
        ran = e.last_step()
        if len(ran) == batch and all(n == 1 for _, n, _ in ran):
            break

    def chunk(n):
        e.sync()
        for i in ids:
            e.rewind(i, 1)
        e.step()
        e.step()                                   # (two: the second is queued ahead of the first's ids)
        l0 = e.get_stats().launches
        e.mark(sync_first=True)
        for _ in range(n):
            e.step()
        e.mark()
        return e.ms_between_marks(), e.get_stats().launches - l0

    for _ in range(max(1, (warmup + steps - 1) // steps)):
        chunk(steps)
    regions, launches = [], 0
    for _ in range(N_REGIONS):
        ms, n = 0.0, 0
        while ms < REGION_MS:
            t, launches = chunk(steps)
            ms += t
            n += steps
        regions.append(ms / n)
    for i in ids:
        e.abort(i)
    e.close()
    return statistics.median(regions), launches, regions


def time_prefill(eng, n_prompts, prompt_len, warmup, behind_sleep=False):
    """One step of n_prompts whole prompts; the median of N_REGIONS regions of at least REGION_MS
    of device time each (a region is steps in a row, each on fresh requests).  The events stand
    around the call of the step, so the host's preparation of a 2,048-token step (about 0.2 ms
    during which the device waits) is inside; with behind_sleep the step is queued behind a
    millisecond of device sleep instead, which hides the host's part as a scheduler that prepares
    a step while the last one runs does: the device's own time for the step."""
    import numpy as np
    import torch
    from sglang_c_b200.engine import StepEntry
    V = eng.plan.vocab_size
    rng = np.random.default_rng(99)
    it = [0]

    def once():
        it[0] += 1
        reqs = [f"p{it[0]}_{i}" for i in range(n_prompts)]
        for r in reqs:
            eng.add_request(r)
        # (ids as arrays, as the scheduler hands a prompt's portions to the engine)
        entries = [StepEntry(r, rng.integers(0, V, size=prompt_len).astype(np.int32), [prompt_len - 1])
                   for r in reqs]
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        if behind_sleep:
            torch.cuda._sleep(2_000_000)
        e0.record()
        eng.step(entries)
        e1.record()
        torch.cuda.synchronize()
        for r in reqs:
            eng.end_request(r)
        return e0.elapsed_time(e1)

    for _ in range(max(warmup, 3)):
        once()
    regions = []
    for _ in range(N_REGIONS):
        ms, n = 0.0, 0
        while ms < REGION_MS:
            ms += once()
            n += 1
        regions.append(ms / n)
    return statistics.median(regions)


def kernel_table(eng, batch, context, prompt_len):
    """Where a step's time goes, kernel by kernel: a decode step of `batch` requests at `context`
    and a prefill step of two prompts, each run once operation by operation (no graph) with a pair
    of CUDA events around every launch, queued behind a few milliseconds of device sleep so that
    the host's launch cost does not fall between the events; the cost of an empty pair of events
    is measured in the same queue and taken off every launch.  Kernels are kept from overlapping
    by the events, so the figures are each kernel's own time, not its share of an overlapped step."""
    import numpy as np
    import torch
    from sglang_c_b200.csrc import ops
    from sglang_c_b200.engine import StepEntry
    V = eng.plan.vocab_size
    rng = np.random.default_rng(7)
    graphs, eng.use_graphs = eng.use_graphs, False
    out = {}
    try:
        reqs = [f"k{i}" for i in range(batch)]
        for r in reqs:
            eng.add_request(r)
        done = 0
        while done < context:
            n = min(eng.max_step_tokens // batch, context - done)
            eng.step([StepEntry(r, [int(t) for t in rng.integers(0, V, size=n)], []) for r in reqs])
            done += n
        for name, make in (("decode", lambda: [StepEntry(r, [1], [0]) for r in reqs]), ("prefill", None)):
            if make is None:
                for r in reqs:
                    eng.end_request(r)
                reqs = ["kp0", "kp1"]
                for r in reqs:
                    eng.add_request(r)
                make = lambda: [StepEntry(r, [int(t) for t in rng.integers(0, V, size=prompt_len)],
                                          [prompt_len - 1]) for r in reqs]
            entries = make()
            if name == "decode":
                eng.step(entries)                      # the kernels' first call is not what is timed
                for r in reqs:
                    eng.truncate(r, context)
            torch.cuda.synchronize()
            torch.cuda._sleep(20_000_000)              # about 10 ms: the step is queued whole behind it
            empty = []
            for _ in range(16):                        # what a pair of events costs with nothing between
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
                b.record()
                empty.append((a, b))
            ops.profile_begin()
            eng.step(entries)
            rows = ops.profile_end()
            pair_us = statistics.median(a.elapsed_time(b) for a, b in empty) * 1e3
            out[name] = {k: {"launches": n, "us": round(max(us - n * pair_us, 0.0), 1)}
                         for k, (n, us) in sorted(rows.items())}
            out[name]["event_pair_us"] = round(pair_us, 2)
        for r in reqs:
            eng.end_request(r)
    finally:
        eng.use_graphs = graphs
    return out


def time_e2e(model_dir, batch, context, steps, warmup, dtype="bfloat16"):
    """The same decode through the Python entry point: token ids on the host in, token ids on
    the host out, every step; wall clock.  A region is fresh requests with prompts of `context`
    tokens, run until all decode, `warmup` steps, then enough steps for REGION_MS (at least
    `steps`; the context grows by that many); the median of N_REGIONS regions."""
    import numpy as np
    import torch
    from sglang_c_b200.engine import sched_new
    from sglang_c_b200.sampling import SamplingParams
    n_timed = max(steps, 100)
    s = sched_new(model_dir, seed=0, dtype=dtype, page_size=PAGE,
                  max_tokens=batch * (context + n_timed + warmup + 64), max_requests=max(batch, 1),
                  max_step_tokens=PREFILL_TOKENS, prefill_chunk=512)
    V = s.engine.plan.vocab_size
    rng = np.random.default_rng(5)
    sp = SamplingParams(temperature=0.0, ignore_eos=True)
    regions = []
    for _ in range(N_REGIONS):
        ids = [s.submit_ids([int(t) for t in rng.integers(0, V, size=context)], warmup + n_timed + 32, sp)
               for _ in range(batch)]
        while s.waiting or any(r.n_computed < len(r.prompt) for r in s.running):
            s.step()                               # prompts done; every request decodes from here
        for _ in range(warmup):
            s.step()
        torch.cuda.synchronize()
        n0 = s.stats.decode_tokens
        t0 = time.perf_counter()
        for _ in range(n_timed):
            s.step()
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        regions.append((s.stats.decode_tokens - n0) / dt)
        for i in ids:
            s.abort(i)
        while s.poll() is not None:
            pass
    h2d = s.engine.bufs.total * 4 + batch * 40      # the packed step data and the sampling records
    d2h = batch * 4                                 # the sampled token ids
    return statistics.median(regions), h2d, d2h


def time_e2e_c(model_dir, batch, context, steps, warmup, dtype="bfloat16"):
    """The same decode through the Python entry point on the native engine
    (`sched_new(..., native=True)`: the engine behind the C interface csrc/sglc_engine.h): token
    ids on the host in, token ids on the host out, every step; wall clock; regions as time_e2e.
    Returns (tokens a second, bytes up a step, bytes down a step)."""
    import numpy as np
    from sglang_c_b200.engine import sched_new
    from sglang_c_b200.sampling import SamplingParams
    n_timed = max(steps, 100)
    e = sched_new(model_dir, seed=0, dtype=dtype, page_size=PAGE, max_tokens=batch * (context + n_timed + warmup + 64),
                  max_requests=max(batch, 1), max_step_tokens=PREFILL_TOKENS, prefill_chunk=512, native=True)
    V = e.vocab_size
    rng = np.random.default_rng(5)
    sp = SamplingParams(temperature=0.0, ignore_eos=True)
    regions = []
    for _ in range(N_REGIONS):
        ids = [e.submit_ids([int(t) for t in rng.integers(0, V, size=context)], warmup + n_timed + 32, sp)
               for _ in range(batch)]
        while True:                                # prompts done; every request decodes from here
            e.step()
            ran = e.last_step()
            if len(ran) == batch and all(n == 1 for _, n, _ in ran):
                break
        for _ in range(warmup):
            e.step()
        n0 = e.get_stats().decode_tokens
        t0 = time.perf_counter()
        for _ in range(n_timed):
            e.step()                               # returns with the step's ids on the host
        dt = time.perf_counter() - t0
        regions.append((e.get_stats().decode_tokens - n0) / dt)
        for i in ids:
            e.abort(i)
        while e.poll() is not None:
            pass
    up = e.get_stats().step_upload_bytes          # the packed step arrays (greedy records stay on the device)
    e.close()
    return statistics.median(regions), up, (4 + batch) * 4       # down: two error words (padded to four) and the ids


def time_prefill_c(model_dir, n_prompts, prompt_len, warmup=3):
    """One step of n_prompts whole prompts through the C interface, wall clock around the call of
    sglc_engine_step: the host's preparation, the step, the sampling of one token per prompt and
    the ids back on the host.  Median of N_REGIONS regions of at least REGION_MS."""
    import numpy as np
    from sglang_c_b200.engine.c_api import CEngine
    from sglang_c_b200.sampling import SamplingParams
    e = CEngine(model_dir, dtype="bfloat16", page_size=PAGE, max_tokens=n_prompts * (prompt_len + 64),
                max_requests=max(n_prompts, 1), max_step_tokens=n_prompts * prompt_len, prefill_chunk=prompt_len,
                run_ahead=False)              # (the call returns with the step's ids)
    rng = np.random.default_rng(99)
    sp = SamplingParams(temperature=0.0, ignore_eos=True)

    def once():
        for _ in range(n_prompts):
            assert e.submit_ids([int(t) for t in rng.integers(0, e.vocab_size, size=prompt_len)], 1, sp) > 0
        t0 = time.perf_counter()
        done = e.step()
        dt = time.perf_counter() - t0
        assert done == n_prompts
        while e.poll() is not None:
            pass
        return dt * 1e3

    for _ in range(max(warmup, 3)):
        once()
    regions = []
    for _ in range(N_REGIONS):
        ms, n = 0.0, 0
        while ms < REGION_MS:
            ms += once()
            n += 1
        regions.append(ms / n)
    e.close()
    return statistics.median(regions)


def run_mixed_c(model_dir, cfg_d, n_requests=64, max_new=128, seed=0):
    """run_mixed through the engine's C interface."""
    import numpy as np
    from sglang_c_b200.engine.c_api import CEngine
    from sglang_c_b200.sampling import SamplingParams
    rng = np.random.default_rng(seed)
    P = cfg_d["n_positions"]
    lens = [int(n) for n in rng.integers(16, P - max_new + 1, size=n_requests)]
    e = CEngine(model_dir, seed=seed, dtype="bfloat16", page_size=PAGE,
                max_tokens=sum(n + max_new + PAGE for n in lens), max_requests=n_requests,
                max_step_tokens=PREFILL_TOKENS, prefill_chunk=512)
    V = cfg_d["vocab_size"]
    sp = SamplingParams(temperature=0.0, ignore_eos=True)
    prompts = [[int(t) for t in rng.integers(0, V, size=n)] for n in lens]
    e.submit_ids(prompts[0][:64], 4, sp)
    e.run_until_done()
    e.poll()
    t0 = time.perf_counter()
    for p in prompts:
        assert e.submit_ids(p, max_new, sp) > 0
    steps = e.run_until_done()
    dt = time.perf_counter() - t0
    st = e.get_stats()
    gen = n_requests * max_new
    out = {"requests": n_requests, "prompt_tokens": sum(lens), "generated_tokens": gen, "seconds": dt,
           "steps": steps, "generated_tok_s": gen / dt, "total_tok_s": (gen + sum(lens)) / dt,
           "n_preempt": st.n_preempt, "graph_replays": st.graph_replays}
    e.close()
    return out


def run_mixed(model_dir, cfg_d, n_requests=64, max_new=128, seed=0):
    """The mixed workload: requests with uniform random prompt lengths in [16, 1024] and max_new
    greedy tokens each, all submitted at once to the scheduler (continuous batching, prompt
    portions beside decode tokens).  Returns a dict for the JSON line."""
    import numpy as np
    import torch
    from sglang_c_b200.engine import sched_new
    from sglang_c_b200.sampling import SamplingParams
    rng = np.random.default_rng(seed)
    P = cfg_d["n_positions"]
    lens = [int(n) for n in rng.integers(16, P - max_new + 1, size=n_requests)]
    s = sched_new(model_dir, seed=seed, dtype="bfloat16", page_size=PAGE,
                  max_tokens=sum(n + max_new + PAGE for n in lens), max_requests=n_requests,
                  max_step_tokens=PREFILL_TOKENS, prefill_chunk=512)
    V = cfg_d["vocab_size"]
    sp = SamplingParams(temperature=0.0, ignore_eos=True)
    prompts = [[int(t) for t in rng.integers(0, V, size=n)] for n in lens]
    # warm the kernels and a few graph shapes on a throw-away request
    w = s.submit_ids(prompts[0][:64], 4, sp)
    s.run_until_done()
    s.poll()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for p in prompts:
        assert s.submit_ids(p, max_new, sp) > 0
    steps = s.run_until_done()
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    st = s.get_stats()
    gen = n_requests * max_new
    return {"requests": n_requests, "prompt_tokens": sum(lens), "generated_tokens": gen, "seconds": dt,
            "steps": steps, "generated_tok_s": gen / dt, "total_tok_s": (gen + sum(lens)) / dt,
            "n_preempt": st.n_preempt, "graph_replays": s.engine.graph_replays}


def reference_main(args):
    """The reference arm: the unmodified reference's own GPU path on the same workload
    (baseline/reference_arm.py compiles it into baseline/_ref and drives its C API)."""
    if args.gpus != 1:
        print(f"bench.py: the reference runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    sys.path.insert(0, os.path.join(ROOT, "baseline"))
    import reference_arm
    try:
        reference_arm.build()
    except (reference_arm.Unavailable, subprocess.CalledProcessError, OSError) as e:
        print(json.dumps({"impl": "reference", "unavailable":
                          f"the reference could not be compiled here: {str(e).splitlines()[0][:200]}"}))
        return 0
    pk = peaks()
    warmup = max(3, args.warmup)
    steps = max(1, args.steps)
    cfg = SMALL
    try:
        r = reference_arm.run(cfg, BATCH, CONTEXT, steps, warmup, PREFILL_TOKENS, pk,
                              prefill_flops(cfg, 2, PREFILL_TOKENS // 2),
                              lambda elem: model_bytes_flops(cfg, BATCH, CONTEXT + steps // 2, elem, kv_elem=4),
                              clock_sampler=ClockSampler())
    except reference_arm.Unavailable as e:
        print(json.dumps({"impl": "reference", "unavailable": str(e)[:200]}))
        return 0
    out = {
        "impl": "reference",
        "metric": "decode tok/s at batch 8, context 512 (GPT-2 small layer sizes, random weights)",
        "value": r["value"], "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": warmup,
        "ms_per_step": r["ms_per_step"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "fp32", "data": "synthetic: seeded random weights and uniform random token ids",
        "config": {"model": "gpt2-small layer sizes, random weights", "n_layer": cfg["n_layer"],
                   "n_layer_full": cfg["n_layer"], "n_embd": cfg["n_embd"], "n_head": cfg["n_head"],
                   "n_inner": cfg["n_inner"], "vocab_size": cfg["vocab_size"], "n_positions": cfg["n_positions"],
                   "global_batch": BATCH, "seq_len": CONTEXT, "parallelism": "none (1 GPU)",
                   "prefill_tokens": PREFILL_TOKENS, "prefill_shape": "2 prompts x 1024, one forward each",
                   "decode": "one single-token forward per request per step (its GPT-2 decode)",
                   "same_config": "layer sizes and workload equal; its default is float32 weights and cache, "
                                  "fp16_weights is its SGL_CUDA_FP16=1 switch",
                   "timing": "wall clock around its API calls (each ends in its own stream sync)",
                   "peaks": pk["source"]},
        # its API is host tokens in, host logits out, host sampling: the end-to-end number is the number
        "e2e": {"value": r["value"], "unit": "tokens/s", "h2d_bytes_per_step": 4 * BATCH,
                "d2h_bytes_per_step": 4 * cfg["vocab_size"] * BATCH},
        "prefill": dict(r["prefill"], of=pk["source"]),
        "roofline": dict(r["roofline"], of=pk["source"]),
        "points": r["points"], "fp16_weights": r["fp16_weights"], "clocks": r["clocks"],
    }
    print(json.dumps(out))
    return 0


def measure_model(name, base, n_layer, steps, warmup, pk, points=(1, 64), fp32=True, kernels=True):
    """Every figure of one model size: decode at batch 8 (device-timed and end to end), prefill,
    the points, the 32-bit path and the kernel table."""
    import torch
    from sglang_c_b200.engine import Engine
    cfg_d = dict(base, n_layer=n_layer)
    tmp = tempfile.mkdtemp(prefix="sglc_bench_")
    atexit.register(shutil.rmtree, tmp, True)       # the random model is up to 3 GB
    model_dir = make_model(tmp, base, n_layer)
    eng = Engine.from_dir(model_dir, dtype="bfloat16", page_size=PAGE,
                          max_tokens=64 * (CONTEXT + 256), max_requests=64, max_step_tokens=PREFILL_TOKENS)
    time_decode(eng, BATCH, 32, 2, 3)               # every path once (compiles on a fresh checkout)
    r = {}
    pms_loop, _, _ = time_decode(eng, BATCH, CONTEXT, steps, warmup)      # the Python engine's loop
    ms, launches, regions = time_decode_native(model_dir, BATCH, CONTEXT, steps, warmup)
    r.update(ms=ms, launches=launches, regions=regions, value=BATCH / (ms / 1e3))
    r["bytes"] = model_bytes_flops(cfg_d, BATCH, CONTEXT + steps // 2)
    pms = time_prefill(eng, 2, PREFILL_TOKENS // 2, 3)
    pflops = prefill_flops(cfg_d, 2, PREFILL_TOKENS // 2)
    dms = time_prefill(eng, 2, PREFILL_TOKENS // 2, 3, behind_sleep=True)
    r["prefill"] = {"value": PREFILL_TOKENS / (pms / 1e3), "tokens": PREFILL_TOKENS, "ms": pms,
                    "frac": pflops / (pms / 1e3) / (pk["bf16_tflops"] * 1e12), "of": pk["source"],
                    "device_ms": dms, "device_frac": pflops / (dms / 1e3) / (pk["bf16_tflops"] * 1e12)}
    r["points"] = {"decode_b8_python_engine": BATCH / (pms_loop / 1e3)}
    for b in points:
        t, _, _ = time_decode_native(model_dir, b, CONTEXT, steps, warmup)
        r["points"][f"decode_b{b}"] = b / (t / 1e3)
        nb = model_bytes_flops(cfg_d, b, CONTEXT + steps // 2)
        r["points"][f"decode_b{b}_roofline_frac"] = nb / (t / 1e3) / 1e9 / pk["hbm_gbs"]
    if kernels:
        r["kernels"] = kernel_table(eng, BATCH, CONTEXT, PREFILL_TOKENS // 2)
    del eng
    torch.cuda.empty_cache()
    # end to end through the Python entry point: on the native engine (the headline), and on the
    # Python scheduler (the general one)
    r["e2e"] = time_e2e_c(model_dir, BATCH, CONTEXT, steps, warmup)
    r["points"]["e2e_python_scheduler_b8"] = time_e2e(model_dir, BATCH, CONTEXT, steps, warmup)[0]
    # (a request must leave a position for the token it generates: prompts of 1,023 tokens)
    r["points"]["prefill_c_api_tok_s"] = \
        (PREFILL_TOKENS - 2) / (time_prefill_c(model_dir, 2, PREFILL_TOKENS // 2 - 1) / 1e3)
    if fp32:
        # the true 32-bit path (plain FFMA products, 32-bit cache): same step function and scheduler
        eng = Engine.from_dir(model_dir, dtype="float32", page_size=PAGE, max_tokens=BATCH * (CONTEXT + 256) + 4096,
                              max_requests=BATCH, max_step_tokens=PREFILL_TOKENS)
        t, _, _ = time_decode(eng, BATCH, CONTEXT, steps, warmup)
        r["points"]["fp32_decode_b8"] = BATCH / (t / 1e3)
        pm32 = time_prefill(eng, 2, PREFILL_TOKENS // 2, 3)
        r["points"]["fp32_prefill_tok_s"] = PREFILL_TOKENS / (pm32 / 1e3)
        del eng
        torch.cuda.empty_cache()
    r["model_dir"] = model_dir
    return r


def only(kind, base, n_layer, steps, warmup, batch=BATCH):
    """A handful of steps of one kind, each run as its launches (no graph: a profiler then sees
    the kernels in launch order), and one line of JSON with their device time."""
    import numpy as np
    import torch
    from sglang_c_b200.engine import Engine, StepEntry
    tmp = tempfile.mkdtemp(prefix="sglc_bench_")
    atexit.register(shutil.rmtree, tmp, True)
    model_dir = make_model(tmp, base, n_layer)
    dtype = "float32" if kind == "fp32" else "bfloat16"
    eng = Engine.from_dir(model_dir, dtype=dtype, page_size=PAGE, max_tokens=batch * (CONTEXT + 256) + 4096,
                          max_requests=batch, max_step_tokens=PREFILL_TOKENS, use_graphs=False)
    rng = np.random.default_rng(0)
    V = eng.plan.vocab_size
    out = {"only": kind, "n_layer": n_layer, "dtype": dtype, "batch": batch}

    def timed(fn, n):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / n

    if kind in ("prefill", "fp32"):
        it = [0]

        def prefill():
            it[0] += 1
            reqs = [f"p{it[0]}_{i}" for i in range(2)]
            for r in reqs:
                eng.add_request(r)
            eng.step([StepEntry(r, rng.integers(0, V, size=PREFILL_TOKENS // 2).astype(np.int32), [PREFILL_TOKENS // 2 - 1])
                      for r in reqs])
            torch.cuda.synchronize()
            for r in reqs:
                eng.end_request(r)
        timed(prefill, warmup)
        out["prefill_ms_eager"] = timed(prefill, steps)
    if kind in ("decode", "fp32"):
        reqs = [f"d{i}" for i in range(batch)]
        for r in reqs:
            eng.add_request(r)
        done = 0
        while done < CONTEXT:
            n = min(eng.max_step_tokens // batch, CONTEXT - done)
            eng.step([StepEntry(r, rng.integers(0, V, size=n).astype(np.int32), []) for r in reqs])
            done += n

        def decode():
            eng.step([StepEntry(r, [int(rng.integers(0, V))], [0]) for r in reqs])
        timed(decode, warmup)
        out["decode_ms_eager"] = timed(decode, steps)
    print(json.dumps(out))
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=None, help="fewer layers than the configuration (named in config)")
    ap.add_argument("--skip-points", action="store_true")
    ap.add_argument("--model", default="small", choices=sorted(MODELS),
                    help="layer sizes of the headline line: GPT-2 small (the default), medium or xl")
    ap.add_argument("--full", action="store_true",
                    help="also medium and XL layer sizes (decode at batch 8, prefill) and the mixed workload "
                         "(64 requests, prompts of 16..1024 tokens, 128 generated each) under `points`")
    ap.add_argument("--workload", default="decode", choices=["decode", "mixed"],
                    help="decode: the contract's line; mixed: only the mixed workload through the scheduler")
    ap.add_argument("--batch", type=int, default=BATCH, help="with --only decode: requests decoding together")
    ap.add_argument("--only", default=None, choices=["decode", "prefill", "fp32"],
                    help="a handful of steps of one kind and nothing else (what a profiler is pointed at): "
                         "decode steps at batch 8, prefill steps of 2 x 1,024 tokens, or both on the 32-bit path")
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_main(args)
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    warmup = max(3, args.warmup)
    steps = max(1, args.steps)

    pk = peaks()
    base = MODELS[args.model]
    n_layer = args.layers or base["n_layer"]
    if args.only:
        return only(args.only, base, n_layer, steps, warmup, args.batch)
    if args.workload == "mixed":
        tmp = tempfile.mkdtemp(prefix="sglc_bench_")
        atexit.register(shutil.rmtree, tmp, True)
        r = run_mixed(make_model(tmp, base, n_layer), dict(base, n_layer=n_layer))
        print(json.dumps({"metric": "mixed workload: generated tok/s through the scheduler", "value":
                          r["generated_tok_s"], "unit": "tokens/s", "n_gpus": 1, "dtype": "bf16",
                          "data": "synthetic: seeded random weights and uniform random token ids",
                          "config": {"model": f"gpt2-{args.model} layer sizes, random weights",
                                     "n_layer": n_layer, "n_layer_full": base["n_layer"]}, "mixed": r}))
        return 0
    clocks = ClockSampler()
    clocks.start()
    r = measure_model(args.model, base, n_layer, steps, warmup, pk, points=() if args.skip_points else (1, 64))
    points = r["points"]
    if args.full:
        points["mixed_small_generated_tok_s"] = run_mixed(r["model_dir"], dict(base, n_layer=n_layer))["generated_tok_s"]
        points["mixed_small_c_api_generated_tok_s"] = \
            run_mixed_c(r["model_dir"], dict(base, n_layer=n_layer))["generated_tok_s"]
        # other context lengths (the headline's is 512; the model has 1,024 positions)
        for ctx in (128, 960):
            for b in (8, 64):
                t, _, _ = time_decode_native(r["model_dir"], b, ctx, steps, warmup)
                points[f"decode_b{b}_ctx{ctx}"] = b / (t / 1e3)
                nb = model_bytes_flops(dict(base, n_layer=n_layer), b, ctx + steps // 2)
                points[f"decode_b{b}_ctx{ctx}_roofline_frac"] = nb / (t / 1e3) / 1e9 / pk["hbm_gbs"]
        for other in ("medium", "xl"):
            if other == args.model:
                continue
            o = measure_model(other, MODELS[other], MODELS[other]["n_layer"], steps, warmup, pk, points=(1, 64),
                              fp32=(other == "xl"), kernels=False)
            points[f"{other}_decode_b8"] = o["value"]
            points[f"{other}_decode_b8_roofline_frac"] = o["bytes"] / (o["ms"] / 1e3) / 1e9 / pk["hbm_gbs"]
            points[f"{other}_prefill_tok_s"] = o["prefill"]["value"]
            points[f"{other}_prefill_frac"] = o["prefill"]["frac"]
            for k, v in o["points"].items():
                points[f"{other}_{k}"] = v
            if other == "xl":
                points["mixed_xl_generated_tok_s"] = run_mixed(o["model_dir"], MODELS[other])["generated_tok_s"]
            shutil.rmtree(os.path.dirname(o["model_dir"]), True)
    clk = clocks.stop()              # sampled over all the timed regions above
    ms, nbytes = r["ms"], r["bytes"]
    achieved = nbytes / (ms / 1e3) / 1e9
    e2e_value, h2d, d2h = r["e2e"]
    out = {
        "metric": f"decode tok/s at batch 8, context 512 (GPT-2 {args.model} layer sizes, random weights)",
        "value": r["value"], "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": warmup,
        "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: seeded random weights and uniform random token ids",
        "config": {"model": f"gpt2-{args.model} layer sizes, random weights", "n_layer": n_layer,
                   "n_layer_full": base["n_layer"], "n_embd": base["n_embd"], "n_head": base["n_head"],
                   "n_inner": base["n_inner"], "vocab_size": base["vocab_size"],
                   "n_positions": base["n_positions"], "global_batch": BATCH, "seq_len": CONTEXT,
                   "page_size": PAGE, "parallelism": "none (1 GPU)", "prefill_tokens": PREFILL_TOKENS,
                   "prefill_shape": "2 prompts x 1024", "l2": "a step reads more than L2 holds (no flush)",
                   "timing": f"CUDA events; median of {N_REGIONS} regions of >= {REGION_MS:.0f} ms, each chunks of "
                             f"--steps steps", "cuda_graph": "decode step replays a graph",
                   "peaks": pk["source"]},
        "e2e": {"value": e2e_value, "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
        "gpu_launches": r["launches"],
        "prefill": r["prefill"],
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": achieved / pk["hbm_gbs"], "of": pk["source"], "bytes_per_step": nbytes},
        "points": points,
        "region_ms_per_step": [round(x, 5) for x in r["regions"]],
        "kernels": r.get("kernels"),
        "clocks": clk,
    }
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
