"""The programmatic entry points, named after the reference's C interface:
`sgl_sched_new / submit_ids / step / poll / nactive / abort / get_stats`
(include/sgl/scheduler.h:33-67,102) and `sgl_generate` (include/sgl/generate.h:12-17).
Requests are token ids in, token ids out (the tokenizers are not part of this
engine)."""
import time

from ..sampling import SamplingParams
from .engine import Engine
from .scheduler import Scheduler


def sched_new(model_dir, seed=0, dtype="bfloat16", device="cuda:0", page_size=16, n_pages=None,
              max_tokens=None, max_requests=64, max_step_tokens=2048, prefill_chunk=512,
              token_budget=None, want_logprobs=False, native=False):
    """Load a model folder and return a scheduler on top of a fresh engine.
    The cache holds `n_pages` pages of `page_size` positions (or room for
    `max_tokens` positions; by default 64 full-length requests).

    native=True: the engine behind the C interface (csrc/sglc_engine.h) with the same entry
    points (`submit_ids / step / poll / nactive / abort / get_stats / generated /
    run_until_done`): loader, page tables, scheduler, step arrays, graphs and sampler in C++, for
    architectures made of the built-in parts; the same ids, a few percent faster end to end.
    The default is the Python engine, the general one (parts registered from outside)."""
    if native:
        from .c_api import CEngine
        return CEngine(model_dir, seed=seed, dtype=dtype, device=device, page_size=page_size, n_pages=n_pages,
                       max_tokens=max_tokens, max_requests=max_requests, max_step_tokens=max_step_tokens,
                       prefill_chunk=prefill_chunk, token_budget=token_budget, want_logprobs=want_logprobs)
    if n_pages is None and max_tokens is None:
        from ..config.registry import load_config
        arch, cfg = load_config(model_dir)
        max_tokens = max_requests * arch.build_plan(cfg).max_positions
    eng = Engine.from_dir(model_dir, dtype=dtype, device=device, page_size=page_size, n_pages=n_pages,
                          max_tokens=max_tokens, max_requests=max_requests,
                          max_step_tokens=max_step_tokens)
    return Scheduler(eng, seed=seed, prefill_chunk=prefill_chunk, token_budget=token_budget,
                     want_logprobs=want_logprobs)


def sched_submit_ids(s, ids, max_new=16, sp=None):
    return s.submit_ids(ids, max_new, sp)


def sched_step(s):
    return s.step()


def sched_poll(s):
    return s.poll()


def sched_nactive(s):
    return s.nactive()


def sched_abort(s, req_id):
    return s.abort(req_id)


def sched_get_stats(s):
    return s.get_stats()


def generate(s, prompts, sp=None, max_new=16, on_token=None):
    """Generate for one prompt (a list of ids) or several (a list of lists) and
    return the generated ids in the same form.  `on_token(request_index, token)`
    is called for every new token, like the reference's callback
    (src/generate.c:43-55)."""
    single = bool(prompts) and isinstance(prompts[0], int)
    batch = [prompts] if single else list(prompts)
    sps = sp if isinstance(sp, (list, tuple)) else [sp] * len(batch)
    ids = []
    for p, q in zip(batch, sps):
        rid = s.submit_ids(p, max_new, q or SamplingParams())
        if rid < 0:
            raise ValueError("a prompt was refused: empty, ids outside the vocabulary, "
                             "or prompt + max_new beyond the cache pool or the model's positions")
        ids.append(rid)
    seen = {rid: 0 for rid in ids}
    while s.nactive() > 0:
        s.step()
        if on_token is not None:
            for i, rid in enumerate(ids):
                g = s.generated(rid) or []
                while seen[rid] < len(g):
                    on_token(i, g[seen[rid]])
                    seen[rid] += 1
    out = {}
    while True:
        got = s.poll()
        if got is None:
            break
        out[got[0]] = got[1]
    res = [out[rid] for rid in ids]
    return res[0] if single else res
