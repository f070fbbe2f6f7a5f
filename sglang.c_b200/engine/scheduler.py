"""Continuous-batching scheduler above the step function.

The reference's scheduler (src/scheduler.c) runs, per step, either one prompt
chunk of one request or a decode batch of all running requests (:454-523),
takes all of a request's pages at admission (:337-368) and preempts by
recomputation when admission finds no pages (:429-452).  This one keeps its
request states, finishing rules, statistics and entry-point names, and differs
where the engine allows more:

  * a step is mixed: first one token for every running request that is past its
    prompt, then prompt portions (at most `prefill_chunk` tokens each) of
    requests still in their prompt and of newly admitted ones, until the
    step's token budget is full;
  * pages are taken as a request grows, not at admission;
  * when a step's tokens need more pages than are free, requests are preempted
    from the latest arrival backwards until the rest fits: a preempted request
    gives back its pages and its slot, keeps the tokens it has generated and
    its random stream, and waits; when readmitted it recomputes prompt plus
    generated tokens and continues, so its output does not change.  Admission
    never preempts: a waiting request is admitted only into free pages and a
    free slot, which rules out two requests evicting each other in turn.
  * a request whose prompt plus max_new can never fit the pool or the model's
    positions is refused at submit (the reference: src/scheduler.c:818-825).
"""
import time
from collections import deque
from dataclasses import dataclass, field
from typing import List, Optional

import numpy as np

from .. import log
from ..sampling import Sampler, SamplingParams, request_stream, uniform
from .engine import Engine, OutOfPages
from .step import StepEntry

WAITING, RUNNING, DONE = "waiting", "running", "done"
KEEP_TAKEN = 256       # taken requests whose record is kept for questions after poll()


@dataclass
class Request:
    id: int
    prompt: List[int]
    prompt_arr: object           # the prompt as an int32 array (portions of it go to the engine as views)
    max_new: int
    sp: SamplingParams
    rng: int
    state: str = WAITING
    gen: List[int] = field(default_factory=list)
    logprobs: List[float] = field(default_factory=list)
    n_computed: int = 0          # tokens of prompt+gen that are in the cache
    n_preempted: int = 0
    finish_reason: Optional[str] = None
    taken: bool = False

    @property
    def tokens(self):
        return self.prompt + self.gen

    @property
    def n_pending(self):
        return len(self.prompt) + len(self.gen) - self.n_computed


@dataclass
class SchedStats:
    """The reference's counters (include/sgl/scheduler.h:19-31) that apply here."""
    prefill_tokens: int = 0
    decode_tokens: int = 0
    n_finished: int = 0
    n_running: int = 0
    n_waiting: int = 0
    pool_pages: int = 0
    pool_free: int = 0
    n_preempt: int = 0
    prefill_chunk: int = 0
    n_steps: int = 0
    recomputed_tokens: int = 0


class Scheduler:
    def __init__(self, engine: Engine, seed=0, prefill_chunk=512, token_budget=None,
                 eos_token_id="from_model", want_logprobs=False, sampler=None):
        self.engine = engine
        self.seed = int(seed)
        # the reference: SGL_PREFILL_CHUNK, default 512, <= 0 means 4096 (src/scheduler.c:138-143)
        self.prefill_chunk = int(prefill_chunk) if prefill_chunk and prefill_chunk > 0 else 4096
        self.token_budget = min(int(token_budget or engine.max_step_tokens), engine.max_step_tokens)
        self.eos_token_id = engine.plan.eos_token_id if eos_token_id == "from_model" else eos_token_id
        self.want_logprobs = want_logprobs
        self.requests = {}
        self.waiting: List[Request] = []     # FIFO, preempted requests re-enter by arrival order
        self.running: List[Request] = []     # in order of arrival
        # finished and not yet taken by poll(); a taken request stays in `requests` (for its
        # log-probabilities and finish reason) until KEEP_TAKEN later ones have been taken
        # (the reference frees a taken request at once, src/scheduler.c:577-615)
        self.done = deque()
        self._taken = deque()
        self.next_id = 1
        self.stats = SchedStats(prefill_chunk=self.prefill_chunk, pool_pages=engine.cache.n_pages)
        # any object with Sampler.sample's signature; the default samples on the device
        self.sampler = sampler if sampler is not None else Sampler(engine.rt.device, engine.max_requests)
        # prepare the next step of single tokens on the host while the device runs this one
        # (only engines that offer it: Engine.prepare_repeat)
        # a step's ids are read one call later (see step): needs the engine's prepared steps
        # and a sampler that can be launched without waiting
        self.lagging = hasattr(engine, "prepare_repeat") and hasattr(self.sampler, "launch") \
            and hasattr(self.sampler, "fetch")
        self._ahead = None               # ids of the requests the engine holds a prepared step for
        self._flight = None              # (requests sampled, sampler ticket) of the step not yet read

    # -- entry points (names of the reference's C interface) --------------------
    def submit_ids(self, ids, max_new=16, sp=None):
        """Queue a request given as token ids; returns its id (from 1 up), or -1
        if it can never run."""
        ids = [int(t) for t in ids]
        max_new = int(max_new) if max_new and max_new > 0 else 16     # src/scheduler.c:193
        plan, cache = self.engine.plan, self.engine.cache
        if not ids or any(not (0 <= t < plan.vocab_size) for t in ids):
            return -1
        need = len(ids) + max_new
        if len(ids) >= plan.max_positions:
            return -1
        pool_tokens = cache.n_pages * cache.page_size
        if min(need, plan.max_positions) > pool_tokens:
            return -1
        sp = sp or SamplingParams()
        r = Request(self.next_id, ids, np.asarray(ids, dtype=np.int32), max_new, sp,
                    request_stream(self.seed ^ sp.seed, self.next_id))
        self.next_id += 1
        self.requests[r.id] = r
        self.waiting.append(r)
        return r.id

    def nactive(self):
        return len(self.waiting) + len(self.running)

    def poll(self):
        """One finished request not yet taken: (id, generated ids, n_prompt), or None."""
        if not self.done:
            return None
        r = self.done.popleft()
        r.taken = True
        self._taken.append(r.id)
        while len(self._taken) > KEEP_TAKEN:
            self.requests.pop(self._taken.popleft(), None)
        return r.id, list(r.gen), len(r.prompt)

    def generated(self, req_id):
        """What the request has generated so far (running, or finished and kept), or None."""
        r = self.requests.get(req_id)
        return list(r.gen) if r is not None else None

    def poll_logprobs(self, req_id):
        r = self.requests.get(req_id)
        return list(r.logprobs) if r is not None else None

    def abort(self, req_id):
        r = self.requests.get(req_id)
        if r is None or r.state == DONE:
            return -1
        if r.state == RUNNING:
            self.engine.end_request(r.id)
            self.running.remove(r)
        else:
            self.waiting.remove(r)
        self._finish(r, "abort", free=False)
        return 0

    def get_stats(self):
        s = self.stats
        s.n_running, s.n_waiting = len(self.running), len(self.waiting)
        s.pool_free = self.engine.cache.n_free_pages()
        return s

    # -- one step -----------------------------------------------------------------
    def _finish(self, r, reason, free=True):
        if free and self.engine.has_request(r.id):
            self.engine.end_request(r.id)
        r.state = DONE
        r.finish_reason = reason
        self.done.append(r)
        self.stats.n_finished += 1

    def _preempt(self, r):
        log.debug(f"pages short: request {r.id} gives back {r.n_computed} positions and waits")
        self.engine.end_request(r.id)
        self.running.remove(r)
        self.stats.recomputed_tokens += r.n_computed
        r.n_computed = 0
        r.n_preempted += 1
        r.state = WAITING
        self.stats.n_preempt += 1
        # back into the queue by arrival order, so it is readmitted before later arrivals
        i = 0
        while i < len(self.waiting) and self.waiting[i].id < r.id:
            i += 1
        self.waiting.insert(i, r)

    def plan_step(self):
        """Decide the step: returns the list of (request, n_tokens).  Preempts as
        needed; admits waiting requests into free pages and slots."""
        eng, cache = self.engine, self.engine.cache
        budget = self.token_budget
        chosen = []          # (request, n)
        # 1. one token for every running request past its prompt, then portions of those in it
        for r in self.running:
            if r.n_pending == 1 and r.n_computed > 0 and budget > 0:
                chosen.append((r, 1))
                budget -= 1
        for r in self.running:
            if not (r.n_pending == 1 and r.n_computed > 0) and budget > 0:
                n = min(r.n_pending, self.prefill_chunk, budget)
                chosen.append((r, n))
                budget -= n
        # 2. preempt from the latest arrival backwards until the chosen tokens fit
        preempted = False
        while chosen:
            wants = [(r.id, r.n_computed + n) for r, n in chosen]
            if cache.can_extend_all(wants):
                break
            victim = max(self.running, key=lambda q: q.id)
            chosen = [(r, n) for r, n in chosen if r is not victim]
            self._preempt(victim)
            preempted = True
        # 3. admit waiting requests, first come first served, into what is free: never in a
        #    step that had to preempt, and only if all the request holds so far fits now
        while self.waiting and budget > 0 and cache.n_free_slots() > 0 and not preempted:
            r = self.waiting[0]
            n = min(r.n_pending, self.prefill_chunk, budget)
            eng.add_request(r.id)
            wants = [(q.id, q.n_computed + m) for q, m in chosen] + [(r.id, r.n_pending)]
            if not cache.can_extend_all(wants):
                eng.end_request(r.id)
                break
            self.waiting.pop(0)
            r.state = RUNNING
            self.running.append(r)
            self.running.sort(key=lambda q: q.id)
            chosen.append((r, n))
            budget -= n
        return chosen

    def step(self):
        """Run one step; returns how many requests finished in this call.

        With the device sampler and an engine that can prepare a step ahead, a step's sampled
        ids are read one call later: a call first queues the next step of single tokens behind
        the step in flight (its ids pass from the sampler to the embedding on the device), then
        waits for the ids of the step in flight and appends them, then prepares the step after
        on the host.  So the device always has the next step queued while the host does its
        bookkeeping.  Whatever changes the set of running requests (one ends, is aborted,
        arrives) makes the next call take the plain path: wait, plan, launch.  A request that
        ends while a step with it is already queued has that step's id dropped."""
        flight, self._flight = self._flight, None
        nxt = None
        if flight is not None and self._ahead is not None:
            ahead, self._ahead = self._ahead, None
            if self.engine.has_prepared() and not self.waiting and ahead == [r.id for r in self.running]:
                # queued without having seen the ids of the step in flight
                sampled = list(self.running)
                logits = self.engine.run_prepared(device_tokens=self.sampler.d_out)
                for r in sampled:
                    r.n_computed += 1
                self.stats.n_steps += 1
                nxt = (sampled, self._launch_sampler(logits, sampled), [r.n_computed for r in sampled])
            else:
                self.engine.cancel_prepared()
        finished = self._collect(flight) if flight is not None else 0
        if nxt is None:
            if self._ahead is not None:          # (prepared in the last call, and not usable after all)
                self._ahead = None
                self.engine.cancel_prepared()
            chosen = self.plan_step()
            if not chosen:
                return finished
            entries, sampled = [], []
            for r, n in chosen:
                np_ = len(r.prompt)
                if r.n_computed >= np_:                   # past the prompt: no need to join the lists
                    toks = r.gen[r.n_computed - np_:r.n_computed - np_ + n]
                elif r.n_computed + n <= np_:             # inside the prompt: a view of its array
                    toks = r.prompt_arr[r.n_computed:r.n_computed + n]
                else:
                    toks = r.tokens[r.n_computed:r.n_computed + n]
                last = (r.n_computed + n == np_ + len(r.gen))
                entries.append(StepEntry(r.id, toks, [n - 1] if last else []))
                if last:
                    sampled.append(r)
                if r.n_computed + n <= np_:
                    self.stats.prefill_tokens += n
            logits = self.engine.step(entries)
            for r, n in chosen:
                r.n_computed += n
            self.stats.n_steps += 1
            nxt = (sampled, self._launch_sampler(logits, sampled) if sampled else None,
                   [r.n_computed for r in sampled])
        sampled = nxt[0]
        if not self.lagging:
            # results in the same call (a sampler or an engine that cannot run ahead)
            return finished + self._collect(nxt)
        self._flight = nxt
        # While the device runs the step just queued: if every running request is sampled in it,
        # none waits and none can end by its length, the step after brings one token for each of
        # them, and all of it but the ids is prepared now.  (A request that ends meanwhile ends
        # the preparation with it: Engine.end_request cancels.)
        if not self.waiting and sampled and len(sampled) == len(self.running) \
                and all(len(r.gen) + 1 < r.max_new and not r.sp.has_penalties() for r in sampled):
            ids = [r.id for r in self.running]
            if self.engine.prepare_repeat(ids):
                self._ahead = ids
        return finished

    def _launch_sampler(self, logits, sampled):
        us = []
        for r in sampled:
            if r.sp.greedy:
                us.append(0.0)
            else:
                r.rng, u = uniform(r.rng)
                us.append(u)
        args = (logits, [r.sp for r in sampled], us)
        kw = dict(histories=[r.gen for r in sampled], want_logprobs=self.want_logprobs)
        if self.lagging:
            return self.sampler.launch(*args, **kw)
        return self.sampler.sample(*args, **kw)          # a sampler without launch/fetch: results at once

    def _collect(self, flight):
        """Take a step's sampled ids and append them; returns how many requests ended."""
        sampled, ticket, n_after = flight
        if not sampled:
            return 0
        out = self.sampler.fetch(ticket) if self.lagging else ticket
        toks, lps = out if self.want_logprobs else (out, None)
        finished = 0
        for i, r in enumerate(sampled):
            if r.state != RUNNING:
                continue                 # ended or aborted after this step was queued: its id is dropped
            if self._append(r, toks[i], lps[i] if lps else None, n_after[i]):
                finished += 1
        return finished

    def _append(self, r, tok, logprob, n_computed):
        """The reference's req_sample_append (src/scheduler.c:288-310): eos or a
        stop id ends the request without being appended; then max_new and the
        model's positions.  n_computed: the request's tokens in the cache after the step
        that gave `tok` (a later step may be queued already)."""
        if tok == self.eos_token_id and self.eos_token_id is not None and not r.sp.ignore_eos:
            self.running.remove(r)
            self._finish(r, "eos")
            return True
        if r.sp.is_stop(tok):
            self.running.remove(r)
            self._finish(r, "stop")
            return True
        r.gen.append(int(tok))
        if logprob is not None:
            r.logprobs.append(logprob)
        self.stats.decode_tokens += 1
        if len(r.gen) >= r.max_new:
            self.running.remove(r)
            self._finish(r, "length")
            return True
        if n_computed + 1 >= self.engine.plan.max_positions:
            self.running.remove(r)
            self._finish(r, "context")
            return True
        return False

    def run_until_done(self, max_steps=1000000):
        steps = 0
        while self.nactive() > 0 and steps < max_steps:
            self.step()
            steps += 1
        return steps
