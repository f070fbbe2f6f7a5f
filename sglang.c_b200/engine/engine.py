"""The engine core: model, cache and the one step function.

`Engine.step(entries)` takes a batch of (request, its next tokens, wanted
places): portions of prompts beside single decoded tokens, cut anywhere.  It
runs only the tokens it is given, as one batch, against what earlier steps left
in the cache, and returns the logits at the wanted places.
"""
import numpy as np
import torch

from ..cache import CacheManager
from ..config.registry import load_config
from .model import Model
from .runtime import Runtime
from .step import GroupStep, StepBuffers, StepContext, StepEntry, Workspace


_ORDER_SPREAD = 64      # keys (one stage of the streaming decode attention)


def _spread(lens):
    """Whether the contexts of a step differ enough for their order to matter."""
    return len(lens) > 1 and max(lens) - min(lens) >= _ORDER_SPREAD


class StepError(ValueError):
    """A step that cannot run as asked (bad ids, unknown request, too many tokens)."""


class OutOfPages(RuntimeError):
    """The step needs more pages than are free.  Nothing was run or changed."""


class Engine:
    def __init__(self, plan, runtime, page_size=16, n_pages=None, max_tokens=None, max_requests=64,
                 max_step_tokens=2048, model_dir=None, use_graphs=True, use_host_walker=True):
        self.rt = runtime
        self.plan = plan
        self.model = Model(plan, runtime)
        if model_dir is not None:
            self.model.load(model_dir)
        if n_pages is None:
            if max_tokens is None:
                raise ValueError("give n_pages or max_tokens to size the cache")
            n_pages = (int(max_tokens) + page_size - 1) // page_size
        self.page_size = int(page_size)
        self.max_requests = int(max_requests)
        self.max_step_tokens = int(max_step_tokens)
        needs, cache_of = self.model.cache_needs()
        self.cache = CacheManager(needs, cache_of, self.page_size, n_pages, self.max_requests,
                                  make_tensor=runtime.make_tensor, cache_dtype=runtime.cache_dtype_name)
        self.b_cap = (plan.max_positions + self.page_size - 1) // self.page_size
        self._paged = self.cache.paged_groups()
        self._any_window = any(self.cache.groups[gi].need.window is not None for gi in self._paged)
        self._rep = None                  # what a repeated step of single tokens updates in place
        self._poisoned = set()            # requests a failed step left with positions never computed
        self._prepared = None             # prepare_repeat's mark: indices of requests that took a page
        self.bufs = StepBuffers(runtime.device, self.max_step_tokens, self.max_requests, self.b_cap,
                                len(self.cache.groups))
        self.err_flag = torch.zeros(1, dtype=torch.int32, device=runtime.device)
        self.ws = Workspace(runtime.device, self._workspace_bytes())
        self.logits = None
        from ..csrc import ops as _ops
        self._few_max_weight = _ops.FEW_MAX_WEIGHT
        self.max_graphs = 48
        self.steps_run = 0
        # steps whose launch shapes repeat replay a CUDA graph (see _forward_graphed)
        self.use_graphs = bool(use_graphs)
        self._graphs = {}
        self._graph_seen = set()
        self.graph_replays = 0
        # a model of built-in parts has its launches made by the C++ walker (engine/host_model.py);
        # any other model, and use_host_walker=False, keep the Python forward pass
        self.use_host_walker = bool(use_host_walker)
        self._host = None
        self._host_tried = False

    # -- construction ---------------------------------------------------------
    @classmethod
    def from_dir(cls, model_dir, dtype="bfloat16", device="cuda:0", **kw):
        arch, cfg = load_config(model_dir)
        plan = arch.build_plan(cfg)
        eng = cls(plan, Runtime(dtype, device), model_dir=model_dir, **kw)
        eng.config = cfg
        eng.architecture = arch
        return eng

    def _workspace_bytes(self):
        # what the parts say they take per token, rounded up for the 256-byte alignment of each
        # of a layer's handful of buffers, plus room for a few rows of odds and ends
        return int(self.model.workspace_per_token() * 1.02) * self.max_step_tokens + (8 << 20)

    def _logits_buffer(self, n):
        if self.logits is None or self.logits.shape[0] < n:
            cap = max(n, self.max_requests, min(self.max_step_tokens, 64))
            self.logits = torch.empty((cap, self.plan.vocab_size), dtype=torch.float32,
                                      device=self.rt.device)
        return self.logits

    # -- requests ---------------------------------------------------------------
    def add_request(self, req):
        self.cancel_prepared()
        self._rep = None
        slot = self.cache.add_request(req)
        if slot is None:
            raise StepError(f"all {self.max_requests} request slots are taken")
        return slot

    def end_request(self, req):
        self.cancel_prepared()
        self._rep = None
        self._poisoned.discard(req)
        self.cache.free_request(req)

    def truncate(self, req, new_len):
        """Forget what the request holds beyond new_len positions (pages filled by that alone go
        back to the pool); the next step for it continues from there."""
        self.cancel_prepared()
        self._rep = None
        self.cache.truncate(req, new_len)

    def has_request(self, req):
        return self.cache.has_request(req)

    def length(self, req):
        return self.cache.length(req)

    # -- the step ---------------------------------------------------------------
    def _validate(self, entries):
        seen = set()
        T = 0
        V, P = self.plan.vocab_size, self.plan.max_positions
        for e in entries:
            if e.req in seen:
                raise StepError(f"request {e.req!r} appears twice in one step")
            seen.add(e.req)
            if not self.cache.has_request(e.req):
                raise StepError(f"request {e.req!r} is not live (add_request first)")
            if e.req in self._poisoned:
                raise StepError(f"request {e.req!r} was left half-grown by a step that failed and could not be "
                                "rolled back (its window had released pages); end it")
            n = len(e.tokens)
            if n == 0:
                raise StepError(f"request {e.req!r} brings no tokens")
            if n == 1:
                bad = not (0 <= int(e.tokens[0]) < V)
            else:
                # a portion is made an array once, here (a list of a thousand ids costs 35 us to
                # convert; the packed block below takes the array)
                arr = e.tokens if isinstance(e.tokens, np.ndarray) else np.asarray(e.tokens)
                e.tokens = arr
                bad = bool(arr.min() < 0 or arr.max() >= V)
            if bad:
                t = next(t for t in e.tokens if not (0 <= int(t) < V))
                raise StepError(f"request {e.req!r}: token id {t} is outside the vocabulary of {V}")
            if self.cache.length(e.req) + n > P:
                raise StepError(f"request {e.req!r} would reach {self.cache.length(e.req) + n} positions; "
                                f"the model has {P}")
            for w in e.want:
                if not (0 <= int(w) < n):
                    raise StepError(f"request {e.req!r}: wanted place {w} is outside its {n} tokens")
            T += n
        if T > self.max_step_tokens:
            raise StepError(f"step of {T} tokens exceeds max_step_tokens={self.max_step_tokens}")
        if len(entries) > self.max_requests:
            raise StepError(f"step of {len(entries)} requests exceeds max_requests={self.max_requests}")
        return T

    def pages_available_for(self, wants):
        return self.cache.can_extend_all(wants)

    def step(self, entries):
        """entries: list of StepEntry (or (req, tokens, want) tuples).  Returns a
        float32 device tensor [n_wanted, vocab]: the logits at the wanted
        places, in the order of the entries and of each `want`.  The tensor is
        a view of a buffer that the next step overwrites."""
        entries = [e if isinstance(e, StepEntry) else StepEntry(*e) for e in entries]
        V = self.plan.vocab_size
        if not entries:
            return torch.empty((0, V), dtype=torch.float32, device=self.rt.device)
        if self._rep is not None:
            ctx = self._step_repeat(entries, self._rep)
            if ctx is not None:
                return self._run_or_roll_back(ctx, ctx.h_reqs, [n - 1 for n in ctx.h_kv_len])
            self.cancel_prepared()           # prepared for another step than this one
        T = self._validate(entries)
        wants = [(e.req, self.cache.length(e.req) + len(e.tokens)) for e in entries]
        if not self.cache.can_extend_all(wants):
            raise OutOfPages(f"step needs more pages than the {self.cache.n_free_pages()} free ones")
        old_len = [self.cache.length(e.req) for e in entries]
        for (req, new_len) in wants:
            ok = self.cache.extend(req, new_len)
            assert ok, "extend failed after can_extend_all"

        b = self.bufs
        b.wait_host_free()
        R = len(entries)
        tok, pos, trq, wr = b.npview("tokens"), b.npview("positions"), b.npview("token_req"), b.npview("want_rows")
        qs, kl, ss = b.npview("q_start"), b.npview("kv_len"), b.npview("state_slots")
        dtk = b.npview("decode_tokens")
        n_decode = 0
        paged = [(gi, b.npview(f"slots{gi}"), b.npview(f"bt{gi}").reshape(self.max_requests, self.b_cap))
                 for gi in self._paged]
        ps = self.page_size
        ctx = StepContext(self.rt, self.ws)
        t0 = 0
        nw = 0
        max_keys = 0
        for r, e in enumerate(entries):
            n = len(e.tokens)
            o = old_len[r]
            slot = self.cache.slot(e.req)
            if n == 1:
                tok[t0] = e.tokens[0]
                pos[t0] = o
                trq[t0] = r
                dtk[n_decode] = t0
                n_decode += 1
            else:
                tok[t0:t0 + n] = e.tokens
                pos[t0:t0 + n] = np.arange(o, o + n, dtype=np.int32)
                trq[t0:t0 + n] = r
            qs[r] = t0
            kl[r] = o + n
            ss[r] = slot
            for w in e.want:
                wr[nw] = t0 + int(w)
                nw += 1
            for gi, sl, bt in paged:
                table = self.cache.block_table(gi, e.req)
                bt[r, :len(table)] = table
                if n == 1:
                    sl[t0] = table[o // ps] * ps + o % ps
                else:
                    p = np.arange(o, o + n, dtype=np.int64)
                    sl[t0:t0 + n] = np.asarray(table, dtype=np.int64)[p // ps] * ps + p % ps
            ctx.h_q_len.append(n)
            ctx.h_kv_len.append(o + n)
            ctx.h_fresh.append(o == 0)
            ctx.h_reqs.append(e.req)
            ctx.h_state_slots.append(slot)
            if o + n > max_keys:
                max_keys = o + n
            if n > ctx.max_q_len:
                ctx.max_q_len = n
            t0 += n
        qs[R] = t0
        if n_decode > 1:
            # single tokens in the order of their contexts, longest first: the decode attention
            # deals its blocks long and short ones alike
            d = dtk[:n_decode].copy()
            dtk[:n_decode] = d[np.argsort(-pos[d], kind="stable")]
        b.upload()

        ctx.T, ctx.R, ctx.n_want, ctx.max_keys = T, R, nw, max_keys
        ctx.n_decode = n_decode
        ctx.decode_ordered = n_decode == T and _spread(ctx.h_kv_len)
        # a step of single tokens is likely to come again with the same requests: keep what
        # the next one can update in place
        self._rep = None
        if n_decode == R and not self._any_window:
            self._rep = dict(reqs=[e.req for e in entries], want=[list(e.want) for e in entries],
                             lens=np.asarray(ctx.h_kv_len, dtype=np.int64), slots=list(ctx.h_state_slots), nw=nw)
        return self._run_or_roll_back(ctx, [e.req for e in entries], old_len)

    def _run_or_roll_back(self, ctx, reqs, old_len):
        """_run; if it raises (a shape a kernel refuses, a failed launch), the requests were grown
        for tokens whose keys and values were never written: the growth is taken back, so that no
        later step attends to what happens to lie in those pages."""
        try:
            return self._run(ctx)
        except Exception:
            self._rep = None
            for req, o in zip(reqs, old_len):
                try:
                    self.cache.truncate(req, int(o))
                except Exception:
                    self._poisoned.add(req)
            raise

    def _step_repeat(self, entries, rep):
        """The step after a step of single tokens, for the same requests in the same order with
        the same wanted places: the packed arrays of the last step are updated in place
        (positions and lengths grow by one; a cache slot is the next one unless a page begins)
        instead of being built again.  Returns None, having changed nothing, when the step is
        of another kind or not valid (the general path then words the error)."""
        R = len(entries)
        reqs = rep["reqs"]
        if R != len(reqs):
            return None
        want = rep["want"]
        for r, e in enumerate(entries):
            if e.req != reqs[r] or len(e.tokens) != 1 or list(e.want) != want[r]:
                return None
        toks = np.fromiter((e.tokens[0] for e in entries), dtype=np.int64, count=R)
        if toks.min() < 0 or toks.max() >= self.plan.vocab_size:
            return None
        if self._prepared is None and not self.prepare_repeat(reqs):
            return None
        return self._finish_prepared(toks)

    def prepare_repeat(self, reqs):
        """Everything of the next step that does not depend on its token ids, done ahead (while
        the device still runs the last step): valid when the next step brings one token for each
        of `reqs`, the requests of the last step in the same order.  Grows the requests in the
        cache and updates the packed arrays on the host.  Returns False, having changed nothing,
        if the last step was of another kind, a request would pass the model's positions, or
        pages are short.  Followed by run_prepared(tokens) or cancel_prepared()."""
        rep = self._rep
        if rep is None or self._prepared is not None or list(reqs) != rep["reqs"]:
            return False
        R = len(rep["reqs"])
        o = rep["lens"]
        if int(o.max()) + 1 > self.plan.max_positions:
            return False
        ps = self.page_size
        cross = np.nonzero(o % ps == 0)[0]
        if len(cross) and not self.cache.can_extend_all([(rep["reqs"][r], int(o[r]) + 1) for r in cross]):
            return False
        crossed = set(int(r) for r in cross)
        self.cache.grow_by_one(rep["reqs"], crossed)
        b = self.bufs
        b.wait_host_free()
        b.npview("positions")[:R] = o
        b.npview("kv_len")[:R] = o + 1
        for gi in self._paged:
            sl = b.npview(f"slots{gi}")
            sl[:R] += 1
            if len(cross):
                bt = b.npview(f"bt{gi}").reshape(self.max_requests, self.b_cap)
                for r in cross:
                    blk = int(o[r]) // ps
                    page = self.cache.block_table(gi, rep["reqs"][r])[blk]
                    bt[r, blk] = page
                    sl[r] = page * ps
        self._prepared = crossed
        return True

    def has_prepared(self):
        return self._prepared is not None

    def run_prepared(self, tokens=None, device_tokens=None):
        """Run the step that prepare_repeat set up, with these token ids (one per request): a
        list on the host, or an int32 device tensor whose first entries are the ids in request
        order (what a sampler left on the device: the step is then queued without the host
        having seen them; ids outside the vocabulary raise the embedding kernel's error flag)."""
        if self._prepared is None:
            raise StepError("no prepared step (prepare_repeat first)")
        R = len(self._rep["reqs"])
        if device_tokens is not None:
            if device_tokens.dtype != torch.int32 or device_tokens.numel() < R or not device_tokens.is_cuda:
                self.cancel_prepared()
                raise StepError("run_prepared: device_tokens must be an int32 device tensor of one id per request")
            ctx = self._finish_prepared(None)
            self.bufs.dview("tokens", R).copy_(device_tokens[:R], non_blocking=True)
            return self._run_or_roll_back(ctx, ctx.h_reqs, [n - 1 for n in ctx.h_kv_len])
        toks = np.asarray(tokens, dtype=np.int64)
        if toks.shape != (R,) or toks.min() < 0 or toks.max() >= self.plan.vocab_size:
            self.cancel_prepared()
            raise StepError("run_prepared: one token id inside the vocabulary for each request")
        ctx = self._finish_prepared(toks)
        return self._run_or_roll_back(ctx, ctx.h_reqs, [n - 1 for n in ctx.h_kv_len])

    def cancel_prepared(self):
        """Undo prepare_repeat: the requests shrink back by one position, pages taken for them
        return to the pool.  The next step is built in full."""
        if self._prepared is None:
            return
        self.cache.shrink_by_one(self._rep["reqs"], self._prepared)
        self._prepared = None
        self._rep = None

    def _finish_prepared(self, toks):
        rep = self._rep
        R = len(rep["reqs"])
        o = rep["lens"]
        b = self.bufs
        if toks is not None:
            b.npview("tokens")[:R] = toks
        b.upload()
        self._prepared = None
        rep["lens"] = o + 1
        ctx = StepContext(self.rt, self.ws)
        ctx.repeating = True             # steady decoding: a new launch shape is captured at once
        ctx.T, ctx.R, ctx.n_want, ctx.n_decode = R, R, rep["nw"], R
        ctx.max_keys = int(o.max()) + 1
        ctx.decode_ordered = int(o.max()) - int(o.min()) >= _ORDER_SPREAD
        ctx.max_q_len = 1
        ctx.h_q_len = [1] * R
        ctx.h_kv_len = (o + 1).tolist()
        ctx.h_fresh = [False] * R
        ctx.h_reqs = list(rep["reqs"])
        ctx.h_state_slots = rep["slots"]
        return ctx

    def _run(self, ctx):
        """Run the model on a step whose packed arrays are on their way to the device."""
        b = self.bufs
        T, R, nw, n_decode = ctx.T, ctx.R, ctx.n_want, ctx.n_decode
        if self.use_graphs and self.model.graph_safe:
            # a step whose launch shapes have a captured graph needs nothing but the upload above
            hit = self._graph_lookup(ctx)
            if hit is not None:
                self.steps_run += 1
                return hit
        ctx.decode_tokens = b.dview("decode_tokens", max(n_decode, 1))
        ctx.tokens, ctx.positions = b.dview("tokens", T), b.dview("positions", T)
        ctx.token_req, ctx.want_rows = b.dview("token_req", T), b.dview("want_rows", max(nw, 1))
        ctx.q_start, ctx.kv_len = b.dview("q_start", R + 1), b.dview("kv_len", R)
        ctx.state_slots = b.dview("state_slots", R)
        ctx.err_flag = self.err_flag
        ctx.few_token_ok = 0 < self.model.largest_layer_matrix <= self._few_max_weight
        ctx.groups = []
        for gi in range(len(self.cache.groups)):
            if gi in self._paged:
                ctx.groups.append(GroupStep(b.dview(f"bt{gi}").view(self.max_requests, self.b_cap),
                                            b.dview(f"slots{gi}", T), self.page_size))
            else:
                ctx.groups.append(None)
        if self.use_graphs and self.model.graph_safe:
            logits = self._forward_graphed(ctx)
        else:
            self.ws.reset()
            logits = self._forward(ctx, self._logits_buffer(nw))
        self.steps_run += 1
        return logits

    def _forward(self, ctx, out):
        from ..csrc import ops
        if self.use_host_walker and not self._host_tried:
            from .host_model import HostModel
            self._host_tried = True
            self._host = HostModel.build(self.model, self.cache, self.page_size)
        if self._host is not None and self.use_host_walker and ops._PROFILE is None:
            return self._host.forward(ctx, self.ws, out)
        with ops.pinned_stream():        # one stream lookup for the pass's hundred launches
            return self.model.forward(ctx, self.cache, out)

    def _graph_key(self, ctx):
        bound = self.model.graph_bound(ctx)
        return (ctx.T, ctx.R, ctx.n_want, (ctx.max_q_len + 127) // 128 if ctx.max_q_len > 1 else 0,
                bound, ctx.n_decode, ctx.decode_ordered), bound

    def _graph_lookup(self, ctx):
        """Replay the graph of this step's shape if there is one (and its output buffer still
        stands); returns the logits view or None."""
        from ..csrc import ops
        key, _ = self._graph_key(ctx)
        hit = self._graphs.get(key)
        if hit is None or self.logits is None or self.logits.shape[0] < max(ctx.n_want, 1):
            return None
        graph, n_launches = hit
        self._graphs[key] = self._graphs.pop(key)          # most recently used last
        graph.replay()
        ops.LAUNCHES += n_launches
        self.graph_replays += 1
        return self.logits[:ctx.n_want]

    def _forward_graphed(self, ctx):
        """Replay a CUDA graph when this step's launch shapes have been seen before.  The
        shapes depend on the number of tokens, requests and wanted rows, on the longest
        portion (in 128-query tiles) and on an upper bound of the context length (see _graph_key).  Everything else a step
        varies in lies in device arrays at fixed addresses.  A shape runs eagerly the first
        time it is seen, is captured the second time, and replayed afterwards; the least
        recently used graphs are dropped beyond `max_graphs`.  (A step of steady decoding, which
        will come again, is captured the first time.)"""
        from ..csrc import ops
        key, ctx.max_keys = self._graph_key(ctx)
        before_buf = self.logits
        out = self._logits_buffer(max(ctx.n_want, 1))
        if out is not before_buf:
            self._graphs.clear()             # captured graphs wrote into the old buffer
        hit = self._graphs.get(key)
        if hit is not None:
            graph, n_launches = hit
            self._graphs[key] = self._graphs.pop(key)      # most recently used last
            graph.replay()
            ops.LAUNCHES += n_launches
            self.graph_replays += 1
            return out[:ctx.n_want]
        if key not in self._graph_seen and not ctx.repeating:
            if len(self._graph_seen) > 4096:
                self._graph_seen.clear()
            self._graph_seen.add(key)
            self.ws.reset()
            return self._forward(ctx, out)
        graph = torch.cuda.CUDAGraph()
        torch.cuda.synchronize()
        before = ops.LAUNCHES
        with torch.cuda.graph(graph):
            self.ws.reset()
            self._forward(ctx, out)
        n_launches = ops.LAUNCHES - before
        ops.LAUNCHES = before
        while len(self._graphs) >= self.max_graphs:
            self._graphs.pop(next(iter(self._graphs)))
        self._graphs[key] = (graph, n_launches)
        graph.replay()
        ops.LAUNCHES += n_launches
        self.graph_replays += 1
        return out[:ctx.n_want]

    def check_device_errors(self):
        """Raise if a kernel flagged corrupted step data (synchronises)."""
        if int(self.err_flag.item()) != 0:
            self.err_flag.zero_()
            raise RuntimeError("a kernel met an out-of-range token or position id")
        from ..csrc import ops
        flag = ops.tc_error_flag(self.rt.device)
        word = int(flag.item())
        if word != 0:
            flag.zero_()
            if word & 4:
                raise RuntimeError("a kernel of the bounds-check build met an index outside its range "
                                   "(a page id beyond the pool); the access was skipped, the output is invalid")
            raise RuntimeError("a tensor-core kernel gave up on a bounded wait; its output is invalid")
