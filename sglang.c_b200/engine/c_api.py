"""A thin binding of the engine's C interface (csrc/sglc_engine.h, built from csrc/host_engine.cu):
the same entry points as the Python scheduler (`submit_ids / step / poll / nactive / abort /
get_stats`, the reference's include/sgl/scheduler.h:33-67), with everything behind them native.
For tests, for measuring the native path, and as the example of how a C program uses the library;
models with parts registered from outside the package need the Python engine."""
import ctypes as C

from ..csrc import build
from ..sampling import SamplingParams


class CSampling(C.Structure):
    _fields_ = [("temperature", C.c_float), ("top_k", C.c_int), ("top_p", C.c_float), ("min_p", C.c_float),
                ("repetition_penalty", C.c_float), ("frequency_penalty", C.c_float),
                ("presence_penalty", C.c_float), ("ignore_eos", C.c_int), ("stop_ids", C.c_int * 8),
                ("n_stop_ids", C.c_int), ("seed", C.c_ulonglong)]


class COptions(C.Structure):
    _fields_ = [("device", C.c_int), ("bf16", C.c_int), ("page_size", C.c_int), ("n_pages", C.c_longlong),
                ("max_tokens", C.c_longlong), ("max_requests", C.c_int), ("max_step_tokens", C.c_int),
                ("prefill_chunk", C.c_int), ("token_budget", C.c_int), ("seed", C.c_ulonglong),
                ("use_graphs", C.c_int), ("eos_token_id", C.c_int), ("want_logprobs", C.c_int),
                ("run_ahead", C.c_int), ("dry_run", C.c_int), ("library_dir", C.c_char_p)]


class CStats(C.Structure):
    _fields_ = [(n, C.c_longlong) for n in
                ("prefill_tokens", "decode_tokens", "n_finished", "n_running", "n_waiting", "pool_pages",
                 "pool_free", "n_preempt", "prefill_chunk", "n_steps", "recomputed_tokens", "graph_replays",
                 "launches", "weight_bytes", "cache_bytes", "steps_ahead", "step_upload_bytes")]


FINISH = {0: None, 1: "eos", 2: "stop", 3: "length", 4: "context", 5: "abort"}
_DTYPES = {"bfloat16": 1, "bf16": 1, "float32": 0, "fp32": 0, "f32": 0}


class CEngineError(RuntimeError):
    pass


def _lib(dry_run):
    if not dry_run:
        build.build_all()              # the kernel libraries the engine loads lie beside it
    lib = build.load("host_engine")
    if not getattr(lib, "_sglc_typed", False):
        lib.sglc_engine_new.restype = C.c_void_p
        lib.sglc_engine_new.argtypes = [C.c_char_p, C.POINTER(COptions), C.c_char_p, C.c_int]
        lib.sglc_engine_free.argtypes = [C.c_void_p]
        lib.sglc_engine_submit_ids.restype = C.c_longlong
        lib.sglc_engine_submit_ids.argtypes = [C.c_void_p, C.POINTER(C.c_int), C.c_int, C.c_int, C.POINTER(CSampling)]
        lib.sglc_engine_step.argtypes = [C.c_void_p]
        lib.sglc_engine_nactive.argtypes = [C.c_void_p]
        lib.sglc_engine_poll.argtypes = [C.c_void_p, C.POINTER(C.c_longlong), C.POINTER(C.c_int), C.c_int,
                                         C.POINTER(C.c_int), C.POINTER(C.c_int), C.POINTER(C.c_int)]
        lib.sglc_engine_poll_logprobs.argtypes = [C.c_void_p, C.c_longlong, C.POINTER(C.c_float), C.c_int]
        lib.sglc_engine_abort.argtypes = [C.c_void_p, C.c_longlong]
        lib.sglc_engine_generated.argtypes = [C.c_void_p, C.c_longlong, C.POINTER(C.c_int), C.c_int]
        lib.sglc_engine_sync.argtypes = [C.c_void_p]
        lib.sglc_engine_mark.argtypes = [C.c_void_p, C.c_int]
        lib.sglc_engine_ms_between_marks.restype = C.c_double
        lib.sglc_engine_ms_between_marks.argtypes = [C.c_void_p]
        lib.sglc_engine_rewind.argtypes = [C.c_void_p, C.c_longlong, C.c_int]
        lib.sglc_engine_get_stats.argtypes = [C.c_void_p, C.POINTER(CStats)]
        lib.sglc_engine_run_until_done.restype = C.c_longlong
        lib.sglc_engine_run_until_done.argtypes = [C.c_void_p, C.c_longlong]
        lib.sglc_engine_check.argtypes = [C.c_void_p]
        lib.sglc_engine_last_step.argtypes = [C.c_void_p, C.POINTER(C.c_longlong), C.POINTER(C.c_int),
                                              C.POINTER(C.c_int), C.c_int]
        lib.sglc_engine_last_error.restype = C.c_char_p
        lib.sglc_engine_last_error.argtypes = [C.c_void_p]
        for f in (lib.sglc_engine_vocab_size, lib.sglc_engine_max_positions, lib.sglc_engine_eos_token_id):
            f.argtypes = [C.c_void_p]
        lib.sglc_sampling_default.argtypes = [C.POINTER(CSampling)]
        lib.sglc_engine_options_default.argtypes = [C.POINTER(COptions)]
        lib._sglc_typed = True
    return lib


class CEngine:
    """The native engine on a model folder.  Arguments as `sched_new` takes them; dry_run=True
    needs no device (configuration, tensor checks, page tables and scheduling run; tokens come
    from a fixed formula)."""

    def __init__(self, model_dir, seed=0, dtype="bfloat16", device=0, page_size=16, n_pages=None, max_tokens=None,
                 max_requests=64, max_step_tokens=2048, prefill_chunk=512, token_budget=None, want_logprobs=False,
                 use_graphs=True, eos_token_id="from_model", run_ahead=True, dry_run=False):
        self.lib = _lib(dry_run)
        o = COptions()
        self.lib.sglc_engine_options_default(C.byref(o))
        if isinstance(device, str):
            device = int(device.split(":")[1]) if ":" in device else 0
        o.device, o.bf16, o.page_size = int(device), _DTYPES[dtype], int(page_size)
        o.n_pages, o.max_tokens = int(n_pages or 0), int(max_tokens or 0)
        o.max_requests, o.max_step_tokens = int(max_requests), int(max_step_tokens)
        o.prefill_chunk, o.token_budget, o.seed = int(prefill_chunk or 0), int(token_budget or 0), int(seed)
        o.use_graphs, o.want_logprobs, o.dry_run = int(use_graphs), int(want_logprobs), int(dry_run)
        o.run_ahead = int(run_ahead)
        o.eos_token_id = -2 if eos_token_id == "from_model" else (-1 if eos_token_id is None else int(eos_token_id))
        err = C.create_string_buffer(1 << 16)
        self.h = self.lib.sglc_engine_new(str(model_dir).encode(), C.byref(o), err, len(err))
        if not self.h:
            raise CEngineError(err.value.decode(errors="replace"))
        self.want_logprobs = bool(want_logprobs)
        self._buf = (C.c_int * 4096)()

    def close(self):
        if getattr(self, "h", None):
            self.lib.sglc_engine_free(self.h)
            self.h = None

    __del__ = close

    def _sampling(self, sp):
        s = CSampling()
        self.lib.sglc_sampling_default(C.byref(s))
        if sp is not None:
            s.temperature, s.top_k, s.top_p, s.min_p = sp.temperature, sp.top_k, sp.top_p, sp.min_p
            s.repetition_penalty, s.frequency_penalty = sp.repetition_penalty, sp.frequency_penalty
            s.presence_penalty, s.ignore_eos, s.seed = sp.presence_penalty, int(sp.ignore_eos), int(sp.seed)
            s.n_stop_ids = len(sp.stop_ids)
            for i, t in enumerate(sp.stop_ids):
                s.stop_ids[i] = int(t)
        return s

    def submit_ids(self, ids, max_new=16, sp: SamplingParams = None):
        arr = (C.c_int * max(len(ids), 1))(*[int(t) for t in ids])
        return int(self.lib.sglc_engine_submit_ids(self.h, arr, len(ids), int(max_new or 0), C.byref(self._sampling(sp))))

    def step(self):
        n = self.lib.sglc_engine_step(self.h)
        if n < 0:
            raise CEngineError(self.last_error())
        return n

    def nactive(self):
        return self.lib.sglc_engine_nactive(self.h)

    def poll(self):
        """One finished request not yet taken: (id, generated ids, n_prompt), or None."""
        rid, n, npr, why = C.c_longlong(), C.c_int(), C.c_int(), C.c_int()
        if not self.lib.sglc_engine_poll(self.h, C.byref(rid), None, -1, C.byref(n), None, None):     # a look
            return None
        if n.value > len(self._buf):
            self._buf = (C.c_int * (2 * n.value))()
        self.last_logprobs = self.poll_logprobs(rid.value) if self.want_logprobs else None
        self.lib.sglc_engine_poll(self.h, C.byref(rid), self._buf, len(self._buf), C.byref(n), C.byref(npr), C.byref(why))
        self.last_finish = FINISH[why.value]
        return rid.value, list(self._buf[:n.value]), npr.value

    def poll_logprobs(self, req_id):
        n = self.lib.sglc_engine_poll_logprobs(self.h, int(req_id), None, 0)
        if n < 0:
            return None
        out = (C.c_float * max(n, 1))()
        self.lib.sglc_engine_poll_logprobs(self.h, int(req_id), out, n)
        return list(out[:n])

    def generated(self, req_id):
        """What the request has generated so far (running, or finished and not yet taken), or None."""
        n = self.lib.sglc_engine_generated(self.h, int(req_id), None, 0)
        if n < 0:
            return None
        if n > len(self._buf):
            self._buf = (C.c_int * (2 * n))()
        n = self.lib.sglc_engine_generated(self.h, int(req_id), self._buf, len(self._buf))
        return list(self._buf[:n])

    def sync(self):
        """Wait for the step in flight (run_ahead) and take its ids in; the requests it ended."""
        n = self.lib.sglc_engine_sync(self.h)
        if n < 0:
            raise CEngineError(self.last_error())
        return n

    def mark(self, sync_first=False):
        """A mark on the stream the steps run on, behind everything queued so far."""
        if self.lib.sglc_engine_mark(self.h, int(sync_first)) != 0:
            raise CEngineError(self.last_error())

    def ms_between_marks(self):
        """Device time between the last two marks (waits for the second)."""
        return self.lib.sglc_engine_ms_between_marks(self.h)

    def rewind(self, req_id, keep):
        """A running request forgets what it generated beyond its first `keep` ids (no step in flight)."""
        if self.lib.sglc_engine_rewind(self.h, int(req_id), int(keep)) != 0:
            raise CEngineError(f"request {req_id} cannot be rewound to {keep} generated ids")

    def abort(self, req_id):
        return self.lib.sglc_engine_abort(self.h, int(req_id))

    def get_stats(self):
        s = CStats()
        self.lib.sglc_engine_get_stats(self.h, C.byref(s))
        return s

    def run_until_done(self, max_steps=1000000):
        n = self.lib.sglc_engine_run_until_done(self.h, int(max_steps))
        if n < 0:
            raise CEngineError(self.last_error())
        return n

    def last_step(self):
        """[(request id, tokens, whether a token was sampled)] of the last step, in batch order."""
        cap = 1024
        ids, n, smp = (C.c_longlong * cap)(), (C.c_int * cap)(), (C.c_int * cap)()
        k = min(self.lib.sglc_engine_last_step(self.h, ids, n, smp, cap), cap)
        return [(ids[i], n[i], bool(smp[i])) for i in range(k)]

    def check(self):
        if self.lib.sglc_engine_check(self.h) != 0:
            raise CEngineError(self.last_error())
        return True

    def last_error(self):
        return self.lib.sglc_engine_last_error(self.h).decode(errors="replace")

    @property
    def vocab_size(self):
        return self.lib.sglc_engine_vocab_size(self.h)

    @property
    def max_positions(self):
        return self.lib.sglc_engine_max_positions(self.h)

    @property
    def eos_token_id(self):
        e = self.lib.sglc_engine_eos_token_id(self.h)
        return None if e < 0 else e
