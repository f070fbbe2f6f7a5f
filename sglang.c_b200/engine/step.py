"""One step: a batch of (request, its next tokens) as flat device arrays.

The reference has two entry points, one prompt portion of one request or a
batch of single decode tokens (include/sgl/model.h:29-35, src/scheduler.c:454-523).
Here a step is any mix of both.  Everything that varies from step to step lives
in one packed int32 block that is copied to the device once; the kernels read
it from fixed addresses.
"""
from dataclasses import dataclass
from typing import List

import torch


@dataclass
class StepEntry:
    """The next `tokens` of request `req`; `want` lists the places among them
    whose logits are asked for (may be empty)."""
    req: object
    tokens: List[int]            # or an integer array
    want: List[int]


@dataclass
class GroupStep:
    block_table: torch.Tensor   # int32 [R_cap, B_cap]; row r = pages of the step's r-th request
    slots: torch.Tensor         # int32 [T]: where token t's keys/values go (page*page_size+offset)
    page_size: int


_ELEMENT_SIZE = {torch.float32: 4, torch.bfloat16: 2, torch.int32: 4, torch.uint8: 1, torch.float16: 2,
                 torch.int64: 8}


class Workspace:
    """A bump allocator over one device buffer, so that a step allocates
    nothing and the same step shape uses the same addresses."""

    def __init__(self, device, nbytes):
        self.device = device
        self.buf = torch.empty(max(int(nbytes), 256), dtype=torch.uint8, device=device)
        self.off = 0
        self.peak = 0
        self._views = {}      # (start, dtype, shape) -> view: every layer asks for the same ones
        self._cols = {}       # (id of a view, first column, end) -> its column range

    def reset(self):
        self.off = 0

    def alloc(self, shape, dtype):
        start = (self.off + 255) & ~255
        key = (start, dtype, shape if type(shape) is tuple else tuple(shape))
        hit = self._views.get(key)
        if hit is not None:
            view, end = hit
            self.off = end
            if end > self.peak:
                self.peak = end
            return view
        n = 1
        for s in shape:
            n *= int(s)
        nbytes = n * _ELEMENT_SIZE[dtype]
        if start + nbytes > self.buf.numel():
            raise MemoryError(
                f"step workspace of {self.buf.numel()} bytes is too small for {nbytes} more bytes: a part "
                "asks ctx.alloc for more than its workspace_per_token() declared")
        self.off = start + nbytes
        self.peak = max(self.peak, self.off)
        view = self.buf[start:start + nbytes].view(dtype).view(*shape)
        if len(self._views) >= 4096:
            self._views.clear()
            self._cols.clear()
        self._views[key] = (view, self.off)
        return view

    def columns(self, t, first, end):
        """t[:, first:end] of a view that alloc() gave out, made once (alloc hands the same
        object out again, so its identity is a key for as long as the view is kept)."""
        key = (id(t), first, end)
        hit = self._cols.get(key)
        if hit is None or hit[0] is not t:
            hit = (t, t[:, first:end])
            self._cols[key] = hit
        return hit[1]


class StepContext:
    """What parts see of a step.  Device arrays (int32): tokens[T], positions[T],
    token_req[T] (index of the token's request within this step), q_start[R+1],
    kv_len[R] (length of each request after this step), state_slots[R],
    want_rows[W].  Host copies: h_q_len, h_kv_len, h_state_slots, h_fresh (request
    starts at position 0 in this step), max_keys (most keys any token sees)."""

    def __init__(self, rt, workspace):
        self.rt = rt
        self.ws = workspace
        self.T = 0
        self.R = 0
        self.n_want = 0
        self.tokens = self.positions = self.token_req = None
        self.q_start = self.kv_len = self.state_slots = self.want_rows = None
        self.h_q_len = []
        self.h_kv_len = []
        self.h_fresh = []
        self.h_reqs = []
        self.h_state_slots = []
        self.max_keys = 0
        self.max_q_len = 0
        self.repeating = False         # the step repeats the last one's shape (steady decoding)
        self.n_decode = 0              # tokens of requests that bring exactly one token
        self.decode_tokens = None      # their indices (device int32), longest context first
        self.decode_ordered = False    # a step of single tokens whose contexts differ by a tile of keys or more
        self.groups: List[GroupStep] = []
        self.err_flag = None
        self.few_token_ok = False      # every matrix of the model's layers is small (see Runtime.gemm)

    def group(self, i):
        return self.groups[i]

    def alloc(self, shape, dtype):
        return self.ws.alloc(shape, dtype)

    def columns(self, t, first, end):
        return self.ws.columns(t, first, end)

    def mark(self):
        return self.ws.off

    def release(self, mark):
        self.ws.off = mark


class StepBuffers:
    """Pinned host and device copies of the packed step data, with fixed views."""

    def __init__(self, device, t_cap, r_cap, b_cap, n_groups):
        self.t_cap, self.r_cap, self.b_cap, self.n_groups = t_cap, r_cap, b_cap, n_groups
        sizes = [("tokens", t_cap), ("positions", t_cap), ("token_req", t_cap), ("want_rows", t_cap),
                 ("decode_tokens", r_cap),
                 ("q_start", r_cap + 1), ("kv_len", r_cap), ("state_slots", r_cap)]
        for g in range(n_groups):
            sizes += [(f"slots{g}", t_cap), (f"bt{g}", r_cap * b_cap)]
        self.offsets = {}
        off = 0
        for name, n in sizes:
            self.offsets[name] = (off, n)
            off += (n + 3) & ~3           # 16-byte aligned fields
        self.total = off
        self.host = torch.zeros(off, dtype=torch.int32).pin_memory()
        self.np = self.host.numpy()            # the same pinned memory, for fast host-side filling
        self.dev = torch.zeros(off, dtype=torch.int32, device=device)
        self.copied = torch.cuda.Event()
        self._copied_once = False

    def hview(self, name):
        o, n = self.offsets[name]
        return self.host[o:o + n]

    def npview(self, name):
        o, n = self.offsets[name]
        return self.np[o:o + n]

    def dview(self, name, n=None):
        o, cap = self.offsets[name]
        return self.dev[o:o + (cap if n is None else n)]

    def upload(self, n_words=None):
        """Copy the packed block (or its first n_words) to the device on the current stream."""
        if n_words is None or n_words >= self.total:
            self.dev.copy_(self.host, non_blocking=True)
        else:
            self.dev[:n_words].copy_(self.host[:n_words], non_blocking=True)
        self.copied.record()
        self._copied_once = True

    def wait_host_free(self):
        if self._copied_once:
            self.copied.synchronize()
