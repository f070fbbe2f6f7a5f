"""A model of built-in parts described for the C++ walker (csrc/step_walker.cu), which then
makes a step's launches itself instead of Python doing so one by one.

`HostModel.build(model, cache, page_size)` returns None when the model has a part the walker does
not know (any part registered from outside, a position encoding that acts inside a mixer, weights
in another layout): such a model keeps the Python forward pass, which is the general one.  The
walker chooses kernels exactly as `Runtime.gemm`, `Runtime.attend` and `ops.attention_decode` do
and calls the same launchers, so both ways give the same bits (tests/test_host_walker_gpu.py).
"""
import ctypes as C

import torch

from ..csrc import build, ops
from ..parts.attention import CausalAttention
from ..parts.block import PreNormBlock
from ..parts.embedding import TokenEmbedding
from ..parts.feed_forward import MLP
from ..parts.head import LinearHead
from ..parts.norm import LayerNorm
from ..parts.position import LearnedAbsolutePositions, NoPositions


class WalkLinear(C.Structure):
    _fields_ = [("w", C.c_void_p), ("bias", C.c_void_p), ("N", C.c_int), ("K", C.c_int)]


class WalkNorm(C.Structure):
    _fields_ = [("gamma", C.c_void_p), ("beta", C.c_void_p), ("eps", C.c_float), ("size", C.c_int)]


class WalkLayer(C.Structure):
    _fields_ = [("norm1", WalkNorm), ("norm2", WalkNorm), ("qkv", WalkLinear), ("out", WalkLinear),
                ("up", WalkLinear), ("down", WalkLinear), ("n_heads", C.c_int), ("n_kv_heads", C.c_int),
                ("head_dim", C.c_int), ("window", C.c_int), ("scale", C.c_float), ("act", C.c_int),
                ("inner_size", C.c_int), ("pad", C.c_int)]


class WalkCall(C.Structure):
    _fields_ = [("layer", C.c_int), ("group", C.c_int), ("write", C.c_int), ("n_pages", C.c_int),
                ("cache", C.c_void_p)]


class WalkModel(C.Structure):
    _fields_ = [("table", C.c_void_p), ("pos_table", C.c_void_p), ("layers", C.POINTER(WalkLayer)),
                ("order", C.POINTER(WalkCall)), ("final_norm", WalkNorm), ("head", WalkLinear),
                ("vocab", C.c_int), ("n_positions", C.c_int), ("hidden", C.c_int), ("n_layers", C.c_int),
                ("n_calls", C.c_int), ("bf16", C.c_int), ("page_size", C.c_int), ("pad", C.c_int)]


class WalkStep(C.Structure):
    _fields_ = [("tokens", C.c_void_p), ("positions", C.c_void_p), ("token_req", C.c_void_p),
                ("want_rows", C.c_void_p), ("q_start", C.c_void_p), ("kv_len", C.c_void_p),
                ("decode_tokens", C.c_void_p), ("block_tables", C.POINTER(C.c_void_p)),
                ("slots", C.POINTER(C.c_void_p)), ("workspace", C.c_void_p), ("workspace_bytes", C.c_longlong),
                ("logits", C.c_void_p), ("err_flag", C.c_void_p), ("tc_err", C.c_void_p), ("tc_ws", C.c_void_p),
                ("tc_ws_floats", C.c_longlong), ("tc_counters", C.c_void_p), ("tc_n_counters", C.c_int),
                ("T", C.c_int), ("R", C.c_int), ("n_want", C.c_int), ("max_q_len", C.c_int), ("max_keys", C.c_int),
                ("n_decode", C.c_int), ("decode_ordered", C.c_int), ("few_ok", C.c_int), ("bt_stride", C.c_int),
                ("stream_min_items", C.c_int), ("use_tma_decode", C.c_int), ("few_max_tokens", C.c_int),
                ("few_max_weight", C.c_longlong), ("stream", C.c_void_p), ("launches", C.c_longlong),
                ("workspace_peak", C.c_longlong), ("where", C.c_char * 96)]


_LIBS = {"sglc_embed": "embed", "sglc_layernorm": "layernorm", "sglc_gemm_simt": "gemm_simt",
         "sglc_gemm_tc": "gemm_tc", "sglc_gemm_tc_kv": "gemm_tc", "sglc_gemm_few_supports": "gemm_few", "sglc_gemm_few": "gemm_few",
         "sglc_kv_write": "kv_cache", "sglc_attention_simt": "attention_simt",
         "sglc_attention_prefill_tc": "attention_prefill_tc", "sglc_attention_decode_splits": "attention_decode",
         "sglc_attention_decode_scratch": "attention_decode", "sglc_attention_decode": "attention_decode",
         "sglc_attention_decode_tma": "attention_decode_tma",
         "sglc_attention_decode_stream_supports": "attention_decode_tma",
         "sglc_attention_decode_stream": "attention_decode_tma"}
_bound = {}


def _walker():
    """The walker's library with every launcher it calls bound by address (once per build flavour)."""
    lib = build.load("step_walker")
    key = id(lib)
    if key not in _bound:
        sizes = (C.c_int * 6)()
        lib.sglc_walker_struct_sizes(sizes)
        mine = [C.sizeof(t) for t in (WalkLinear, WalkNorm, WalkLayer, WalkCall, WalkModel, WalkStep)]
        if list(sizes) != mine:
            raise RuntimeError(f"step walker: structure sizes differ between C ({list(sizes)}) and Python ({mine})")
        names = C.POINTER(C.c_char_p)()
        n = lib.sglc_walker_names(C.byref(names))
        fns = (C.c_void_p * n)()
        for i in range(n):
            name = names[i].decode()
            fns[i] = C.cast(getattr(build.load(_LIBS[name]), name), C.c_void_p).value
        code = lib.sglc_walker_bind(fns, n)
        if code != 0:
            raise RuntimeError("step walker: binding the launchers failed")
        lib.sglc_walker_forward.argtypes = [C.POINTER(WalkModel), C.POINTER(WalkStep)]
        _bound[key] = True
    return lib


def _lin(linear):
    return WalkLinear(linear.weight.data_ptr(), linear.bias.data_ptr() if linear.bias is not None else None,
                      linear.out_size, linear.in_size)


def _norm(part):
    return WalkNorm(part.weight.data_ptr(), part.bias.data_ptr(), float(part.params["eps"]), int(part.params["size"]))


class HostModel:
    def __init__(self, model, cache, page_size, wm, keep):
        self.model, self.cache, self.page_size = model, cache, page_size
        self.wm = wm
        self._keep = keep                 # the arrays the structure points into
        self.lib = _walker()
        self.step = WalkStep()
        self.n_groups = len(cache.groups)
        self._bts = (C.c_void_p * self.n_groups)()
        self._slots = (C.c_void_p * self.n_groups)()
        self.step.block_tables = C.cast(self._bts, C.POINTER(C.c_void_p))
        self.step.slots = C.cast(self._slots, C.POINTER(C.c_void_p))
        self.step.stream_min_items = ops.STREAM_MIN_ITEMS
        self.step.few_max_tokens = ops.FEW_MAX_TOKENS
        self.step.few_max_weight = ops.FEW_MAX_WEIGHT
        ws, counters, err = ops._tc_buffers(model.rt.device)
        self.step.tc_err, self.step.tc_ws, self.step.tc_ws_floats = err.data_ptr(), ws.data_ptr(), ws.numel()
        self.step.tc_counters, self.step.tc_n_counters = counters.data_ptr(), counters.numel()

    @classmethod
    def build(cls, model, cache, page_size):
        """The description of `model` for the walker, or None if a part of it has none."""
        rt = model.rt
        if type(model.embedding) is not TokenEmbedding or type(model.head) is not LinearHead \
                or type(model.final_norm) is not LayerNorm \
                or type(model.position) not in (LearnedAbsolutePositions, NoPositions):
            return None
        ptab = model.position.additive_table()
        if ptab is not None and ptab.dtype != model.embedding.table.dtype:
            return None
        if any(g.need.kind != "paged_kv" for g in cache.groups):
            return None
        layers = (WalkLayer * len(model.layers))()
        for i, layer in enumerate(model.layers):
            if type(layer.block) is not PreNormBlock or set(layer.parts) != {"norm1", "mixer", "norm2", "ffn"}:
                return None
            n1, mx, n2, ff = layer.norm1, layer.mixer, layer.norm2, layer.ffn
            if type(n1) is not LayerNorm or type(n2) is not LayerNorm or type(mx) is not CausalAttention \
                    or type(ff) is not MLP:
                return None
            p = mx.params
            layers[i] = WalkLayer(_norm(n1), _norm(n2), _lin(mx.qkv), _lin(mx.out), _lin(ff.up), _lin(ff.down),
                                  int(p["n_heads"]), int(p["n_kv_heads"]), int(p["head_dim"]),
                                  int(p.get("window") or 0), float(p["scale"]), ops.ACT[ff.params["activation"]],
                                  int(ff.params["inner_size"]), 0)
        order = (WalkCall * len(model.plan.order))()
        for i, call in enumerate(model.plan.order):
            b = cache.binding(i)
            if b is None or b.kind != "paged_kv":
                return None
            order[i] = WalkCall(call.layer, b.group, 1 if b.write else 0, b.tensor.shape[0], b.tensor.data_ptr())
        table = model.embedding.table
        wm = WalkModel(table.data_ptr(), ptab.data_ptr() if ptab is not None else None, layers, order,
                       _norm(model.final_norm), _lin(model.head.linear), table.shape[0],
                       ptab.shape[0] if ptab is not None else 0, model.plan.hidden_size, len(model.layers),
                       len(model.plan.order), 1 if rt.dtype == "bfloat16" else 0, int(page_size), 0)
        return cls(model, cache, page_size, wm, (layers, order))

    def forward(self, ctx, workspace, logits_out):
        """The step's launches, made by the walker on the current stream; returns logits_out[:n_want]."""
        s = self.step
        s.tokens, s.positions, s.token_req = ctx.tokens.data_ptr(), ctx.positions.data_ptr(), ctx.token_req.data_ptr()
        s.want_rows, s.q_start, s.kv_len = ctx.want_rows.data_ptr(), ctx.q_start.data_ptr(), ctx.kv_len.data_ptr()
        s.decode_tokens = ctx.decode_tokens.data_ptr()
        for gi in range(self.n_groups):
            g = ctx.groups[gi]
            self._bts[gi], self._slots[gi] = g.block_table.data_ptr(), g.slots.data_ptr()
            s.bt_stride = g.block_table.stride(0)
        s.workspace, s.workspace_bytes = workspace.buf.data_ptr(), workspace.buf.numel()
        s.logits = logits_out.data_ptr()
        s.err_flag = ctx.err_flag.data_ptr()
        s.T, s.R, s.n_want, s.max_q_len, s.max_keys = ctx.T, ctx.R, ctx.n_want, ctx.max_q_len, ctx.max_keys
        s.n_decode, s.decode_ordered, s.few_ok = ctx.n_decode, int(ctx.decode_ordered), int(ctx.few_token_ok)
        s.use_tma_decode = int(ops.USE_TMA_DECODE)
        s.stream = torch.cuda.current_stream().cuda_stream
        code = self.lib.sglc_walker_forward(C.byref(self.wm), C.byref(s))
        ops.LAUNCHES += int(s.launches)
        if code != 0:
            what = s.where.decode() or "step walker"
            msg = self.lib.sglc_error_string(code).decode()
            raise ops.KernelError(f"{what}: {msg} (code {code})")
        if s.workspace_peak > workspace.peak:
            workspace.peak = int(s.workspace_peak)
        return logits_out[:ctx.n_want]
