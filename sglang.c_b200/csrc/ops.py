"""Python bindings of the CUDA kernels: argument checks, then a ctypes call on
the current stream.  Every function works on CUDA tensors only and raises if
the kernels' library is missing or the GPU is absent: there is no CPU path.
"""
import ctypes

import torch

from . import build

F32, BF16 = 0, 1
ACT = {None: 0, "none": 0, "gelu_tanh": 1, "gelu_erf": 2}
_DT = {torch.float32: F32, torch.bfloat16: BF16}


# how many kernels of this package were launched (bench and tests read it)
LAUNCHES = 0


class KernelError(RuntimeError):
    pass


def _ptr(t):
    return ctypes.c_void_p(t.data_ptr() if t is not None else 0)


_PINNED_STREAM = None


# Set by profile_begin(): a list of (label, start event, end event), one per launch.  Every
# binding below evaluates _stream() just before its launch and _check() just after, so the two
# bracket the kernel.
_PROFILE = None
_PROFILE_START = None


def _stream():
    global _PROFILE_START
    if _PROFILE is not None:
        _PROFILE_START = torch.cuda.Event(enable_timing=True)
        _PROFILE_START.record()
    if _PINNED_STREAM is not None:
        return _PINNED_STREAM
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def profile_begin():
    """From here on every kernel launch of this package is bracketed by a pair of CUDA events
    (which also keeps a kernel from starting under the one ahead: the times are the kernels'
    own, not their share of an overlapped step).  Queue the work behind something long, so that
    the host's launch cost does not show between the events."""
    global _PROFILE
    _PROFILE = []


def profile_end():
    """{kernel label: (launches, microseconds)} since profile_begin(); synchronises."""
    global _PROFILE
    rows, _PROFILE = _PROFILE, None
    torch.cuda.synchronize()
    out = {}
    for label, e0, e1 in rows or []:
        n, us = out.get(label, (0, 0.0))
        out[label] = (n + 1, us + e0.elapsed_time(e1) * 1e3)
    return out


class pinned_stream:
    """Within the block every kernel goes to the stream that is current at entry, looked up
    once (the lookup costs as much as a launch; a forward pass makes a hundred)."""

    def __enter__(self):
        global _PINNED_STREAM
        self.before = _PINNED_STREAM
        _PINNED_STREAM = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)

    def __exit__(self, *exc):
        global _PINNED_STREAM
        _PINNED_STREAM = self.before


def _dt(t, what):
    try:
        return _DT[t.dtype]
    except KeyError:
        raise KernelError(f"{what}: dtype {t.dtype} is not handled (float32 or bfloat16)") from None


UNSUPPORTED = -2      # a launcher's "size not supported by this kernel"


def _need_cuda(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError("kernels run on CUDA tensors only; got a CPU tensor "
                              "(this engine has no CPU path)")


def _check(lib, code, what, n_kernels=1):
    global LAUNCHES
    LAUNCHES += n_kernels
    if _PROFILE is not None and _PROFILE_START is not None:
        end = torch.cuda.Event(enable_timing=True)
        end.record()
        _PROFILE.append((what.split(" ")[0], _PROFILE_START, end))
    if code != 0:
        msg = lib.sglc_error_string(code).decode()
        raise KernelError(f"{what}: {msg} (code {code})")


def _i32(t, what):
    if t.dtype != torch.int32 or not t.is_contiguous():
        raise KernelError(f"{what} must be a contiguous int32 tensor")


# ---------------------------------------------------------------------------
def embed(tokens, table, out, positions=None, pos_table=None, err_flag=None):
    """out[t,:] = table[tokens[t],:] (+ pos_table[positions[t],:]); out is float32 [T,E]."""
    _need_cuda(tokens, table, out, positions, pos_table)
    _i32(tokens, "tokens")
    T, E = out.shape
    if out.dtype != torch.float32 or not out.is_contiguous():
        raise KernelError("embed: out must be contiguous float32")
    if table.shape[1] != E or not table.is_contiguous():
        raise KernelError(f"embed: table {tuple(table.shape)} does not match width {E}")
    P = 0
    if pos_table is not None:
        _i32(positions, "positions")
        if pos_table.dtype != table.dtype or pos_table.shape[1] != E or not pos_table.is_contiguous():
            raise KernelError("embed: position table must have the token table's dtype and width")
        P = pos_table.shape[0]
    lib = build.load("embed")
    code = lib.sglc_embed(_ptr(tokens), _ptr(positions), _ptr(table), _ptr(pos_table), _ptr(out),
                          T, E, table.shape[0], P, _dt(table, "embed table"), _ptr(err_flag), _stream())
    _check(lib, code, "embed")


def add_rows(x, idx, table):
    """x[t,:] += table[idx[t],:] (x float32)."""
    _need_cuda(x, idx, table)
    _i32(idx, "idx")
    T, E = x.shape
    if x.dtype != torch.float32 or not x.is_contiguous() or table.shape[1] != E:
        raise KernelError("add_rows: x must be contiguous float32 of the table's width")
    lib = build.load("embed")
    code = lib.sglc_add_rows(_ptr(x), _ptr(idx), _ptr(table), T, E, table.shape[0],
                             _dt(table, "table"), _stream())
    _check(lib, code, "add_rows")


def layernorm(x, gamma, beta, eps, out, rows=None):
    """out[r,:] = LayerNorm(x[rows[r] or r,:]); x float32 [*,E]; out float32 or bfloat16."""
    _need_cuda(x, gamma, beta, out, rows)
    E = x.shape[-1]
    n = out.shape[0]
    if x.dtype != torch.float32 or not x.is_contiguous() or not out.is_contiguous():
        raise KernelError("layernorm: x must be contiguous float32 and out contiguous")
    if gamma.dtype != torch.float32 or beta.dtype != torch.float32 or gamma.numel() != E or beta.numel() != E:
        raise KernelError("layernorm: gain and bias must be float32 vectors of the row width")
    if rows is not None:
        _i32(rows, "rows")
        if rows.numel() < n:
            raise KernelError("layernorm: fewer row indices than output rows")
    elif x.shape[0] < n:
        raise KernelError("layernorm: fewer input rows than output rows")
    lib = build.load("layernorm")
    code = lib.sglc_layernorm(_ptr(x), _ptr(rows), _ptr(gamma), _ptr(beta), _ptr(out), n, E,
                              ctypes.c_float(eps), _dt(out, "layernorm out"), _stream())
    _check(lib, code, f"layernorm (width {E})")


def gemm_simt(a, w, bias, out=None, residual=None, act=None):
    """out = act(a·wᵀ + bias), or residual += a·wᵀ + bias.  a [M,K] (row stride free),
    w [N,K] contiguous; plain FFMA with 32-bit accumulation."""
    _need_cuda(a, w, bias, out, residual)
    M, K = a.shape
    N = w.shape[0]
    if w.shape[1] != K or not w.is_contiguous() or a.stride(1) != 1 or a.dtype != w.dtype:
        raise KernelError(f"gemm: a {tuple(a.shape)}/{a.dtype} and w {tuple(w.shape)}/{w.dtype} do not match")
    if bias is not None and (bias.dtype != torch.float32 or bias.numel() != N):
        raise KernelError("gemm: bias must be a float32 vector of N")
    dst = residual if residual is not None else out
    if dst is None or dst.shape[0] < M or dst.shape[1] != N or dst.stride(1) != 1:
        raise KernelError("gemm: output does not match [M,N]")
    if residual is not None and residual.dtype != torch.float32:
        raise KernelError("gemm: the residual stream is float32")
    lib = build.load("gemm_simt")
    code = lib.sglc_gemm_simt(_ptr(a), _ptr(w), _ptr(bias), _ptr(out), _ptr(residual), M, N, K,
                              a.stride(0), dst.stride(0), _dt(a, "gemm input"),
                              _dt(dst, "gemm output"), ACT[act], _stream())
    _check(lib, code, f"gemm_simt M={M} N={N} K={K}")


def kv_write(k_src, v_src, cache, slots, n_kv_heads, head_dim):
    """Scatter keys and values of T tokens into one layer's pages.
    k_src, v_src: [T, n_kv_heads*head_dim] views (row stride free); cache:
    [n_pages, 2, n_kv_heads, page_size, head_dim]; slots int32 [T]."""
    _need_cuda(k_src, v_src, cache, slots)
    _i32(slots, "slots")
    T = k_src.shape[0]
    n_pages, two, H, page_size, D = cache.shape
    if two != 2 or H != n_kv_heads or D != head_dim or not cache.is_contiguous():
        raise KernelError(f"kv_write: cache {tuple(cache.shape)} does not match heads {n_kv_heads} x {head_dim}")
    if k_src.shape[1] != H * D or k_src.stride(1) != 1 or v_src.stride(1) != 1 \
            or k_src.stride(0) != v_src.stride(0) or k_src.dtype != cache.dtype:
        raise KernelError("kv_write: key/value rows do not match the cache")
    lib = build.load("kv_cache")
    code = lib.sglc_kv_write(_ptr(k_src), _ptr(v_src), k_src.stride(0), _ptr(cache), _ptr(slots), T,
                             H, D, page_size, n_pages, _dt(k_src, "kv source"), _dt(cache, "cache"),
                             _stream())
    _check(lib, code, "kv_write")


def attention_simt(q, cache, block_table, token_req, positions, out, n_heads, scale, window,
                   max_keys, max_q_len=None):
    """Causal attention of T tokens over the paged cache, 32-bit arithmetic.
    q: [T, n_heads*head_dim] view; out likewise; block_table int32 [R, max_blocks].
    max_q_len: the longest portion among the tokens (1 when every request brings one token;
    unknown: None); it only decides how many tokens share a block."""
    _need_cuda(q, cache, block_table, token_req, positions, out)
    for t, nm in ((block_table, "block_table"), (token_req, "token_req"), (positions, "positions")):
        _i32(t, nm)
    T = q.shape[0]
    n_pages, two, Hkv, page_size, D = cache.shape
    if q.shape[1] != n_heads * D or q.stride(1) != 1 or out.stride(1) != 1 or q.dtype != out.dtype:
        raise KernelError("attention: query/output rows do not match heads x head_dim")
    if q.dtype != cache.dtype:
        raise KernelError("attention: queries and cache must have one dtype")
    lib = build.load("attention_simt")
    code = lib.sglc_attention_simt(_ptr(q), q.stride(0), _ptr(cache), _ptr(block_table),
                                   block_table.stride(0), _ptr(token_req), _ptr(positions), _ptr(out),
                                   out.stride(0), T, n_heads, Hkv, D, page_size, ctypes.c_float(scale),
                                   int(window or 0), int(max_keys), _dt(q, "attention q"),
                                   _dt(cache, "cache"), n_pages, _ptr(tc_error_flag(q.device)),
                                   int(max_q_len) if max_q_len else 2, _stream())
    _check(lib, code, f"attention_simt (head_dim {D}, up to {max_keys} keys)")


# ---------------------------------------------------------------------------
# tensor-core GEMM (bfloat16, tcgen05 + TMA)
_tc_scratch = {}
TC_WS_FLOATS = 8 << 20          # 32 MB of split-K partial sums
TC_COUNTERS = 8192


def _tc_buffers(device):
    """Split-K workspace, tile counters (zero between launches) and the error word of the
    tensor-core kernels, one set per device, allocated at first use."""
    b = _tc_scratch.get(device)
    if b is None:
        b = (torch.empty(TC_WS_FLOATS, dtype=torch.float32, device=device),
             torch.zeros(TC_COUNTERS, dtype=torch.int32, device=device),
             torch.zeros(1, dtype=torch.int32, device=device))
        _tc_scratch[device] = b
    return b


def tc_error_flag(device):
    return _tc_buffers(device)[2]


def wait_probe(device, polls=300, peer_cycles=200000):
    """Makes a bounded wait run out, on purpose and harmlessly: two tiny kernels (csrc/wait_probe.cu)
    wait, with a limit of `polls`, on barriers that nobody arrives on, give up, tear down as the
    tensor-core kernels do and set the error word those kernels share.  Returns the kernels' trace
    [waiter, its block's other warps, cluster waiter, peer left, waiter left] (2 = ran out,
    1 = happened); the error word is left set for the caller to find."""
    lib = build.load("wait_probe")
    err = _tc_buffers(torch.device(device))[2]
    trace = torch.zeros(5, dtype=torch.int32, device=device)
    code = lib.sglc_wait_probe(_ptr(err), _ptr(trace), ctypes.c_uint(int(polls)), int(peer_cycles), _stream())
    _check(lib, code, "wait_probe", n_kernels=2)
    return trace.tolist()


def gemm_tc_supported(a, w):
    """TMA needs 16-byte aligned rows: K and the row stride multiples of 8 elements."""
    return (a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and a.dim() == 2
            and a.shape[1] % 8 == 0 and a.stride(1) == 1 and a.stride(0) % 8 == 0
            and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0 and w.is_contiguous())


def gemm_tc(a, w, bias, out=None, residual=None, act=None, supported=False):
    """out = act(a·wᵀ + bias) (bfloat16 or float32), or residual += a·wᵀ + bias, on the
    tensor cores.  a [M,K] bfloat16 (row stride free), w [N,K] bfloat16 contiguous.
    supported=True: the caller has just asked gemm_tc_supported(a, w)."""
    _need_cuda(a, w, bias, out, residual)
    if not supported and not gemm_tc_supported(a, w):
        raise KernelError(f"gemm_tc: operands a {tuple(a.shape)} stride {a.stride()} / w {tuple(w.shape)} "
                          "do not meet the 16-byte row rule of TMA (K and row stride multiples of 8)")
    M, K = a.shape
    N = w.shape[0]
    if w.shape[1] != K:
        raise KernelError(f"gemm_tc: a {tuple(a.shape)} and w {tuple(w.shape)} do not match")
    if bias is not None and (bias.dtype != torch.float32 or bias.numel() != N):
        raise KernelError("gemm_tc: bias must be a float32 vector of N")
    dst = residual if residual is not None else out
    if dst is None or dst.shape[0] < M or dst.shape[1] != N or dst.stride(1) != 1:
        raise KernelError("gemm_tc: output does not match [M,N]")
    if residual is not None:
        if residual.dtype != torch.float32:
            raise KernelError("gemm_tc: the residual stream is float32")
        if act not in (None, "none"):
            raise KernelError("gemm_tc: no activation when adding into the residual stream")
    elif dst.dtype not in (torch.float32, torch.bfloat16):
        raise KernelError("gemm_tc: output must be float32 or bfloat16")
    lib = build.load("gemm_tc")
    err = _tc_buffers(a.device)[2]
    code = lib.sglc_gemm_tc(_ptr(a), _ptr(w), _ptr(bias), _ptr(out), _ptr(residual), M, N, K,
                            a.stride(0), dst.stride(0), 1 if dst.dtype == torch.float32 else 0,
                            ACT[act], _ptr(err), _stream())
    _check(lib, code, f"gemm_tc M={M} N={N} K={K}")


def gemm_tc_kv(a, w, bias, out, cache, slots, n_heads, n_kv_heads, head_dim):
    """The query/key/value projection of a step with prompt portions, with the cache write in its
    epilogue: out[:, :n_heads*head_dim] takes the queries; keys and values go straight into the
    paged cache [n_pages, 2, n_kv_heads, page_size, head_dim] at slots[token].  Returns False,
    having launched nothing, when the product would not take the many-token kernel or the sizes
    do not fall on its tiles (the caller then projects and writes the cache separately)."""
    _need_cuda(a, w, bias, out, cache, slots)
    M, K = a.shape
    N = w.shape[0]
    if not gemm_tc_supported(a, w) or w.shape[1] != K or out.dtype != torch.bfloat16 or cache.dtype != torch.bfloat16 \
            or out.shape[1] != N or out.stride(1) != 1 or not cache.is_contiguous() \
            or N != (n_heads + 2 * n_kv_heads) * head_dim:
        return False
    _i32(slots, "slots")
    n_pages, two, Hkv, page_size, D = cache.shape
    if two != 2 or Hkv != n_kv_heads or D != head_dim or slots.numel() < M:
        raise KernelError("gemm_tc_kv: the cache or the slots do not match the projection")
    lib = build.load("gemm_tc")
    err = _tc_buffers(a.device)[2]
    code = lib.sglc_gemm_tc_kv(_ptr(a), _ptr(w), _ptr(bias), _ptr(out), M, N, K, a.stride(0), out.stride(0), ACT[None],
                               _ptr(cache), _ptr(slots), n_heads * head_dim, n_kv_heads, head_dim, page_size, n_pages,
                               _ptr(err), _stream())
    if code == UNSUPPORTED:
        return False
    _check(lib, code, f"gemm_tc_kv M={M} N={N} K={K}")
    return True


def gemm_tc_form(M, N, K, act=None):
    """Which of gemm_tc's kernels a product of these sizes takes: "few" (up to 128 tokens: weights on
    the MMA's 128-row side, split-K over a cluster), "stream" (many tokens, one block a tile) or "pair"
    (many tokens on pairs of SMs)."""
    return ("few", "stream", "pair")[build.load("gemm_tc").sglc_gemm_tc_form(int(M), int(N), int(K), ACT[act])]


FEW_MAX_TOKENS = 2           # products of so few tokens go to gemm_few ...
FEW_MAX_WEIGHT = 3 << 20     # ... if the weight matrix has no more elements than this


def gemm_few(a, w, bias, out=None, residual=None, act=None):
    """The same product as gemm_tc for up to 8 tokens: 8 output features a block over the whole
    of K, operands from global memory straight into the registers of the warp-level
    tensor-core instruction, no block waiting for another."""
    _need_cuda(a, w, bias, out, residual)
    M, K = a.shape
    N = w.shape[0]
    lib = build.load("gemm_few")
    if w.shape[1] != K or not gemm_tc_supported(a, w) or not lib.sglc_gemm_few_supports(M, N, K, a.stride(0)):
        raise KernelError(f"gemm_few: a {tuple(a.shape)} stride {a.stride()} / w {tuple(w.shape)}: up to 8 "
                          "tokens, K and the row stride multiples of 8, 16-byte aligned operands")
    if bias is not None and (bias.dtype != torch.float32 or bias.numel() != N):
        raise KernelError("gemm_few: bias must be a float32 vector of N")
    dst = residual if residual is not None else out
    if dst is None or dst.shape[0] < M or dst.shape[1] != N or dst.stride(1) != 1:
        raise KernelError("gemm_few: output does not match [M,N]")
    if residual is not None:
        if residual.dtype != torch.float32:
            raise KernelError("gemm_few: the residual stream is float32")
        if act not in (None, "none"):
            raise KernelError("gemm_few: no activation when adding into the residual stream")
    elif dst.dtype not in (torch.float32, torch.bfloat16):
        raise KernelError("gemm_few: output must be float32 or bfloat16")
    code = lib.sglc_gemm_few(_ptr(a), _ptr(w), _ptr(bias), _ptr(out), _ptr(residual), M, N, K,
                             a.stride(0), dst.stride(0), 1 if dst.dtype == torch.float32 else 0,
                             ACT[act], _stream())
    _check(lib, code, f"gemm_few M={M} N={N} K={K}")


# ---------------------------------------------------------------------------
STREAM_MIN_ITEMS = 160     # (token, head) items from which the streaming decode kernel is used
USE_TMA_DECODE = True      # tests switch it off to reach the register-staged kernel at head size 64/128


def attention_decode(q, cache, block_table, token_req, positions, out, n_heads, scale, window,
                     max_keys, k_new=None, v_new=None, slots=None, token_list=None, n_tokens=None,
                     n_splits=None, variant=None):
    """Attention of single decoded tokens over the paged bfloat16 cache, keys split across
    blocks and merged in a fixed order.  With k_new/v_new/slots (the step's own keys and
    values, [T, n_kv_heads*head_dim] views, and their cache slots) the same launch also writes
    them into the cache; this is valid only when every request brings exactly one token.
    `token_list` (int32, its first `n_tokens` entries) names the tokens to serve; a list of all
    tokens is an order in which the streaming kernel takes them (long contexts first balance
    its blocks).
    Three kernels serve it, chosen by the size of the launch (or named by `variant`, for tests
    and tuning: "stream", "tma", "register")."""
    _need_cuda(q, cache, block_table, token_req, positions, out, k_new, v_new, slots, token_list)
    for t, nm in ((block_table, "block_table"), (positions, "positions")):
        _i32(t, nm)
    if token_req is not None:           # None: token t belongs to the step's t-th request
        _i32(token_req, "token_req")
    T = q.shape[0]
    order_only = False
    if token_list is not None:          # serve only the listed tokens (the first n_tokens entries)
        _i32(token_list, "token_list")
        if token_req is None or k_new is not None:
            # without a token -> request table, or with the cache write, the list can only be an
            # order of all tokens (long ones first); the streaming kernel alone makes use of it
            if int(n_tokens) != T:
                raise KernelError("attention_decode: a list of some tokens needs token_req and no fused cache write")
            order_only = True
        T = int(n_tokens)
    n_pages, two, Hkv, page_size, D = cache.shape
    if q.dtype != torch.bfloat16 or cache.dtype != torch.bfloat16 or out.dtype != torch.bfloat16:
        raise KernelError("attention_decode: bfloat16 queries, cache and output only")
    if q.shape[1] != n_heads * D or q.stride(1) != 1 or out.stride(1) != 1:
        raise KernelError("attention_decode: query/output rows do not match heads x head_dim")
    lib = build.load("attention_decode")
    ws, counters, err = _tc_buffers(q.device)
    splits = int(n_splits) if n_splits else lib.sglc_attention_decode_splits(T, n_heads, int(max_keys))
    need_ws, need_c = ctypes.c_longlong(0), ctypes.c_int(0)
    lib.sglc_attention_decode_scratch(T, n_heads, D, splits, ctypes.byref(need_ws), ctypes.byref(need_c))
    if need_ws.value > ws.numel() or need_c.value > counters.numel():
        splits = 1
    new_stride = 0
    if k_new is not None:
        _i32(slots, "slots")
        if v_new is None or k_new.dtype != torch.bfloat16 or tuple(k_new.shape) != (T, Hkv * D) \
                or k_new.stride(1) != 1 or v_new.stride(1) != 1 or k_new.stride(0) != v_new.stride(0):
            raise KernelError("attention_decode: new keys/values do not match the cache")
        new_stride = k_new.stride(0)
    if variant not in (None, "stream", "tma", "register"):
        raise KernelError(f"attention_decode: unknown variant {variant!r}")
    if variant == "stream" or (variant is None and USE_TMA_DECODE and T * n_heads >= STREAM_MIN_ITEMS):
        # many (token, head) items: resident blocks stream them through a ring of TMA stages
        tlib = build.load("attention_decode_tma")
        if tlib.sglc_attention_decode_stream_supports(D, page_size, int(max_keys), int(window or 0)) \
                and (page_size * D * 2) % 128 == 0:
            code = tlib.sglc_attention_decode_stream(_ptr(q), q.stride(0), _ptr(cache), _ptr(block_table),
                                                     block_table.stride(0), _ptr(token_req), _ptr(positions),
                                                     _ptr(out), out.stride(0), T, n_heads, Hkv, D, page_size,
                                                     ctypes.c_float(scale), int(window or 0), int(max_keys),
                                                     _ptr(k_new), _ptr(v_new), new_stride, _ptr(slots),
                                                     _ptr(err), _ptr(token_list), n_pages, _stream())
            _check(tlib, code, f"attention_decode_stream (head_dim {D}, up to {max_keys} keys)")
            return
        if variant == "stream":
            raise KernelError(f"attention_decode_stream does not take head_dim {D}, page size {page_size}, "
                              f"{max_keys} keys")
    if order_only:
        token_list = None
    if D in (64, 128) and splits <= 8 and (page_size * D * 2) % 128 == 0 and page_size <= 256 \
            and ((variant is None and USE_TMA_DECODE and T * n_heads * splits <= 1536) or variant == "tma"):
        # keys and values staged through shared memory by TMA (measured faster up to about a
        # thousand blocks; beyond, the register-staged kernel is a few percent ahead)
        tlib = build.load("attention_decode_tma")
        code = tlib.sglc_attention_decode_tma(_ptr(q), q.stride(0), _ptr(cache), _ptr(block_table),
                                              block_table.stride(0), _ptr(token_req), _ptr(positions),
                                              _ptr(out), out.stride(0), T, n_heads, Hkv, D, page_size,
                                              ctypes.c_float(scale), int(window or 0), int(max_keys), splits,
                                              _ptr(k_new), _ptr(v_new), new_stride, _ptr(slots), _ptr(err),
                                              _ptr(token_list), n_pages, _stream())
        if code != -2 or variant == "tma":  # -2: the range does not fit its shared memory; use the other kernel
            _check(tlib, code, f"attention_decode_tma (head_dim {D}, up to {max_keys} keys)")
            return
    code = lib.sglc_attention_decode(_ptr(q), q.stride(0), _ptr(cache), _ptr(block_table),
                                     block_table.stride(0), _ptr(token_req), _ptr(positions), _ptr(out),
                                     out.stride(0), T, n_heads, Hkv, D, page_size, ctypes.c_float(scale),
                                     int(window or 0), int(max_keys), splits, _ptr(ws), _ptr(counters),
                                     _ptr(k_new), _ptr(v_new), new_stride, _ptr(slots), _ptr(err),
                                     _ptr(token_list), n_pages, _stream())
    _check(lib, code, f"attention_decode (head_dim {D}, up to {max_keys} keys)")


# ---------------------------------------------------------------------------
def attention_prefill_tc_supported(q, cache, scale):
    D = cache.shape[-1]
    return (q.dtype == torch.bfloat16 and cache.dtype == torch.bfloat16 and D in (64, 128)
            and scale > 0 and q.stride(0) % 8 == 0 and q.data_ptr() % 16 == 0)


def attention_prefill_tc(q, cache, block_table, q_start, kv_len, out, n_heads, scale, window,
                         n_requests, max_q_len, skip_single=False):
    """Causal attention of prompt portions on the tensor cores (tcgen05), bfloat16, head
    sizes 64 and 128.  q_start int32 [R+1], kv_len int32 [R] (lengths after this step)."""
    _need_cuda(q, cache, block_table, q_start, kv_len, out)
    for t, nm in ((block_table, "block_table"), (q_start, "q_start"), (kv_len, "kv_len")):
        _i32(t, nm)
    n_pages, two, Hkv, page_size, D = cache.shape
    if not attention_prefill_tc_supported(q, cache, scale):
        raise KernelError(f"attention_prefill_tc: head size {D} / dtype {q.dtype} / scale {scale} not "
                          "supported (bfloat16, head size 64 or 128, positive scale)")
    if q.shape[1] != n_heads * D or q.stride(1) != 1 or out.stride(1) != 1 or out.dtype != torch.bfloat16 \
            or out.stride(0) % 8 != 0 or out.data_ptr() % 16 != 0:
        raise KernelError("attention_prefill_tc: query/output rows do not match heads x head_dim")
    lib = build.load("attention_prefill_tc")
    err = _tc_buffers(q.device)[2]
    code = lib.sglc_attention_prefill_tc(_ptr(q), q.stride(0), _ptr(cache), _ptr(block_table),
                                         block_table.stride(0), _ptr(q_start), _ptr(kv_len), _ptr(out),
                                         out.stride(0), int(n_requests), int(max_q_len), n_heads, Hkv, D,
                                         page_size, ctypes.c_float(scale), int(window or 0), q.shape[0],
                                         n_pages, 1 if skip_single else 0, _ptr(err), _stream())
    _check(lib, code, f"attention_prefill_tc (head_dim {D})")


# ---------------------------------------------------------------------------
def sample(logits, params, hist_tok, hist_cnt, out_tok, out_logprob=None):
    """One token per row of `logits` ([n, V] float32, row stride free; penalties
    change the rows in place).  `params`: int32 tensor [n, 10] holding the packed
    per-row records (see sampling.cu); hist_tok/hist_cnt: int32 (token, count)
    pairs of the rows' histories."""
    _need_cuda(logits, params, hist_tok, hist_cnt, out_tok, out_logprob)
    n, V = logits.shape
    if logits.dtype != torch.float32 or logits.stride(1) != 1:
        raise KernelError("sample: logits must be float32 rows")
    if params.dtype != torch.int32 or params.shape != (n, 10) or not params.is_contiguous():
        raise KernelError("sample: params must be a contiguous int32 [n,10] tensor")
    _i32(out_tok, "out_tok")
    lib = build.load("sampling")
    code = lib.sglc_sample(_ptr(logits), logits.stride(0), V, n, _ptr(params), _ptr(hist_tok),
                           _ptr(hist_cnt), _ptr(out_tok), _ptr(out_logprob), _stream())
    _check(lib, code, "sample")


def set_pdl(on):
    """Turn programmatic dependent launch on or off in every kernel library (on by default)."""
    for name in build.sources():
        build.load(name).sglc_set_pdl(1 if on else 0)
