"""Plain, slow GPT-2 forward pass: the oracle that every engine test compares with.

Whole sequences, no cache, no paging, no batching: one function per part, numpy
only, float64 unless another dtype is asked for.  It shares no code with the
package under test: it has its own safetensors reader, its own config reading
and its own formulas, each restated from the reference's CPU code
(integemjack/sglang.c; paths below are relative to that project).

Anchoring: `tests/golden/make_golden.py` compiles the reference's own
`src/gpt2.c` on the CPU and stores its logits for the tiny configuration that
the reference can express (`n_inner = 4*n_embd`, tanh GELU, no inverse layer
scaling); `tests/test_plain.py` checks this file against those stored logits.
The options the reference cannot express (`n_inner`, erf GELU,
`scale_attn_by_inverse_layer_idx`, `scale_attn_weights`) rest on the formulas
alone.
"""
import json
import math
import os
import struct

import numpy as np


# --------------------------------------------------------------------------
# model folder reading (own minimal safetensors reader)
# --------------------------------------------------------------------------
def read_safetensors(path):
    """u64 little-endian header length, JSON header {name: {dtype, shape,
    data_offsets}}, then the data area (src/safetensors.c:147-179)."""
    with open(path, "rb") as f:
        raw = f.read()
    (hlen,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + hlen].decode("utf-8"))
    data = raw[8 + hlen:]
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        b, e = info["data_offsets"]
        buf = data[b:e]
        dt = info["dtype"]
        if dt == "F32":
            arr = np.frombuffer(buf, dtype="<f4").astype(np.float64)
        elif dt == "F64":
            arr = np.frombuffer(buf, dtype="<f8").astype(np.float64)
        elif dt == "BF16":
            u = np.frombuffer(buf, dtype="<u2").astype(np.uint32) << 16
            arr = u.view(np.float32).astype(np.float64)
        elif dt == "F16":
            arr = np.frombuffer(buf, dtype="<f2").astype(np.float64)
        else:
            raise ValueError(f"plain reader: dtype {dt} of {name} not handled")
        out[name] = arr.reshape(info["shape"])
    return out


def read_model_dir(model_dir):
    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = json.load(f)
    w = read_safetensors(os.path.join(model_dir, "model.safetensors"))
    # accept the "transformer." prefix of some checkpoints
    w = {(k[len("transformer."):] if k.startswith("transformer.") else k): v for k, v in w.items()}
    return cfg, w


def settings(cfg):
    """The numbers the forward pass needs, with the reference's defaults
    (src/gpt2.c:37-42); n_inner, activation_function and the two attention
    scale switches are read the same way although the reference fixes them
    (src/gpt2.c:60, src/ops.c:233-241, src/gpt2.c:253)."""
    E = int(cfg.get("n_embd", 768))
    n_inner = cfg.get("n_inner", None)
    return dict(
        L=int(cfg.get("n_layer", 12)),
        H=int(cfg.get("n_head", 12)),
        E=E,
        I=int(n_inner) if n_inner is not None else 4 * E,
        V=int(cfg.get("vocab_size", 50257)),
        P=int(cfg.get("n_ctx", cfg.get("n_positions", 1024))),
        eps=float(cfg.get("layer_norm_epsilon", 1e-5)),
        act=str(cfg.get("activation_function", "gelu_new")),
        scale_attn_weights=bool(cfg.get("scale_attn_weights", True)),
        inv_layer=bool(cfg.get("scale_attn_by_inverse_layer_idx", False)),
    )


# --------------------------------------------------------------------------
# parts
# --------------------------------------------------------------------------
def embedding(tokens, wte, wpe, pos0=0):
    """x[t,:] = wte[tok[t],:] + wpe[pos0+t,:]  (src/gpt2.c:211-216)."""
    tokens = np.asarray(tokens, dtype=np.int64)
    pos = pos0 + np.arange(len(tokens))
    return wte[tokens] + wpe[pos]


def layer_norm(x, gamma, beta, eps):
    """mean, biased variance, inv = 1/sqrt(var+eps),
    y = (x-mean)*inv*gamma + beta  (src/ops.c:199-218)."""
    mean = x.mean(axis=-1, keepdims=True)
    d = x - mean
    var = (d * d).mean(axis=-1, keepdims=True)
    inv = 1.0 / np.sqrt(var + eps)
    return d * inv * gamma + beta


def conv1d(x, w, b):
    """y = x·W + b with W in [in, out] layout, no transpose
    (src/ops.c:160-197; used at src/gpt2.c:222-223,272,283,286)."""
    return x @ w + b


def gelu_new(u):
    """0.5*u*(1+tanh(sqrt(2/pi)*(u+0.044715*u^3)))  (src/ops.c:233-241)."""
    k = 0.7978845608028654
    return 0.5 * u * (1.0 + np.tanh(k * (u + 0.044715 * u * u * u)))


def gelu_erf(u):
    """0.5*u*(1+erf(u/sqrt(2))): the exact form that config value "gelu" names.
    The reference has only the tanh form; this one rests on the formula."""
    erf = np.vectorize(math.erf, otypes=[np.float64])
    return (0.5 * u * (1.0 + erf(u.astype(np.float64) / math.sqrt(2.0)))).astype(u.dtype)


ACTIVATIONS = {"gelu_new": gelu_new, "gelu": gelu_erf,
               "gelu_pytorch_tanh": gelu_new, "gelu_fast": gelu_new}


def causal_attention(q, k, v, n_head, scale, window=None):
    """Per head h (columns [h*D,(h+1)*D) of q, k, v): s[p] = (q·K_p)*scale for
    p = 0..t (the causal mask is the loop bound), m = max s, e = exp(s-m),
    w = e/sum(e), o = sum_p w[p]*V_p; heads land side by side
    (src/gpt2.c:238-270).  `window` (not in the reference) keeps only the last
    `window` keys, p > t-window."""
    T, E = q.shape
    D = E // n_head
    out = np.zeros_like(q)
    for h in range(n_head):
        qh = q[:, h * D:(h + 1) * D]
        kh = k[:, h * D:(h + 1) * D]
        vh = v[:, h * D:(h + 1) * D]
        for t in range(T):
            lo = 0 if window is None else max(0, t - window + 1)
            s = (kh[lo:t + 1] @ qh[t]) * scale
            e = np.exp(s - s.max())
            w = e / e.sum()
            out[t, h * D:(h + 1) * D] = w @ vh[lo:t + 1]
    return out


def attention_scale(st, layer_idx):
    """1/sqrt(D) (src/gpt2.c:253) unless scale_attn_weights is false; divided
    by layer_idx+1 when scale_attn_by_inverse_layer_idx is set."""
    D = st["E"] // st["H"]
    s = 1.0 / math.sqrt(D) if st["scale_attn_weights"] else 1.0
    if st["inv_layer"]:
        s /= float(layer_idx + 1)
    return s


def _same(a):
    return a


def bf16_round(a):
    """The nearest bfloat16 (8 bits of mantissa, ties to even) of every element, as float64."""
    f = np.ascontiguousarray(a, dtype=np.float32)
    bits = f.view(np.uint32).astype(np.uint64)
    bits = (bits + 0x7FFF + ((bits >> 16) & 1)) & 0xFFFF0000
    return bits.astype(np.uint32).view(np.float32).astype(np.float64).reshape(f.shape)


def attention_block(x, w, l, st, r=_same):
    """ln_1 → c_attn → split q|k|v → attention → c_proj → residual
    (src/gpt2.c:220-278).  `r` rounds what an engine keeps in reduced precision: the normalised
    rows, the projected queries/keys/values (as they lie in the cache) and the attention output;
    the residual stream stays as it is."""
    E = st["E"]
    p = f"h.{l}."
    h = r(layer_norm(x, w[p + "ln_1.weight"], w[p + "ln_1.bias"], st["eps"]))
    qkv = r(conv1d(h, w[p + "attn.c_attn.weight"], w[p + "attn.c_attn.bias"]))
    q, k, v = qkv[:, :E], qkv[:, E:2 * E], qkv[:, 2 * E:]
    a = r(causal_attention(q, k, v, st["H"], attention_scale(st, l)))
    return x + conv1d(a, w[p + "attn.c_proj.weight"], w[p + "attn.c_proj.bias"])


def mlp_block(x, w, l, st, r=_same):
    """ln_2 → c_fc → activation → c_proj → residual  (src/gpt2.c:281-292)."""
    p = f"h.{l}."
    h = r(layer_norm(x, w[p + "ln_2.weight"], w[p + "ln_2.bias"], st["eps"]))
    u = conv1d(h, w[p + "mlp.c_fc.weight"], w[p + "mlp.c_fc.bias"])
    g = r(ACTIVATIONS[st["act"]](u))
    return x + conv1d(g, w[p + "mlp.c_proj.weight"], w[p + "mlp.c_proj.bias"])


def lm_head(hf, wte):
    """logits[j] = sum_k hf[k]*wte[j,k], tied to the token table, no bias
    (src/gpt2.c:184-193)."""
    return hf @ wte.T


def forward(cfg, w, tokens, dtype=np.float64, rounded=False):
    """Logits at every position of one whole sequence, [T, V]
    (the order of src/gpt2.c:210-297; the reference returns the last row only).
    rounded=True rounds to bfloat16 what a bfloat16 engine keeps in bfloat16 (matrices and tables,
    normalised rows, projections, cached keys and values, attention and activation outputs) and
    keeps every sum, statistic and the residual stream in float64: against it an engine's
    bfloat16 run differs by the order of its additions only, not by the rounding itself."""
    st = settings(cfg)
    w = {k: v.astype(dtype) for k, v in w.items()}
    r = _same
    if rounded:
        r = bf16_round
        w = {k: (bf16_round(v) if v.ndim >= 2 else v.astype(np.float64)) for k, v in w.items()}
    if len(tokens) > st["P"]:
        raise ValueError("sequence longer than n_positions")
    x = embedding(tokens, w["wte.weight"], w["wpe.weight"])
    for l in range(st["L"]):
        x = attention_block(x, w, l, st, r)
        x = mlp_block(x, w, l, st, r)
    hf = r(layer_norm(x, w["ln_f.weight"], w["ln_f.bias"], st["eps"]))
    return lm_head(hf, w["wte.weight"])


def forward_dir(model_dir, tokens, dtype=np.float64, rounded=False):
    cfg, w = read_model_dir(model_dir)
    return forward(cfg, w, tokens, dtype, rounded)


# --------------------------------------------------------------------------
# sampling, restated (src/sampling.c)
# --------------------------------------------------------------------------
def greedy(logits):
    """First maximum wins (src/sampling.c:23-28)."""
    return int(np.argmax(logits))


def xorshift64star(state):
    """One step of the reference's generator; returns (new_state, output)
    (src/sampling.c:10-17)."""
    m = (1 << 64) - 1
    x = state & m
    x ^= x >> 12
    x ^= (x << 25) & m
    x ^= x >> 27
    return x, (x * 0x2545F4914F6CDD1D) & m


def uniform(state):
    """(next >> 11) / 2^53 in [0,1)  (src/sampling.c:19-21)."""
    state, out = xorshift64star(state)
    return state, (out >> 11) / 9007199254740992.0


def temperature_probs(logits, temperature):
    """p_i = exp((l_i - l_max)/T) / sum  (src/sampling.c:137-145)."""
    lg = np.asarray(logits, dtype=np.float64)
    e = np.exp((lg - lg.max()) / temperature)
    return e / e.sum()


def greedy_generate(cfg, w, prompt, n_new):
    """Greedy continuation by recomputing the whole sequence each step."""
    seq = list(prompt)
    out = []
    for _ in range(n_new):
        lg = forward(cfg, w, seq)[-1]
        t = greedy(lg)
        out.append(t)
        seq.append(t)
    return out
