"""Each part alone: built from its params, given weights, run on a hand-made step context,
and compared with a plain PyTorch restatement."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


class Store:
    """What a part's load() needs: tensors to the device in the runtime's precision."""

    def __init__(self, rt):
        self.rt = rt

    def matrix(self, ref, transpose=False):
        t = ref.tensor.t() if transpose else ref.tensor
        return t.to(self.rt.matrix_dtype).contiguous().to(self.rt.device)

    def vector(self, ref):
        return ref.tensor.float().contiguous().to(self.rt.device)


def make_part(category, kind, params, dtype, seed=0):
    from sglang_c_b200.engine import Runtime
    from sglang_c_b200.parts import get_part
    from sglang_c_b200.weights import TensorRef
    rt = Runtime(dtype, DEV)
    cls = get_part(category, kind)
    part = cls(params, rt)
    g = torch.Generator().manual_seed(seed)
    tensors = {}
    for role, decl in cls.declare_weights(params).items():
        t = torch.randn(*decl.shape, generator=g) * (0.1 if len(decl.shape) > 1 else 0.5)
        if decl.init == "norm_gain":
            t = t + 1.0
        if dtype == "bfloat16" and len(decl.shape) > 1:
            t = t.to(torch.bfloat16).float()       # the reference uses the values the device holds
        tensors[role] = TensorRef(role, t)
    part.load(tensors, Store(rt))
    return part, {k: v.tensor.double() for k, v in tensors.items()}, rt


def make_ctx(rt, tokens=None, positions=None, T=None):
    from sglang_c_b200.engine.step import StepContext, Workspace
    ctx = StepContext(rt, Workspace(rt.device, 64 << 20))
    ctx.T = T if T is not None else len(tokens)
    if tokens is not None:
        ctx.tokens = torch.tensor(tokens, dtype=torch.int32, device=DEV)
    if positions is not None:
        ctx.positions = torch.tensor(positions, dtype=torch.int32, device=DEV)
    ctx.err_flag = torch.zeros(1, dtype=torch.int32, device=DEV)
    return ctx


def tol(dtype):
    return 2e-5 if dtype == "float32" else 3e-2


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_layer_norm_part(dtype):
    part, w, rt = make_part("norm", "layer_norm", {"size": 80, "eps": 1e-3}, dtype)
    x = torch.randn(9, 80, device=DEV) * 2 + 1
    out = torch.empty(9, 80, dtype=rt.act_dtype, device=DEV)
    part.forward(make_ctx(rt, T=9), x, out)
    xd = x.double().cpu()
    ref = (xd - xd.mean(-1, keepdim=True)) / torch.sqrt(xd.var(-1, unbiased=False, keepdim=True) + 1e-3)
    ref = ref * w["weight"] + w["bias"]
    assert float((out.double().cpu() - ref).abs().max()) < tol(dtype)
    rows = torch.tensor([8, 0, 3], dtype=torch.int32, device=DEV)
    out3 = torch.empty(3, 80, dtype=rt.act_dtype, device=DEV)
    part.forward(make_ctx(rt, T=9), x, out3, rows=rows)
    assert torch.equal(out3, out[[8, 0, 3]])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_embedding_and_position_parts(dtype):
    emb, we, rt = make_part("embedding", "token_table", {"vocab_size": 301, "size": 48}, dtype, seed=1)
    pos, wp, _ = make_part("position", "learned_absolute", {"max_positions": 70, "size": 48}, dtype, seed=2)
    nopos, _, _ = make_part("position", "none", {}, dtype)
    tokens, positions = [5, 300, 0, 17, 17], [0, 69, 3, 4, 5]
    ctx = make_ctx(rt, tokens, positions)
    out = torch.empty(5, 48, device=DEV)
    emb.forward(ctx, out, pos)                               # fused gather + add
    ref = we["table"][tokens] + wp["table"][positions]
    assert float((out.double().cpu() - ref).abs().max()) < 1e-6
    out2 = torch.empty(5, 48, device=DEV)
    emb.forward(ctx, out2, nopos)
    assert float((out2.double().cpu() - we["table"][tokens]).abs().max()) < 1e-6
    pos.apply_embedding(ctx, out2)                           # the unfused way gives the same
    assert torch.equal(out2, out)
    assert pos.additive_table() is not None and nopos.additive_table() is None


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("act,layout", [("gelu_tanh", "conv1d"), ("gelu_erf", "linear")])
def test_mlp_part(dtype, act, layout):
    params = {"size": 96, "inner_size": 200, "activation": act, "bias": True, "weight_layout": layout}
    part, w, rt = make_part("feed_forward", "mlp", params, dtype, seed=3)
    h = (torch.randn(21, 96) * 0.7).to(rt.act_dtype).to(DEV)
    res = torch.randn(21, 96, device=DEV)
    res0 = res.double().cpu()
    part.forward(make_ctx(rt, T=21), h, res)
    hd = h.double().cpu()
    up_w = w["up_weight"] if layout == "conv1d" else w["up_weight"].t()
    down_w = w["down_weight"] if layout == "conv1d" else w["down_weight"].t()
    u = hd @ up_w + w["up_bias"]
    g = torch.nn.functional.gelu(u, approximate="tanh" if act == "gelu_tanh" else "none")
    ref = res0 + g @ down_w + w["down_bias"]
    assert float((res.double().cpu() - ref).abs().max()) < tol(dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_linear_head_part(dtype):
    part, w, rt = make_part("head", "linear", {"vocab_size": 333, "size": 64}, dtype, seed=4)
    h = (torch.randn(7, 64)).to(rt.act_dtype).to(DEV)
    out = torch.empty(7, 333, device=DEV)
    part.forward(make_ctx(rt, T=7), h, out)
    ref = h.double().cpu() @ w["weight"].t()
    assert out.dtype == torch.float32
    assert float((out.double().cpu() - ref).abs().max()) < tol(dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,Hkv,D,window", [(4, 4, 16, None), (6, 2, 32, None), (2, 2, 64, 9)])
def test_attention_part_with_its_cache(dtype, H, Hkv, D, window):
    """The mixer alone over two steps of two requests: a portion each, then a mixed step
    (a second portion of one, a single token of the other)."""
    from sglang_c_b200.cache import CacheManager
    from sglang_c_b200.engine.step import GroupStep
    E = 40
    params = {"size": E, "n_heads": H, "n_kv_heads": Hkv, "head_dim": D, "scale": 1.0 / math.sqrt(D),
              "window": window, "bias": True, "weight_layout": "conv1d"}
    part, w, rt = make_part("mixer", "causal_attention", params, dtype, seed=5)
    ps = 4
    cache = CacheManager([part.cache_need()], [None], ps, 32, 4, make_tensor=rt.make_tensor,
                         cache_dtype=rt.cache_dtype_name)
    lens = {"a": 13, "b": 7}
    hs = {r: (torch.randn(n, E, generator=torch.Generator().manual_seed(n)) * 0.8).to(rt.act_dtype)
          for r, n in lens.items()}
    for r in lens:
        cache.add_request(r)
    outs = {r: [] for r in lens}
    steps = [[("a", 0, 9), ("b", 0, 6)], [("a", 9, 13), ("b", 6, 7)]]
    for step in steps:
        ctx = make_ctx(rt, T=sum(e - s for _, s, e in step))
        rows, pos, trq, slots, bts = [], [], [], [], []
        for i, (r, s, e) in enumerate(step):
            assert cache.extend(r, e)
            rows.append(hs[r][s:e])
            pos += list(range(s, e))
            trq += [i] * (e - s)
            slots += [cache.slot_of_position(0, r, p) for p in range(s, e)]
            table = cache.block_table(0, r)
            bts.append(table + [0] * (8 - len(table)))
            ctx.h_q_len.append(e - s)
            ctx.h_kv_len.append(e)
        ctx.R = len(step)
        ctx.positions = torch.tensor(pos, dtype=torch.int32, device=DEV)
        ctx.token_req = torch.tensor(trq, dtype=torch.int32, device=DEV)
        qs = [0]
        for n in ctx.h_q_len:
            qs.append(qs[-1] + n)
        ctx.q_start = torch.tensor(qs, dtype=torch.int32, device=DEV)
        ctx.kv_len = torch.tensor(ctx.h_kv_len, dtype=torch.int32, device=DEV)
        ctx.max_keys = max(ctx.h_kv_len)
        ctx.max_q_len = max(ctx.h_q_len)
        ctx.groups = [GroupStep(torch.tensor(bts, dtype=torch.int32, device=DEV),
                                torch.tensor(slots, dtype=torch.int32, device=DEV), ps)]
        h = torch.cat(rows).to(DEV)
        res = torch.zeros(h.shape[0], E, device=DEV)
        part.forward(ctx, h, res, cache.binding(0), None)
        o = 0
        for r, s, e in step:
            outs[r].append(res[o:o + e - s].double().cpu())
            o += e - s
    for r, n in lens.items():
        got = torch.cat(outs[r])
        hd = hs[r].double()
        qkv = hd @ w["qkv_weight"] + w["qkv_bias"]
        q, k, v = qkv[:, :H * D], qkv[:, H * D:(H + Hkv) * D], qkv[:, (H + Hkv) * D:]
        if dtype == "bfloat16":
            q, k, v = (t.to(torch.bfloat16).double() for t in (q, k, v))
        att = torch.zeros(n, H * D, dtype=torch.float64)
        for hh in range(H):
            hk = hh // (H // Hkv)
            for t in range(n):
                lo = 0 if window is None else max(0, t - window + 1)
                s_ = (k[lo:t + 1, hk * D:(hk + 1) * D] @ q[t, hh * D:(hh + 1) * D]) / math.sqrt(D)
                att[t, hh * D:(hh + 1) * D] = torch.softmax(s_, 0) @ v[lo:t + 1, hk * D:(hk + 1) * D]
        ref = att @ w["out_weight"] + w["out_bias"]
        assert float((got - ref).abs().max()) < tol(dtype), r


def test_registry_lists_parts_and_refuses_unknown_kinds():
    from sglang_c_b200.parts import get_part, registered
    assert "causal_attention" in registered("mixer") and "mlp" in registered("feed_forward")
    assert "layer_norm" in registered("norm") and "learned_absolute" in registered("position")
    with pytest.raises(KeyError) as e:
        get_part("mixer", "nothing_like_this")
    assert "causal_attention" in str(e.value)
