"""Attention mixers."""
from ..cache.needs import CacheNeed
from .base import Part
from .linear import Linear, declare_linear
from .position import PositionEncoding
from .registry import register_part


@register_part("mixer", "causal_attention")
class CausalAttention(Part):
    """Causal multi-head attention over a paged cache:
    qkv = h·W + b, split q|k|v along the last axis, heads side by side; new keys
    and values go to the cache; each query attends to the keys at positions up to
    its own (within `window` if set); the heads' outputs, side by side, go
    through the output projection into the residual
    (reference src/gpt2.c:222-278).
    params: size, n_heads, n_kv_heads, head_dim, scale (the multiplier of q·k),
    window (None or a count of keys), bias, weight_layout."""

    @classmethod
    def declare_weights(cls, params):
        lay, bias = params.get("weight_layout", "linear"), params.get("bias", True)
        qkv_out = (params["n_heads"] + 2 * params["n_kv_heads"]) * params["head_dim"]
        qkv = declare_linear(params["size"], qkv_out, lay, bias)
        out = declare_linear(params["n_heads"] * params["head_dim"], params["size"], lay, bias,
                             init="residual_matrix")
        d = {"qkv_" + k: v for k, v in qkv.items()}
        d.update({"out_" + k: v for k, v in out.items()})
        return d

    def load(self, tensors, store):
        lay = self.params.get("weight_layout", "linear")
        self.qkv = Linear.from_refs(store, tensors["qkv_weight"], tensors.get("qkv_bias"), lay)
        self.out = Linear.from_refs(store, tensors["out_weight"], tensors.get("out_bias"), lay)

    def cache_need(self):
        p = self.params
        return CacheNeed.paged_kv(p["n_kv_heads"], p["head_dim"], p.get("window"))

    def workspace_per_token(self):
        p = self.params
        return (4 if self.rt.dtype == "float32" else 2) * (2 * p["n_heads"] + 2 * p["n_kv_heads"]) * p["head_dim"]

    def graph_bound(self, ctx):
        # A step of single tokens in few (token, head) items goes to the decode attention that
        # stages a block's whole key range in shared memory sized by the bound, and what a block
        # holds of an SM decides whether it can start, and prefetch, while the kernels ahead still
        # run: there the bound moves in steps of 128 keys up to 1024 and of about an eighth of the
        # length beyond (a capture every 128 steps costs less than the tighter bound wins).
        from ..csrc import ops
        if ctx.n_decode == ctx.T and ctx.T * self.params["n_heads"] < ops.STREAM_MIN_ITEMS:
            g = 128
            while g * 8 < ctx.max_keys:
                g *= 2
            return ((ctx.max_keys + g - 1) // g) * g
        return None

    def forward(self, ctx, h, residual, cache, position=None):
        p = self.params
        H, Hkv, D = p["n_heads"], p["n_kv_heads"], p["head_dim"]
        T = h.shape[0]
        qkv = ctx.alloc((T, (H + 2 * Hkv) * D), self.rt.act_dtype)
        grp = ctx.group(cache.group)
        # a position part that acts inside the mixer turns the keys before they are cached: then
        # the projection cannot write them; one that leaves PositionEncoding.rotate as it is does not
        turns = position is not None and getattr(type(position), "rotate", None) is not PositionEncoding.rotate
        if turns:
            self.qkv.forward(ctx, h, out=qkv)
            kv_written = False
        else:
            kv_written = ctx.rt.project_qkv(ctx, h, self.qkv, qkv, cache, grp, H, Hkv, D)
        q = ctx.columns(qkv, 0, H * D)
        k = ctx.columns(qkv, H * D, (H + Hkv) * D)
        v = ctx.columns(qkv, (H + Hkv) * D, (H + 2 * Hkv) * D)
        if position is not None:
            position.rotate(ctx, q, k)
        o = ctx.alloc((T, H * D), self.rt.act_dtype)
        ctx.rt.attend(ctx, q, k, v, cache, grp, o, H, Hkv, D, float(p["scale"]), p.get("window"),
                      kv_written=kv_written)
        self.out.forward(ctx, o, residual=residual)
        return residual
