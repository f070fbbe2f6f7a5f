"""Arrangements of norm, mixer and feed-forward around the residual stream."""
from .base import Part
from .registry import register_part


@register_part("block", "pre_norm")
class PreNormBlock(Part):
    """x += mixer(norm1(x)); x += ffn(norm2(x))  (reference src/gpt2.c:219-293).
    The residual stream x stays 32-bit; the normalised rows are in the
    runtime's activation precision."""

    def workspace_per_token(self, layer):
        act = 4 if self.rt.dtype == "float32" else 2
        return act * layer.norm1.params["size"] + max(layer.mixer.workspace_per_token(),
                                                      layer.ffn.workspace_per_token())

    def forward(self, ctx, x, layer, cache, position=None):
        T = x.shape[0]
        mark = ctx.mark()
        h = ctx.alloc((T, x.shape[1]), self.rt.act_dtype)
        layer.norm1.forward(ctx, x, h)
        inner = ctx.mark()
        layer.mixer.forward(ctx, h, residual=x, cache=cache, position=position)
        ctx.release(inner)               # the mixer's buffers make room for the feed-forward's
        layer.norm2.forward(ctx, x, h)
        layer.ffn.forward(ctx, h, residual=x)
        ctx.release(mark)
        return x
