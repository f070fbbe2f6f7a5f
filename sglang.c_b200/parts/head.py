"""Heads: hidden rows to vocabulary logits (always float32)."""
from .base import Part
from .linear import Linear
from .plan import WeightDecl
from .registry import register_part


@register_part("head", "linear")
class LinearHead(Part):
    """logits[j] = sum_k h[k]*W[j,k], no bias (reference src/gpt2.c:184-193).
    A plan ties the head to the token table by naming the same tensor for both.
    params: vocab_size, size."""

    @classmethod
    def declare_weights(cls, params):
        return {"weight": WeightDecl((params["vocab_size"], params["size"]), "embedding")}

    def load(self, tensors, store):
        self.linear = Linear(store.matrix(tensors["weight"]), None)

    def forward(self, ctx, h, out):
        return self.linear.forward(ctx, h, out=out)
