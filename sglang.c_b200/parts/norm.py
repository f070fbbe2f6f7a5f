"""Normalisation parts."""
from ..csrc import ops
from .base import Part
from .plan import WeightDecl
from .registry import register_part


@register_part("norm", "layer_norm")
class LayerNorm(Part):
    """y = (x-mean)/sqrt(var+eps)*weight + bias over the last axis, biased
    variance, statistics in 32-bit (reference src/ops.c:199-218).
    params: size, eps."""

    @classmethod
    def declare_weights(cls, params):
        return {"weight": WeightDecl((params["size"],), "norm_gain"),
                "bias": WeightDecl((params["size"],), "norm_bias")}

    def load(self, tensors, store):
        self.weight = store.vector(tensors["weight"])
        self.bias = store.vector(tensors["bias"])

    def forward(self, ctx, x, out, rows=None):
        ops.layernorm(x, self.weight, self.bias, float(self.params["eps"]), out, rows=rows)
        return out
