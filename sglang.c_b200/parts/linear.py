"""y = a·Wᵀ + b as the parts use it: a weight kept [out, in] on the device (a
file's Conv1D [in, out] layout is transposed once at load, as the reference does
at upload, src/cuda_backend.cu:5232-5241), a 32-bit bias, and a choice of
kernel by precision and shape."""
import torch

from ..csrc import ops
from .plan import WeightDecl


def declare_linear(in_size, out_size, layout, bias, init="matrix"):
    shape = (in_size, out_size) if layout == "conv1d" else (out_size, in_size)
    d = {"weight": WeightDecl(shape, init)}
    if bias:
        d["bias"] = WeightDecl((out_size,), "bias")
    return d


class Linear:
    def __init__(self, weight, bias):
        self.weight = weight      # [N,K], float32 or bfloat16
        self.bias = bias          # float32 [N] or None
        self.out_size, self.in_size = weight.shape

    @classmethod
    def from_refs(cls, store, weight_ref, bias_ref, layout):
        w = store.matrix(weight_ref, transpose=(layout == "conv1d"))
        b = store.vector(bias_ref) if bias_ref is not None else None
        return cls(w, b)

    def forward(self, ctx, a, out=None, act=None, residual=None):
        """out = act(a·Wᵀ + b)  or  residual += a·Wᵀ + b (32-bit, in place)."""
        ctx.rt.gemm(a, self.weight, self.bias, out=out, residual=residual, act=act, few_ok=ctx.few_token_ok)
        return residual if residual is not None else out
