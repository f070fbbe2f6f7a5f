"""Feed-forward parts."""
from .base import Part
from .linear import Linear, declare_linear
from .registry import register_part


@register_part("feed_forward", "mlp")
class MLP(Part):
    """residual += act(h·W_up + b_up)·W_down + b_down
    (reference src/gpt2.c:283-292; activation src/ops.c:233-241).
    params: size, inner_size, activation ("gelu_tanh" | "gelu_erf"), bias,
    weight_layout ("conv1d" = [in,out] in the file, "linear" = [out,in])."""

    @classmethod
    def declare_weights(cls, params):
        lay, bias = params.get("weight_layout", "linear"), params.get("bias", True)
        up = declare_linear(params["size"], params["inner_size"], lay, bias)
        down = declare_linear(params["inner_size"], params["size"], lay, bias, init="residual_matrix")
        d = {"up_" + k: v for k, v in up.items()}
        d.update({"down_" + k: v for k, v in down.items()})
        return d

    def load(self, tensors, store):
        lay = self.params.get("weight_layout", "linear")
        self.up = Linear.from_refs(store, tensors["up_weight"], tensors.get("up_bias"), lay)
        self.down = Linear.from_refs(store, tensors["down_weight"], tensors.get("down_bias"), lay)

    def workspace_per_token(self):
        return (4 if self.rt.dtype == "float32" else 2) * self.params["inner_size"]

    def forward(self, ctx, h, residual):
        T = h.shape[0]
        u = ctx.alloc((T, self.params["inner_size"]), self.rt.act_dtype)
        self.up.forward(ctx, h, out=u, act=self.params["activation"])
        self.down.forward(ctx, u, residual=residual)
        return residual
