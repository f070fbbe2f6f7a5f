"""Token embedding."""
from ..csrc import ops
from .base import Part
from .plan import WeightDecl
from .registry import register_part


@register_part("embedding", "token_table")
class TokenEmbedding(Part):
    """out[t,:] = table[tokens[t],:] in 32-bit (reference sgl_embedding_get,
    src/ops.c:281-286).  When the position part offers an additive table of the
    same dtype, its rows are added in the same kernel (k_embed_pos,
    src/cuda_backend.cu:477-483).  params: vocab_size, size."""

    @classmethod
    def declare_weights(cls, params):
        return {"table": WeightDecl((params["vocab_size"], params["size"]), "embedding")}

    def load(self, tensors, store):
        self.table = store.matrix(tensors["table"])

    def forward(self, ctx, out, position=None):
        ptab = position.additive_table() if position is not None else None
        if ptab is not None and ptab.dtype == self.table.dtype:
            ops.embed(ctx.tokens, self.table, out, positions=ctx.positions, pos_table=ptab,
                      err_flag=ctx.err_flag)
        else:
            ops.embed(ctx.tokens, self.table, out, err_flag=ctx.err_flag)
            if position is not None:
                position.apply_embedding(ctx, out)
        return out
