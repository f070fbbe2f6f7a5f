"""Position encodings.  A position part can act at the embedding (a table added
to the token rows), inside a mixer (a change of queries and keys), or both."""
from ..csrc import ops
from .base import Part
from .plan import WeightDecl
from .registry import register_part


class PositionEncoding(Part):
    def additive_table(self):
        return None

    def apply_embedding(self, ctx, x):
        pass

    def rotate(self, ctx, q, k):
        pass


@register_part("position", "none")
class NoPositions(PositionEncoding):
    pass


@register_part("position", "learned_absolute")
class LearnedAbsolutePositions(PositionEncoding):
    """x[t,:] += table[pos[t],:]  (reference src/gpt2.c:212-216).
    params: max_positions, size."""

    @classmethod
    def declare_weights(cls, params):
        return {"table": WeightDecl((params["max_positions"], params["size"]), "embedding")}

    def load(self, tensors, store):
        self.table = store.matrix(tensors["table"])

    def additive_table(self):
        return self.table

    def apply_embedding(self, ctx, x):
        ops.add_rows(x, ctx.positions, self.table)
