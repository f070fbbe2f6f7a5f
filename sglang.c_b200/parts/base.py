"""What every part is: a class built from its `params` (sizes and constants) and
a runtime (device and precision), which declares the tensors it needs, takes
them at load, and runs on a step context.  A part never sees a model
configuration or another layer.

Interfaces by category (ctx is an `engine.step.StepContext`):

  embedding     forward(ctx, out, position)      out[T,E] float32 = rows of the table for
                                                 ctx.tokens, plus the position part's
                                                 additive table when it has one
  position      additive_table() -> tensor|None  a [P,E] table added at the embedding
                apply_embedding(ctx, x)          in-place change of x after the gather
                rotate(ctx, q, k)                in-place change of queries/keys in a mixer
  norm          forward(ctx, x, out, rows=None)  out = norm(x[rows]) ; x float32 residual
  mixer         cache_need() -> CacheNeed|None   what it keeps per request
                forward(ctx, h, residual, cache, position)
                                                 residual += mix(h) using `cache`
                                                 (a cache.CacheBinding, or None)
  feed_forward  forward(ctx, h, residual)        residual += ff(h)
  block         forward(ctx, x, layer, cache, position)
                                                 runs norm1/mixer/norm2/ffn of `layer` on x
  head          forward(ctx, h, out)             out[W,V] float32 logits of h[W,E]
"""
from typing import Dict

import torch

from .plan import WeightDecl  # noqa: F401  (re-exported for part authors)


class Part:
    category = None
    kind = None
    # False for a part whose forward reads per-step values on the host (ctx.h_*): a step
    # that holds such a part is never captured into a CUDA graph
    graph_safe = True

    def __init__(self, params, runtime):
        self.params = dict(params)
        self.rt = runtime

    @classmethod
    def declare_weights(cls, params) -> Dict[str, WeightDecl]:
        """role -> WeightDecl for the given params."""
        return {}

    def load(self, tensors, store):
        """Take the tensors (`role -> weights.TensorRef`).  `store` moves them to
        the device in the runtime's precision and shares a tensor that several
        parts name."""

    def cache_need(self):
        return None

    def workspace_per_token(self, *args):
        """Bytes per token of the step that this part takes from ctx.alloc while it runs (a
        block gets its built layer as argument and answers for the whole layer).  The engine
        sizes the step workspace from the answers."""
        return 0

    def graph_bound(self, ctx):
        """Mixers only: an upper bound of the context length for this step's launches, if the
        mixer's kernels want another than the next power of two (None: no wish)."""
        return None
