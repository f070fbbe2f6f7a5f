"""A model built from a plan: parts are looked up in the registries by kind,
given their params, and bound to the tensors the plan names.  The forward pass
walks the plan's running order; nothing here knows an architecture."""
from dataclasses import dataclass

import torch

from ..parts.registry import get_part
from ..weights.loader import DeviceStore, load_checked


@dataclass
class Layer:
    name: str
    block: object
    norm1: object
    mixer: object
    norm2: object
    ffn: object


class Model:
    def __init__(self, plan, runtime):
        self.plan = plan
        self.rt = runtime
        mk = lambda cat, spec: get_part(cat, spec.kind)(spec.params, runtime)
        self.embedding = mk("embedding", plan.embedding)
        self.position = mk("position", plan.position)
        self.layers = [Layer(lp.name, mk("block", lp.block), mk("norm", lp.norm1),
                             mk("mixer", lp.mixer), mk("norm", lp.norm2), mk("feed_forward", lp.ffn))
                       for lp in plan.layers]
        self.final_norm = mk("norm", plan.final_norm)
        self.head = mk("head", plan.head)
        for i, call in enumerate(plan.order):
            if not (0 <= call.layer < len(self.layers)):
                raise ValueError(f"running order entry {i} names layer {call.layer}, which does not exist")
            if call.cache_of is not None and not (0 <= call.cache_of < i):
                raise ValueError(f"running order entry {i} reads the cache of entry {call.cache_of}, "
                                 "which must come earlier")
        self.weight_bytes = 0
        # a part that reads per-step host values (not only device arrays) cannot be replayed
        parts = [self.embedding, self.position, self.final_norm, self.head]
        for layer in self.layers:
            parts += [layer.block, layer.norm1, layer.mixer, layer.norm2, layer.ffn]
        self.graph_safe = all(getattr(p, "graph_safe", True) for p in parts)

    def load(self, model_dir):
        refs = load_checked(self.plan, model_dir)
        store = DeviceStore(self.rt)
        pairs = [(self.embedding, self.plan.embedding), (self.position, self.plan.position)]
        for layer, lp in zip(self.layers, self.plan.layers):
            pairs += [(layer.norm1, lp.norm1), (layer.mixer, lp.mixer), (layer.norm2, lp.norm2),
                      (layer.ffn, lp.ffn)]
        pairs += [(self.final_norm, self.plan.final_norm), (self.head, self.plan.head)]
        for part, spec in pairs:
            part.load({role: refs[name] for role, name in spec.weights.items()}, store)
        self.weight_bytes = store.bytes
        return self

    def cache_needs(self):
        """(need per call of the running order, cache_of per call)."""
        needs = [self.layers[c.layer].mixer.cache_need() for c in self.plan.order]
        return needs, [c.cache_of for c in self.plan.order]

    def forward(self, ctx, cache, logits_out):
        """Run the step's tokens through every call of the running order; write
        the logits of the wanted rows into logits_out[:n_want]."""
        E = self.plan.hidden_size
        x = ctx.alloc((ctx.T, E), torch.float32)          # the residual stream, 32-bit
        self.embedding.forward(ctx, x, self.position)
        for i, call in enumerate(self.plan.order):
            layer = self.layers[call.layer]
            layer.block.forward(ctx, x, layer, cache.binding(i), self.position)
        if ctx.n_want > 0:
            hf = ctx.alloc((ctx.n_want, E), self.rt.act_dtype)
            self.final_norm.forward(ctx, x, hf, rows=ctx.want_rows)
            self.head.forward(ctx, hf, logits_out[:ctx.n_want])
        return logits_out[:ctx.n_want]
