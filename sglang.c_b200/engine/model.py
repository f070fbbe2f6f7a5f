"""A model built from a plan: parts are looked up in the registries by kind,
given their params, and bound to the tensors the plan names.  The forward pass
walks the plan's running order; nothing here knows an architecture."""
import torch

from ..parts.registry import get_part
from ..weights.loader import DeviceStore, load_checked


class Layer:
    """A built layer: `block` and the built sub-parts as attributes named by their roles."""

    def __init__(self, name, block, parts, mixer_role):
        self.name, self.block, self.parts = name, block, parts
        self.mixer_role = mixer_role
        for role, part in parts.items():
            setattr(self, role, part)

    @property
    def the_mixer(self):
        return self.parts[self.mixer_role] if self.mixer_role is not None else None


class Model:
    def __init__(self, plan, runtime):
        self.plan = plan
        self.rt = runtime
        mk = lambda cat, spec: get_part(cat, spec.kind)(spec.params, runtime)
        self.embedding = mk("embedding", plan.embedding)
        self.position = mk("position", plan.position)
        self.layers = [Layer(lp.name, mk("block", lp.block),
                             {role: mk(cat, spec) for role, (cat, spec) in lp.parts.items()}, lp.mixer_role())
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
            parts += [layer.block] + list(layer.parts.values())
        self.graph_safe = all(getattr(p, "graph_safe", True) for p in parts)
        self.largest_layer_matrix = 0     # elements of the largest matrix a layer holds (set by load)

    def load(self, model_dir):
        refs = load_checked(self.plan, model_dir)
        store = DeviceStore(self.rt)
        pairs = [(self.embedding, self.plan.embedding), (self.position, self.plan.position)]
        n_head = len(pairs)
        for layer, lp in zip(self.layers, self.plan.layers):
            pairs += [(layer.parts[role], spec) for role, (_, spec) in lp.parts.items()]
        n_layers_end = len(pairs)
        pairs += [(self.final_norm, self.plan.final_norm), (self.head, self.plan.head)]
        for i, (part, spec) in enumerate(pairs):
            store.in_layer = n_head <= i < n_layers_end
            part.load({role: refs[name] for role, name in spec.weights.items()}, store)
        self.weight_bytes = store.bytes
        self.largest_layer_matrix = store.largest_layer_matrix
        return self

    def cache_needs(self):
        """(need per call of the running order, cache_of per call)."""
        mixers = [self.layers[c.layer].the_mixer for c in self.plan.order]
        needs = [m.cache_need() if m is not None else None for m in mixers]
        return needs, [c.cache_of for c in self.plan.order]

    def workspace_per_token(self):
        """Bytes of step workspace a token needs: the 32-bit residual stream, the widest layer (as
        its block says), and the final norm's rows."""
        E = self.plan.hidden_size
        act = 4 if self.rt.dtype == "float32" else 2
        blocks = [layer.block.workspace_per_token(layer) for layer in self.layers]
        return 4 * E + max(blocks + [0]) + act * E

    def graph_bound(self, ctx):
        """The upper bound of the context length that this step's kernels are launched for (a
        captured graph serves until the contexts pass it): the next power of two, unless a mixer
        asks for a tighter one."""
        bound = 128
        while bound < ctx.max_keys:
            bound *= 2
        asked = [b for b in (layer.the_mixer.graph_bound(ctx) for layer in self.layers
                             if layer.the_mixer is not None) if b is not None]
        if asked:
            bound = max(asked)
        return min(bound, self.plan.max_positions)

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
