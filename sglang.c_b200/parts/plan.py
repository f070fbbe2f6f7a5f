"""The model plan: which parts make a model, as data.

An architecture turns its typed configuration into a `ModelPlan`.  The plan
names parts by `kind` (a key of the part registries), gives each its sizes and
constants as `params`, and maps each part's weight roles to tensor names in the
file.  Layers are listed once; `order` says in which sequence they run and may
name a layer twice, or let a call read the cache that an earlier call wrote.
Nothing in a plan, and no part, knows which architecture it came from.
"""
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple


@dataclass(frozen=True)
class WeightDecl:
    """One tensor a part needs.  `shape` is the shape in the file.  `init`
    names the tensor's role for random initialisation: "matrix",
    "residual_matrix" (a projection back into the residual stream),
    "embedding", "bias", "norm_gain", "norm_bias".  `kind` is "float" or "int"
    (integer tables stay int32)."""
    shape: Tuple[int, ...]
    init: str
    kind: str = "float"


@dataclass
class PartSpec:
    kind: str
    params: Dict = field(default_factory=dict)
    weights: Dict[str, str] = field(default_factory=dict)   # role -> tensor name


# the category of a layer's sub-part when only its role is given
_ROLE_CATEGORY = {"norm1": "norm", "norm2": "norm", "norm": "norm", "mixer": "mixer", "ffn": "feed_forward"}


class LayerPlan:
    """A layer: a `block` (the arrangement) and the sub-parts it arranges, by role.  The roles are
    the block's business: the pre-norm block asks for norm1, mixer, norm2, ffn; another block may
    ask for one norm beside a mixer and a feed-forward, or for a pair of norms behind them.
    `parts` maps role -> (category, PartSpec); the four usual roles can also be given (and later
    replaced) as attributes.  A layer has at most one sub-part of category "mixer": its cache
    need is the layer's."""

    def __init__(self, name, block, norm1=None, mixer=None, norm2=None, ffn=None, parts=None):
        object.__setattr__(self, "name", name)
        object.__setattr__(self, "block", block)
        object.__setattr__(self, "parts", {})
        for role, spec in (("norm1", norm1), ("mixer", mixer), ("norm2", norm2), ("ffn", ffn)):
            if spec is not None:
                self.parts[role] = (_ROLE_CATEGORY[role], spec)
        for role, v in (parts or {}).items():
            setattr(self, role, v)

    def __getattr__(self, role):
        parts = object.__getattribute__(self, "parts")
        if role in parts:
            return parts[role][1]
        raise AttributeError(f"layer '{self.name}' has no sub-part '{role}'")

    def __setattr__(self, role, value):
        if role in ("name", "block"):
            object.__setattr__(self, role, value)
        elif isinstance(value, tuple):
            self.parts[role] = (value[0], value[1])
        else:
            cat = self.parts[role][0] if role in self.parts else _ROLE_CATEGORY.get(role)
            if cat is None:
                raise ValueError(f"sub-part '{role}': give (category, PartSpec), the role alone does not say which")
            self.parts[role] = (cat, value)

    def mixer_role(self):
        roles = [r for r, (cat, _) in self.parts.items() if cat == "mixer"]
        if len(roles) > 1:
            raise ValueError(f"layer '{self.name}' has {len(roles)} mixers; a layer keeps one cache")
        return roles[0] if roles else None


@dataclass(frozen=True)
class LayerCall:
    """One entry of the running order.  `layer` indexes `ModelPlan.layers`.
    `cache_of` is None when this call keeps a cache of its own, else the index
    (in `order`) of the earlier call whose cache it reads without writing."""
    layer: int
    cache_of: Optional[int] = None


@dataclass
class ModelPlan:
    hidden_size: int
    vocab_size: int
    max_positions: int
    embedding: PartSpec
    position: PartSpec
    layers: List[LayerPlan]
    order: List[LayerCall]
    final_norm: PartSpec
    head: PartSpec
    eos_token_id: Optional[int] = None
    # tensor names a checkpoint may hold that the model does not use (fnmatch patterns)
    ignorable: Tuple[str, ...] = ()
    # prefixes to try when a name is not found as written
    name_prefixes: Tuple[str, ...] = ("",)

    def part_specs(self):
        yield self.embedding
        yield self.position
        for layer in self.layers:
            for _, spec in layer.parts.values():
                yield spec
        yield self.final_norm
        yield self.head
