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


@dataclass
class LayerPlan:
    name: str
    block: PartSpec            # the arrangement of the four parts below
    norm1: PartSpec
    mixer: PartSpec
    norm2: PartSpec
    ffn: PartSpec


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
            yield layer.norm1
            yield layer.mixer
            yield layer.norm2
            yield layer.ffn
        yield self.final_norm
        yield self.head
