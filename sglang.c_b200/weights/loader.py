"""Weights by tensor name.

A plan's parts declare the tensors they need (name, shape in the file, kind);
the loader checks the whole file against that list before anything is moved
and raises ONE error that lists missing tensors, unexpected tensors and wrong
shapes.  (The reference fetches tensors by name with expected shapes,
src/gpt2.c:61-96, but checks only four of them for presence, :65-68,98-102.)

Tensors keep their stored precision on the host.  On the device, matrices are
float32 in the 32-bit runtime and bfloat16 in the bfloat16 runtime; vectors
(norm gains, biases) are float32 in both, which changes no stored value;
integer tables are int32.
"""
import fnmatch
import os
from dataclasses import dataclass

import torch

from ..parts.registry import get_part
from .safetensors_io import SafetensorsError, SafetensorsFile


class WeightError(ValueError):
    pass


@dataclass
class TensorRef:
    name: str           # name in the file, as found
    tensor: torch.Tensor


def required_tensors(plan):
    """name -> WeightDecl over all parts; a name used by several parts (a tied
    head) must be declared with one shape."""
    need = {}
    for spec in plan.part_specs():
        cls = get_part(_category_of(plan, spec), spec.kind)
        decls = cls.declare_weights(spec.params)
        for role, decl in decls.items():
            if role not in spec.weights:
                raise WeightError(f"plan gives no tensor name for role '{role}' of part '{spec.kind}'")
            name = spec.weights[role]
            if name in need and need[name].shape != decl.shape:
                raise WeightError(f"tensor '{name}' is declared with shapes {need[name].shape} and {decl.shape}")
            need.setdefault(name, decl)
    return need


def _category_of(plan, spec):
    if spec is plan.embedding:
        return "embedding"
    if spec is plan.position:
        return "position"
    if spec is plan.final_norm:
        return "norm"
    if spec is plan.head:
        return "head"
    for layer in plan.layers:
        for cat, s in layer.parts.values():
            if spec is s:
                return cat
    raise WeightError("part spec does not belong to the plan")


class ShardedWeights:
    """The shards that `model.safetensors.index.json` names, seen as one file: its `weight_map`
    gives the shard of every tensor (the reference resolves a folder the same way, index first:
    src/safetensors.c:676-843).  A tensor the index names must be in the shard it names; tensors a
    shard holds beyond the index are not visible."""

    def __init__(self, model_dir, index_path):
        import json
        self.path = index_path
        try:
            with open(index_path) as f:
                index = json.load(f)
            wmap = index["weight_map"]
            if not isinstance(wmap, dict) or not wmap:
                raise KeyError("weight_map")
        except (OSError, ValueError, KeyError, TypeError) as e:
            raise WeightError(f"{index_path}: not a shard index with a weight_map ({e})") from None
        self._files = {}
        self._where = {}
        try:
            for name, shard in wmap.items():
                if not isinstance(shard, str) or os.path.basename(shard) != shard:
                    raise WeightError(f"{index_path}: shard name {shard!r} of tensor '{name}' must be a file name "
                                      "in the same folder")
                if shard not in self._files:
                    sp = os.path.join(model_dir, shard)
                    if not os.path.exists(sp):
                        raise WeightError(f"{index_path} names shard {shard}, which is not in {model_dir}")
                    self._files[shard] = SafetensorsFile(sp)
                self._where[name] = self._files[shard]
            lost = [n for n, f in self._where.items() if n not in set(f.names())]
            if lost:
                raise WeightError(f"{index_path}: tensors not found in the shard it names: " + ", ".join(sorted(lost)))
        except SafetensorsError as e:
            self.close()
            raise WeightError(str(e)) from None
        except WeightError:
            self.close()
            raise

    def names(self):
        return list(self._where)

    def shape(self, name):
        return self._where[name].shape(name)

    def dtype(self, name):
        return self._where[name].dtype(name)

    def tensor(self, name):
        return self._where[name].tensor(name)

    def close(self):
        for f in self._files.values():
            f.close()


def open_weights(model_dir):
    """(weights, path for messages): the shards of model.safetensors.index.json if the folder
    has that index, else model.safetensors."""
    index = os.path.join(model_dir, "model.safetensors.index.json")
    if os.path.exists(index):
        return ShardedWeights(model_dir, index), index
    path = os.path.join(model_dir, "model.safetensors")
    if not os.path.exists(path):
        raise WeightError(f"no model.safetensors (or model.safetensors.index.json) in {model_dir}")
    try:
        return SafetensorsFile(path), path
    except SafetensorsError as e:
        raise WeightError(str(e)) from None


def load_checked(plan, model_dir):
    """{declared name: TensorRef} after checking the file against the plan."""
    need = required_tensors(plan)
    f, where = open_weights(model_dir)
    try:
        names = set(f.names())
        found = {}
        missing, wrong = [], []
        for name, decl in need.items():
            actual = next((p + name for p in plan.name_prefixes if p + name in names), None)
            if actual is None:
                missing.append(name)
                continue
            found[name] = actual
            if tuple(f.shape(actual)) != tuple(decl.shape):
                wrong.append(f"{actual}: file has {list(f.shape(actual))}, model needs {list(decl.shape)}")
            elif decl.kind == "float" and not f.dtype(actual).is_floating_point:
                wrong.append(f"{actual}: file has {f.dtype(actual)}, model needs a floating-point tensor")
            elif decl.kind == "int" and f.dtype(actual).is_floating_point:
                wrong.append(f"{actual}: file has {f.dtype(actual)}, model needs an integer tensor")
        used = set(found.values())
        unexpected = []
        for n in sorted(names - used):
            bare = n
            for p in plan.name_prefixes:
                if p and n.startswith(p):
                    bare = n[len(p):]
            if not any(fnmatch.fnmatchcase(bare, pat) for pat in plan.ignorable):
                unexpected.append(n)
        if missing or wrong or unexpected:
            lines = [f"{where} does not fit the model:"]
            if missing:
                lines.append(f"  missing tensors ({len(missing)}): " + ", ".join(sorted(missing)))
            if unexpected:
                lines.append(f"  unexpected tensors ({len(unexpected)}): " + ", ".join(unexpected))
            if wrong:
                lines.append(f"  wrong shape or type ({len(wrong)}):")
                lines.extend("    " + w for w in wrong)
            raise WeightError("\n".join(lines))
        out = {}
        for name, actual in found.items():
            t = f.tensor(actual)
            if t.dtype == torch.float16:
                t = t.to(torch.float32)          # exact; the device side has float32 and bfloat16
            elif t.dtype == torch.float64:
                t = t.to(torch.float32)
            elif t.dtype in (torch.int64, torch.uint8):
                t = t.to(torch.int32)
            out[name] = TensorRef(actual, t)
        return out
    finally:
        f.close()


class DeviceStore:
    """Moves tensors to the device in the runtime's precision, once per
    (tensor, form): parts that name the same tensor share it."""

    def __init__(self, runtime):
        self.rt = runtime
        self._cache = {}
        self.bytes = 0
        self.in_layer = False              # set by the model while a layer's parts load
        self.largest_layer_matrix = 0      # elements of the largest matrix a layer's part took

    def _put(self, key, make):
        t = self._cache.get(key)
        if t is None:
            t = make()
            self._cache[key] = t
            self.bytes += t.numel() * t.element_size()
        return t

    def matrix(self, ref, transpose=False):
        """A 2-D weight in the runtime's matrix precision, optionally transposed
        ([in,out] in the file -> [out,in] on the device)."""
        def make():
            t = ref.tensor
            if transpose:
                t = t.t()
            return t.to(self.rt.matrix_dtype).contiguous().to(self.rt.device)
        t = self._put((ref.name, "matrix", transpose), make)
        if self.in_layer:
            self.largest_layer_matrix = max(self.largest_layer_matrix, t.numel())
        return t

    def vector(self, ref):
        return self._put((ref.name, "vector"),
                         lambda: ref.tensor.to(torch.float32).contiguous().to(self.rt.device))

    def int_table(self, ref):
        return self._put((ref.name, "int"),
                         lambda: ref.tensor.to(torch.int32).contiguous().to(self.rt.device))

    def raw(self, ref, dtype=None):
        return self._put((ref.name, "raw", dtype),
                         lambda: (ref.tensor if dtype is None else ref.tensor.to(dtype)).contiguous().to(self.rt.device))
