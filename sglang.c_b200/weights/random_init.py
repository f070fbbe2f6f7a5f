"""Random weights: writes a model folder (config.json, model.safetensors) from a
configuration and a seed.

Every tensor has its own random stream, derived from the seed and the tensor's
name, so a tensor's values do not depend on which other tensors exist.  Two
schemes, chosen by `scheme`:

  "standard"  matrices and tables N(0, 0.02); projections back into the residual
              stream N(0, 0.02/sqrt(2*n_layers)); biases 0; norm gains 1, norm
              biases 0.
  "varied"    matrices, tables and biases N(0, 0.02); norm gains 1 + N(0, 0.1),
              norm biases N(0, 0.02): nothing is zero or one, so a dropped bias
              or gain shows in the output.

(The reference has no generator for this architecture; its pattern for others
is a seeded script that writes a full folder, tests/gen_random_mistral.py.)
"""
import hashlib
import json
import math
import os

import numpy as np
import torch

from ..config.registry import Architecture
from .loader import required_tensors
from .safetensors_io import write_safetensors

SCHEMES = ("standard", "varied")


def _stream(seed, name):
    h = hashlib.sha256(f"{int(seed)}:{name}".encode()).digest()
    return np.random.Generator(np.random.Philox(key=int.from_bytes(h[:8], "little")))


def random_tensor(seed, name, decl, scheme, n_layers, vocab_size=None):
    rng = _stream(seed, name)
    shape = tuple(decl.shape)
    if decl.kind == "int":
        hi = vocab_size or 2
        return torch.from_numpy(rng.integers(0, hi, size=shape, dtype=np.int32))
    std = 0.02
    if decl.init in ("matrix", "embedding"):
        a = rng.standard_normal(shape) * std
    elif decl.init == "residual_matrix":
        s = std if scheme == "varied" else std / math.sqrt(2.0 * n_layers)
        a = rng.standard_normal(shape) * s
    elif decl.init == "bias":
        a = rng.standard_normal(shape) * std if scheme == "varied" else np.zeros(shape)
    elif decl.init == "norm_gain":
        a = 1.0 + rng.standard_normal(shape) * 0.1 if scheme == "varied" else np.ones(shape)
    elif decl.init == "norm_bias":
        a = rng.standard_normal(shape) * std if scheme == "varied" else np.zeros(shape)
    else:
        raise ValueError(f"tensor '{name}': unknown init role '{decl.init}'")
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32))


def write_random_model(out_dir, arch: Architecture, config, seed, scheme="standard",
                       store_dtype="float32"):
    """Write config.json and model.safetensors for `config` (an instance of the
    architecture's configuration class).  `store_dtype` "bfloat16" stores
    matrices and tables in bfloat16 (vectors stay float32)."""
    if scheme not in SCHEMES:
        raise ValueError(f"unknown scheme '{scheme}'; known: {SCHEMES}")
    if store_dtype not in ("float32", "bfloat16"):
        raise ValueError("store_dtype must be float32 or bfloat16")
    plan = arch.build_plan(config)
    need = required_tensors(plan)
    tensors = {}
    for name, decl in need.items():
        t = random_tensor(seed, name, decl, scheme, len(plan.order), plan.vocab_size)
        if store_dtype == "bfloat16" and decl.kind == "float" and len(decl.shape) >= 2:
            t = t.to(torch.bfloat16)
        tensors[name] = t
    os.makedirs(out_dir, exist_ok=True)
    with open(os.path.join(out_dir, "config.json"), "w") as f:
        json.dump(config.to_dict(), f, indent=2, sort_keys=True)
    write_safetensors(os.path.join(out_dir, "model.safetensors"), tensors,
                      metadata={"format": "pt", "seed": seed, "scheme": scheme})
    return out_dir
