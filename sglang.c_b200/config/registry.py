"""One registry from an architecture's name to its configuration class and
its model plan.

The reference decides by which keys config.json holds (src/model.c:24-41) and
its GPU command line by `model_type` (apps/cuda_cli.c:25-36).  Here the first
entry of `architectures` decides, `model_type` is the fallback, and an unknown
name is an error that lists the known ones.
"""
from dataclasses import dataclass
from typing import Callable, Dict, Tuple

from .base import ConfigError, read_config_json


@dataclass(frozen=True)
class Architecture:
    name: str
    config_class: type            # has from_dict(dict) and to_dict()
    build_plan: Callable          # config -> parts.plan.ModelPlan
    model_types: Tuple[str, ...] = ()


_ARCHITECTURES: Dict[str, Architecture] = {}


def register_architecture(name, config_class, build_plan, model_types=()):
    """Add (or replace) an architecture.  `build_plan(config)` returns the model
    plan: which parts make each layer and in which order layers run."""
    arch = Architecture(name, config_class, build_plan, tuple(model_types))
    _ARCHITECTURES[name] = arch
    return arch


def known_architectures():
    _load_builtin()
    return sorted(_ARCHITECTURES)


def _load_builtin():
    # the built-in architectures register themselves on import
    from .. import models  # noqa: F401


def resolve_architecture(config_dict):
    _load_builtin()
    names = config_dict.get("architectures") or []
    if isinstance(names, str):
        names = [names]
    for n in names:
        if n in _ARCHITECTURES:
            return _ARCHITECTURES[n]
    mt = config_dict.get("model_type")
    if mt is not None:
        for arch in _ARCHITECTURES.values():
            if mt in arch.model_types:
                return arch
    raise ConfigError(
        f"config.json names architectures={names!r}, model_type={mt!r}; "
        f"known architectures: {sorted(_ARCHITECTURES)}")


def load_config(model_dir):
    """(architecture, typed config) of a model folder."""
    d = read_config_json(model_dir)
    arch = resolve_architecture(d)
    return arch, arch.config_class.from_dict(d)
