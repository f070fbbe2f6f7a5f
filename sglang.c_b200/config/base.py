"""Reading config.json into typed values.

The reference reads config.json whole, parses it to a tree and pulls numbers
out by key with defaults (src/gguf.c:1321-1337, src/json.c:267-300,
src/gpt2.c:37-42).  Here every size must be present in the file; only switches
whose absence has a meaning defined by the architecture have defaults.
"""
import json
import os


class ConfigError(ValueError):
    """A config.json that cannot be used; the message names the key."""


_MISSING = object()


def read_config_json(model_dir):
    path = os.path.join(model_dir, "config.json")
    try:
        with open(path) as f:
            d = json.load(f)
    except FileNotFoundError:
        raise ConfigError(f"no config.json in {model_dir}") from None
    except json.JSONDecodeError as e:
        raise ConfigError(f"{path}: not valid JSON ({e})") from None
    if not isinstance(d, dict):
        raise ConfigError(f"{path}: top level must be an object")
    return d


def _lookup(d, keys):
    for k in keys:
        if k in d and d[k] is not None:
            return k, d[k]
    return keys[0], _MISSING


def get_int(d, keys, default=_MISSING, minimum=None):
    """An integer under the first of `keys` that is present.  JSON booleans and
    floats with an integral value are accepted, as the reference's reader does
    (src/json.c:284-292)."""
    keys = [keys] if isinstance(keys, str) else list(keys)
    k, v = _lookup(d, keys)
    if v is _MISSING:
        if default is _MISSING:
            raise ConfigError(f"config.json: key '{keys[0]}' is required")
        return default
    if isinstance(v, bool):
        v = int(v)
    if isinstance(v, float) and v == int(v):
        v = int(v)
    if not isinstance(v, int):
        raise ConfigError(f"config.json: key '{k}' must be an integer, got {v!r}")
    if minimum is not None and v < minimum:
        raise ConfigError(f"config.json: key '{k}' must be >= {minimum}, got {v}")
    return v


def get_float(d, keys, default=_MISSING, positive=False):
    keys = [keys] if isinstance(keys, str) else list(keys)
    k, v = _lookup(d, keys)
    if v is _MISSING:
        if default is _MISSING:
            raise ConfigError(f"config.json: key '{keys[0]}' is required")
        return default
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        raise ConfigError(f"config.json: key '{k}' must be a number, got {v!r}")
    v = float(v)
    if positive and not v > 0:
        raise ConfigError(f"config.json: key '{k}' must be > 0, got {v}")
    return v


def get_bool(d, keys, default=_MISSING):
    keys = [keys] if isinstance(keys, str) else list(keys)
    k, v = _lookup(d, keys)
    if v is _MISSING:
        if default is _MISSING:
            raise ConfigError(f"config.json: key '{keys[0]}' is required")
        return default
    if isinstance(v, bool):
        return v
    if isinstance(v, int) and v in (0, 1):
        return bool(v)
    raise ConfigError(f"config.json: key '{k}' must be true or false, got {v!r}")


def get_str(d, keys, default=_MISSING, choices=None):
    keys = [keys] if isinstance(keys, str) else list(keys)
    k, v = _lookup(d, keys)
    if v is _MISSING:
        if default is _MISSING:
            raise ConfigError(f"config.json: key '{keys[0]}' is required")
        v = default
    if not isinstance(v, str):
        raise ConfigError(f"config.json: key '{k}' must be a string, got {v!r}")
    if choices is not None and v not in choices:
        raise ConfigError(f"config.json: key '{k}' is '{v}', known values: {sorted(choices)}")
    return v
