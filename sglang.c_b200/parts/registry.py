"""Registries of parts, one per category.  A plan names a part by category and
`kind`; building a model looks the class up here.  Anything registered from
outside the package (a test's toy mixer, a new feed-forward) is used the same
way as the built-in parts."""
CATEGORIES = ("embedding", "position", "norm", "mixer", "feed_forward", "block", "head")
_REGISTRY = {c: {} for c in CATEGORIES}


def register_part(category, kind, cls=None):
    """Register `cls` under (category, kind).  Usable as a decorator:
    `@register_part("mixer", "my_mixer")`."""
    if category not in _REGISTRY:
        raise KeyError(f"unknown part category '{category}'; categories: {CATEGORIES}")

    def deco(c):
        _REGISTRY[category][kind] = c
        c.category = category
        c.kind = kind
        return c

    return deco(cls) if cls is not None else deco


def get_part(category, kind):
    _load_builtin()
    try:
        return _REGISTRY[category][kind]
    except KeyError:
        raise KeyError(f"no {category} part named '{kind}'; registered: "
                       f"{sorted(_REGISTRY.get(category, {}))}") from None


def registered(category):
    _load_builtin()
    return sorted(_REGISTRY[category])


def _load_builtin():
    from . import (attention, block, embedding, feed_forward, head, norm,  # noqa: F401
                   position)
