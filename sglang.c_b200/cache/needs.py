"""What a mixer asks of the cache manager."""
from dataclasses import dataclass
from typing import Optional, Tuple


@dataclass(frozen=True)
class CacheNeed:
    """kind "paged_kv": keys and values of every position (or of the last
    `window` positions) in pages; kind "state": one block of fixed shape per
    request.  Calls whose needs are equal share a group: one page id (or slot
    id) is valid in all of them."""
    kind: str
    n_kv_heads: int = 0
    head_dim: int = 0
    window: Optional[int] = None
    state_shape: Tuple[int, ...] = ()
    state_dtype: str = "float32"

    @classmethod
    def paged_kv(cls, n_kv_heads, head_dim, window=None):
        if window is not None and window <= 0:
            raise ValueError("window must be a positive count of keys or None")
        return cls("paged_kv", int(n_kv_heads), int(head_dim), None if window is None else int(window))

    @classmethod
    def state(cls, shape, dtype="float32"):
        return cls("state", state_shape=tuple(int(s) for s in shape), state_dtype=dtype)


@dataclass
class CacheBinding:
    """What a mixer call gets: its own tensor and the group whose block tables
    (or slot ids) index it.  paged_kv: tensor [n_pages, 2, n_kv_heads,
    page_size, head_dim]; state: tensor [n_slots, *state_shape].  `write` is
    false for a call that reads the cache another call wrote."""
    kind: str
    group: int
    tensor: object
    write: bool = True
