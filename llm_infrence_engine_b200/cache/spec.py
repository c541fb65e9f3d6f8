"""What a mixer asks of the cache: pages of keys and values, or a state of fixed size, or nothing."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple


@dataclass(frozen=True)
class PagedKVSpec:
    """Keys and values of every cached token (or of the last ``window`` of them), kept in pages."""

    num_kv_heads: int
    head_dim: int
    window: Optional[int] = None  # None: all keys are kept; n: only keys p - n < j <= p are ever read
    v_head_dim: Optional[int] = None  # size of a value row; None: as the keys; 0: no value pool (values are read out of the key rows)
    keep_first: int = 0           # with a window: keys at positions below this are read for ever, whatever the window
    chunk: Optional[int] = None   # n: position p reads only keys from floor(p / n) * n on (runs of n positions from the request's start)


@dataclass(frozen=True)
class FixedStateSpec:
    """A per-request tensor of fixed shape that a mixer reads and writes in place (32-bit floats)."""

    shape: Tuple[int, ...]


def flatten_specs(spec) -> tuple:
    """The single specs of what a mixer asks for: a mixer may ask for several things at once (pages and a state, two states)
    by giving a tuple, which may nest; ``None`` asks for nothing."""
    if spec is None:
        return ()
    if isinstance(spec, (tuple, list)):
        return tuple(x for part in spec for x in flatten_specs(part))
    return (spec,)


NULL_PAGE = 0  # never handed out; block tables point at it where a request holds no page
