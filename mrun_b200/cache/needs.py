"""What a mixer asks of the cache manager.

A mixer declares one *need* (or none).  Needs with the same ``group_key`` share a page pool and a
block table per request; each schedule entry still has tensors of its own inside the group.
The reference draws the same line per layer between key/value state that grows with the
sequence and recurrent state of fixed size (``LayerState::{Kv, Recurrent}``,
crates/mrun-engine/src/state.rs:87-117).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple


@dataclass(frozen=True)
class PagedKV:
    """Keys and values of every token (``window`` None) or of the last ``window`` tokens.
    ``value_dim``: the values' feature size where it differs from the keys' (``head_dim``)."""

    kv_heads: int
    head_dim: int
    window: Optional[int] = None
    value_dim: Optional[int] = None

    def group_key(self) -> tuple:
        return ("paged", self.window)


@dataclass(frozen=True)
class PagedLatent:
    """One row of ``width`` features per token that serves as the key and as the value of a
    single key/value head (an attention over a shared latent): one tensor of pages, which the
    entry's ``k`` and ``v`` both name.  Shares the pages' books with :class:`PagedKV` of the same
    window."""

    width: int
    window: Optional[int] = None

    def group_key(self) -> tuple:
        return ("paged", self.window)


@dataclass(frozen=True)
class PagedMaps:
    """Keys of ``maps`` attention maps and values cut into ``value_chunks`` chunks a token and kv
    head: key pages [maps, pages, kv_heads, page_size, key_dim] and value pages [value_chunks,
    pages, kv_heads, page_size, value_chunk_dim], so that every map and every chunk is a page
    tensor of the :class:`PagedKV` shape.  Shares the pages' books with :class:`PagedKV` of the
    same window."""

    maps: int
    kv_heads: int
    key_dim: int
    value_chunks: int
    value_chunk_dim: int
    window: Optional[int] = None

    def group_key(self) -> tuple:
        return ("paged", self.window)


@dataclass(frozen=True)
class FixedState:
    """Per-request state of a fixed shape, zero when a request starts.  A part that keeps several
    states gives each a ``name`` and declares them together (see :func:`split_need`)."""

    shape: Tuple[int, ...]
    dtype: str = "float32"
    name: str = "state"

    def group_key(self) -> tuple:
        return ("state",)


PAGED = (PagedKV, PagedLatent, PagedMaps)


def split_need(need):
    """A part's need may be one need, None, or a tuple of at most one paged need and any number
    of :class:`FixedState` with different names: returns (paged need or None, the states)."""
    if need is None:
        return None, ()
    items = tuple(need) if isinstance(need, (tuple, list)) else (need,)
    paged = [n for n in items if isinstance(n, PAGED)]
    states = tuple(n for n in items if isinstance(n, FixedState))
    if len(paged) > 1:
        raise TypeError("a schedule entry may have one paged cache need")
    if len(paged) + len(states) != len(items):
        raise TypeError(f"unknown cache need among {items!r}")
    if len({s.name for s in states}) != len(states):
        raise TypeError("the states of a schedule entry need different names")
    return (paged[0] if paged else None), states
