"""What a mixer may ask of the cache manager.

Two kinds of per-request memory exist, as in the reference's hybrid cache
(src/kvcache.h:8-21,33-56: a KV region that grows with the position, and a
recurrent/conv state of fixed size per layer):

* :class:`PagedKVSpec` — keys and values that grow with the tokens; kept in
  pages.  Mixers with the same (kv heads, head dim, window) form a *group*
  that shares block tables; groups with different needs have pages of their
  own.  A windowed group may keep the first ``keep_first`` keys of every
  sequence readable: the pages that hold them are never given back early.
* :class:`StateSpec` — a fixed-size tensor per request; kept in a slot.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple


@dataclass(frozen=True)
class PagedKVSpec:
    num_kv_heads: int
    head_dim: int
    window: Optional[int] = None      # keys older than this many positions are never read again
    block: Optional[int] = None       # a position reads no key from before its own block of this many positions
    keep_first: int = 0               # with a window: the first keys of a sequence stay readable for good

    @property
    def group_key(self) -> Tuple:
        key = ("kv", self.num_kv_heads, self.head_dim, self.window)
        if self.block is not None:
            key += (("block", self.block),)
        if self.keep_first and self.window is not None:
            key += (("keep_first", self.keep_first),)
        return key


@dataclass(frozen=True)
class StateSpec:
    shape: Tuple[int, ...]            # per request
    dtype: str = "float32"
