"""tensor.BlockPool (tensor/blockpool.go:46-133) through the C ABI: a host-side free-list page
allocator for a paged KV cache.  It never evicts."""
from __future__ import annotations

import ctypes as C
from typing import List, Optional, Sequence

import numpy as np

from . import _lib


class BlockPool:
    def __init__(self, blocks: int, positions_per_block: int):
        self._h = None
        h = C.c_void_p()
        _lib.check(_lib.lib().ab_blockpool_new(blocks, positions_per_block, C.byref(h)))
        self._h = h
        self._blocks = blocks

    def close(self):
        if getattr(self, "_h", None):
            _lib.lib().ab_blockpool_close(self._h)
            self._h = None

    __del__ = close

    def block_size(self) -> int:
        return _lib.lib().ab_blockpool_block_size(self._h)

    def available(self) -> int:
        return _lib.lib().ab_blockpool_available(self._h)

    def grow(self, pages: Optional[Sequence[int]], n: int) -> List[int]:
        """Pages addressing n positions: the given pages, unmoved, then as many new ones as needed."""
        pages = [] if pages is None else list(pages)
        buf = np.zeros(len(pages) + self._blocks + 1, np.uint32)
        buf[:len(pages)] = pages
        r = _lib.check(_lib.lib().ab_blockpool_grow(self._h, buf.ctypes.data, len(pages), n))
        return [int(x) for x in buf[:r]]

    def free(self, pages: Sequence[int]):
        arr = np.ascontiguousarray(list(pages), dtype=np.uint32)
        _lib.check(_lib.lib().ab_blockpool_free(self._h, arr.ctypes.data, arr.size))

    def positions(self, pages: Sequence[int]) -> int:
        return _lib.lib().ab_blockpool_positions(self._h, len(pages))
