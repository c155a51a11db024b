"""Paged KV bookkeeping: reference-counted block pool, per-sequence block tables, automatic prefix cache.

Thin ctypes layer over the C++ implementation (csrc/host/kv_cache.cpp).  Semantics follow the reference driver
(crates/poot-llm/src/driver/block_table.rs:18-303, prefix_cache.rs:15-250): blocks of 16 positions, KV reserved
for prompt + max_tokens at open (never preempt), prefix match at admit, registration of full prompt blocks at
release, the cache holding one reference per cached block, ``evict_unused`` dropping blocks only the cache holds.
"""
from __future__ import annotations

import ctypes
from ctypes import c_int, c_uint64, c_void_p
from typing import List, Optional, Sequence

import numpy as np

from ..ops._lib import host

BLOCK = 16
BASE_IDENTITY = 0


def _lib():
    lib = host()
    if not getattr(lib, "_kv_bound", False):
        P = c_void_p
        lib.poot_pool_new.restype = P
        lib.poot_pool_new.argtypes = [c_int]
        lib.poot_pool_free.argtypes = [P]
        for n in ("poot_pool_available", "poot_pool_total"):
            getattr(lib, n).argtypes = [P]
        lib.poot_pool_refcount.argtypes = [P, c_int]
        lib.poot_pool_alloc.argtypes = [P, c_int, P]
        lib.poot_pool_retain.argtypes = [P, c_int]
        lib.poot_pool_release.argtypes = [P, c_int]
        lib.poot_prefix_new.restype = P
        lib.poot_prefix_free.argtypes = [P]
        lib.poot_prefix_force_collisions.argtypes = [P, c_int]
        lib.poot_prefix_len.argtypes = [P]
        lib.poot_prefix_hit_tokens.argtypes = [P]
        lib.poot_prefix_hit_tokens.restype = c_uint64
        lib.poot_prefix_query_tokens.argtypes = [P]
        lib.poot_prefix_query_tokens.restype = c_uint64
        lib.poot_prefix_match.argtypes = [P, P, c_uint64, P, c_int, c_int, P]
        lib.poot_prefix_register.argtypes = [P, P, c_uint64, P, c_int, P, c_int]
        lib.poot_prefix_evict_unused.argtypes = [P, P, c_int]
        lib.poot_prefix_drop_identity.argtypes = [P, P, c_uint64]
        lib.poot_prefix_count_unused.argtypes = [P, P]
        lib.poot_chain_hash.argtypes = [c_uint64, P]
        lib.poot_chain_hash.restype = c_uint64
        lib.poot_chain_root.restype = c_uint64
        lib._kv_bound = True
    return lib


class OutOfBlocks(RuntimeError):
    """The pool cannot reserve the blocks a sequence needs (admission waits; nothing is preempted)."""


class BlockPool:
    def __init__(self, num_blocks: int):
        self.lib = _lib()
        self.h = self.lib.poot_pool_new(num_blocks)
        self.num_blocks = num_blocks

    def __del__(self):
        if getattr(self, "h", None):
            self.lib.poot_pool_free(self.h)
            self.h = None

    @property
    def available(self) -> int:
        return self.lib.poot_pool_available(self.h)

    def refcount(self, b: int) -> int:
        return self.lib.poot_pool_refcount(self.h, b)

    def alloc(self, n: int) -> List[int]:
        if n == 0:
            return []
        out = (ctypes.c_int32 * n)()
        if self.lib.poot_pool_alloc(self.h, n, out) != n:
            raise OutOfBlocks(f"need {n} blocks, {self.available} free")
        return list(out)

    def retain(self, b: int) -> None:
        self.lib.poot_pool_retain(self.h, b)

    def release(self, b: int) -> int:
        r = self.lib.poot_pool_release(self.h, b)
        if r < 0:
            raise RuntimeError(f"double free of block {b}")
        return r


class PrefixCache:
    def __init__(self, pool: BlockPool):
        self.lib, self.pool = _lib(), pool
        self.h = self.lib.poot_prefix_new()

    def __del__(self):
        if getattr(self, "h", None):
            self.lib.poot_prefix_free(self.h)
            self.h = None

    def __len__(self) -> int:
        return self.lib.poot_prefix_len(self.h)

    @property
    def hit_tokens(self) -> int:
        return int(self.lib.poot_prefix_hit_tokens(self.h))

    @property
    def query_tokens(self) -> int:
        return int(self.lib.poot_prefix_query_tokens(self.h))

    def match(self, tokens: Sequence[int], identity: int = BASE_IDENTITY, max_blocks: Optional[int] = None) -> List[int]:
        """Blocks of the longest cached whole-block prefix (each retained for the caller).  The last prompt token is
        never served from the cache: at least one token must run to produce logits."""
        toks = np.ascontiguousarray(tokens, dtype=np.uint32)
        limit = (len(toks) - 1) // BLOCK if len(toks) else 0
        if max_blocks is not None:
            limit = min(limit, max_blocks)
        if limit <= 0:
            self.lib.poot_prefix_match(self.h, self.pool.h, identity, toks.ctypes.data, len(toks), 0, None)
            return []
        out = (ctypes.c_int32 * limit)()
        n = self.lib.poot_prefix_match(self.h, self.pool.h, identity, toks.ctypes.data, len(toks), limit, out)
        return list(out[:n])

    def register(self, tokens: Sequence[int], blocks: Sequence[int], identity: int = BASE_IDENTITY) -> int:
        toks = np.ascontiguousarray(tokens, dtype=np.uint32)
        blk = np.ascontiguousarray(blocks, dtype=np.int32)
        return self.lib.poot_prefix_register(self.h, self.pool.h, identity, toks.ctypes.data, len(toks),
                                             blk.ctypes.data, len(blk))

    def reclaimable(self) -> int:
        """Cached blocks that no live sequence shares: what ``evict_unused`` can give back."""
        return self.lib.poot_prefix_count_unused(self.h, self.pool.h)

    def evict_unused(self, want: int = 0) -> int:
        return self.lib.poot_prefix_evict_unused(self.h, self.pool.h, want)

    def drop_identity(self, identity: int) -> int:
        return self.lib.poot_prefix_drop_identity(self.h, self.pool.h, identity)

    def force_collisions(self, on: bool) -> None:
        self.lib.poot_prefix_force_collisions(self.h, int(on))


def chain_hash(prev: int, block_tokens: Sequence[int]) -> int:
    b = np.ascontiguousarray(block_tokens, dtype=np.uint32)
    assert b.size == BLOCK
    return int(_lib().poot_chain_hash(prev, b.ctypes.data))


def chain_root() -> int:
    return int(_lib().poot_chain_root())


def blocks_for(tokens: int) -> int:
    return (tokens + BLOCK - 1) // BLOCK
