"""Regions of a communication block with guard words between them.

Peers store into this rank's block through mapped pointers, so an index error in a remote kernel shows up here as
memory some other region owns.  No sanitizer sees that.  The layout therefore puts a guard - ``GUARD_WORDS`` int32 of a
pattern that depends on the region and the rank - after every region (regions start 1 KiB aligned, the guard sits in
the padding right behind the region's last byte, so even a one-element overrun hits it), writes the guards when the
block is set up, and ``check`` reads them back on the host: at drain, after a step that reported a failure, and on
demand in debug runs.  A damaged guard names the region whose end was overrun.  (The reference relies on declared slot
ranges checked at bind and validation layers, website/docs/architecture/graph-ir.mdx "slot ranges"; this is the
counterpart for peer-written buffers.)
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Dict, List, Sequence, Tuple

ALIGN = 1024
GUARD_WORDS = 16
GUARD_BYTES = GUARD_WORDS * 4
_SEED = 0x5AFEC0DE


class CommBufferOverrun(RuntimeError):
    def __init__(self, region: str, rank: int, word: int, found: int, expected: int):
        super().__init__(f"rank {rank}: guard behind region '{region}' was overwritten (word {word}: found "
                         f"{found & 0xFFFFFFFF:#010x}, expected {expected & 0xFFFFFFFF:#010x}): a store ran past the region's end")
        self.region, self.rank, self.word = region, rank, word


@dataclass(frozen=True)
class Region:
    name: str
    offset: int
    nbytes: int

    @property
    def guard_offset(self) -> int:
        return self.offset + (self.nbytes + 3) // 4 * 4


class GuardedLayout:
    """``GuardedLayout([("flags", 128), ("inbox", n), ...])``: offsets in declaration order, total size."""

    def __init__(self, regions: Sequence[Tuple[str, int]]):
        self.regions: Dict[str, Region] = {}
        off = 0
        for name, nbytes in regions:
            if nbytes <= 0 or name in self.regions:
                raise ValueError(f"region {name!r}: needs a unique name and a positive size")
            self.regions[name] = Region(name, off, nbytes)
            end = self.regions[name].guard_offset + GUARD_BYTES
            off = (end + ALIGN - 1) // ALIGN * ALIGN
        self.total = off

    def offset(self, name: str) -> int:
        return self.regions[name].offset

    def pattern(self, index: int, rank: int) -> List[int]:
        return [((_SEED ^ (index * 0x9E3779B1) ^ (rank * 0x85EBCA6B) ^ (w * 0x01000193)) & 0x7FFFFFFF)
                for w in range(GUARD_WORDS)]

    def write(self, rank: int, store: Callable[[int, List[int]], None]) -> None:
        """``store(byte_offset, int32 words)`` writes into this rank's own block."""
        for i, r in enumerate(self.regions.values()):
            store(r.guard_offset, self.pattern(i, rank))

    def check(self, rank: int, load: Callable[[int, int], Sequence[int]]) -> None:
        """``load(byte_offset, n_words)`` reads this rank's own block; raises for the first damaged guard."""
        for i, r in enumerate(self.regions.values()):
            want = self.pattern(i, rank)
            got = [int(v) for v in load(r.guard_offset, GUARD_WORDS)]
            for w, (g, e) in enumerate(zip(got, want)):
                if g != e:
                    raise CommBufferOverrun(r.name, rank, w, g, e)
