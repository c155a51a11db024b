"""Constants of the hashed n-gram embedding of a per-layer embedding block, derived from the checkpoint header the way
the model derives them at construction (crates/poot-models/src/components/ple.rs ``derived_tables``): every hash head
reduces its 64-bit mix by a prime of its own - consecutive primes from ``vocab_base`` up, the block with ordinal ``o``
skipping the primes of blocks ``0..o`` - and owns that many consecutive rows of the block's table, whose row count is
padded to a multiple; the multipliers of the n-gram positions are odd words drawn from SplitMix64."""
from __future__ import annotations

from dataclasses import dataclass
from typing import List

MASK64 = (1 << 64) - 1
SPLITMIX_GAMMA, SPLITMIX_M1, SPLITMIX_M2 = 0x9E3779B97F4A7C15, 0xBF58476D1CE4E5B9, 0x94D049BB133111EB
ORDINAL_STRIDE = 10007


def splitmix64(v: int) -> int:
    z = (v + SPLITMIX_GAMMA) & MASK64
    z = ((z ^ (z >> 30)) * SPLITMIX_M1) & MASK64
    z = ((z ^ (z >> 27)) * SPLITMIX_M2) & MASK64
    return z ^ (z >> 31)


def is_prime(n: int) -> bool:
    if n < 2:
        return False
    if n < 4:
        return True
    if n % 2 == 0:
        return False
    d = 3
    while d * d <= n:
        if n % d == 0:
            return False
        d += 2
    return True


@dataclass(frozen=True)
class NgramTables:
    primes: tuple          # per hash head: the modulus of its id
    offsets: tuple         # per hash head: the first table row of its slice
    rows: int              # table rows (the slices' total, padded)
    multipliers: tuple     # one odd 64-bit word per n-gram position


def ngram_tables(ordinal: int, ngram_size: int, heads_per_order: int, vocab_base: int, divisible_by: int, seed: int,
                 vocab: int) -> NgramTables:
    if ngram_size not in (2, 3):
        raise ValueError(f"n-gram order {ngram_size} outside 2..3")
    if vocab_base < 2 or divisible_by < 1 or heads_per_order < 1 or vocab < 1:
        raise ValueError("n-gram hash: vocab_base >= 2, a positive padding multiple, head count and vocabulary")
    heads = (ngram_size - 1) * heads_per_order
    primes: List[int] = []
    n, skip = vocab_base - 1, ordinal * heads
    while len(primes) < heads:
        n += 1
        if is_prime(n):
            if skip:
                skip -= 1
            else:
                primes.append(n)
    if primes[-1] >= 1 << 32:
        raise ValueError("n-gram hash: a head's modulus exceeds 32 bits")
    offsets, total = [], 0
    for p in primes:
        offsets.append(total)
        total += p
    rows = -(-total // divisible_by) * divisible_by
    if rows > 0x7FFFFFFF:
        raise ValueError("n-gram hash: the table has more rows than a 32-bit index reaches")
    half = max(((1 << 63) - 1) // vocab // 2, 1)
    base = (seed + ORDINAL_STRIDE * ordinal) & MASK64
    mult = tuple(2 * (splitmix64((base + SPLITMIX_GAMMA * (i + 1)) & MASK64) % half) + 1 for i in range(ngram_size))
    return NgramTables(tuple(primes), tuple(offsets), rows, mult)
