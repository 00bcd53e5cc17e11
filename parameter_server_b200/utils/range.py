"""Half-open integer ranges over the uint64 key space.

Same surface as the reference's ``Range<T>`` (src/base/range.h:11-104): set
operations, ``contains``, ``even_divide`` and ``Range.all() = [0, 2**64-1)``.
``even_divide`` uses exact integer arithmetic instead of ``long double`` so that
shard boundaries are reproducible on every platform.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List

U64_MAX = (1 << 64) - 1


@dataclass(frozen=True)
class Range:
    begin: int = 0
    end: int = 0

    @staticmethod
    def all() -> "Range":
        return Range(0, U64_MAX)

    def size(self) -> int:
        return self.end - self.begin

    def valid(self) -> bool:
        return self.end >= self.begin

    def empty(self) -> bool:
        return self.begin >= self.end

    def contains(self, v: int) -> bool:
        return self.begin <= v < self.end

    def intersection(self, o: "Range") -> "Range":
        return Range(max(self.begin, o.begin), min(self.end, o.end))

    def union(self, o: "Range") -> "Range":
        return Range(min(self.begin, o.begin), max(self.end, o.end))

    def even_divide(self, n: int, i: int) -> "Range":
        if not self.valid() or n <= 0 or not (0 <= i < n):
            raise ValueError(f"even_divide({n}, {i}) on {self}")
        size = self.end - self.begin
        b = self.begin + size * i // n
        e = self.end if i + 1 == n else self.begin + size * (i + 1) // n
        return Range(b, e)

    def separators(self, n: int) -> List[int]:
        """n+1 boundaries of the n even parts."""
        return [self.even_divide(n, i).begin for i in range(n)] + [self.end]

    def __add__(self, v: int) -> "Range":
        return Range(self.begin + v, self.end + v)

    def __sub__(self, v: int) -> "Range":
        return Range(self.begin - v, self.end - v)

    def __str__(self) -> str:
        return f"[{self.begin},{self.end})"
