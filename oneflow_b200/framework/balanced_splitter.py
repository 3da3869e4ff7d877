"""Uneven split rule shared by every S(axis) shard computation: the first ``n % k`` parts get one extra
element (reference: oneflow/core/common/balanced_splitter.cpp:19-43). The C++ twin lives in
csrc/core/sbp_math.cpp and is used when the core library is built."""
from __future__ import annotations


class BalancedSplitter:
    def __init__(self, total: int, parts: int):
        if parts <= 0:
            raise ValueError("parts must be positive")
        self.total, self.parts = int(total), int(parts)
        self.base, self.rem = divmod(self.total, self.parts)

    def size(self, idx: int) -> int:
        return self.base + (1 if idx < self.rem else 0)

    def at(self, idx: int):
        """[begin, end) of part idx."""
        if not 0 <= idx < self.parts:
            raise IndexError(idx)
        begin = idx * self.base + min(idx, self.rem)
        return begin, begin + self.size(idx)

    def at_range(self, first: int, last: int):
        """[begin, end) covering parts first..last inclusive."""
        return self.at(first)[0], self.at(last)[1]

    def owner(self, element: int) -> int:
        big = self.rem * (self.base + 1)
        if element < big:
            return element // (self.base + 1)
        return self.rem + (element - big) // max(self.base, 1)
