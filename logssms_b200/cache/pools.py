"""Host-side free lists for pages and state slots.

Plain LIFO free lists with full bookkeeping: an id is either free or held,
never both, never twice.  Every misuse (double free, freeing an id that was
never handed out, asking for more than there is) raises at once.  The
reference keeps its free lists as GPU tensors sliced from the front
(python/logssms/cache/naive/manager.py:53-58, 297-301); here they live on the
host because every decision that needs them is taken on the host.
"""
from __future__ import annotations


class OutOfPages(RuntimeError):
    """More pages (or slots) were asked for than are free."""


class FreeList:
    def __init__(self, count: int, what: str = "page"):
        if count < 0:
            raise ValueError(f"negative {what} count")
        self.count = count
        self.what = what
        self._free = list(range(count - 1, -1, -1))     # pop() hands out 0 first
        self._held = [False] * count

    @property
    def num_free(self) -> int:
        return len(self._free)

    @property
    def num_held(self) -> int:
        return self.count - len(self._free)

    def alloc(self, n: int = 1) -> list[int]:
        if n < 0:
            raise ValueError("negative allocation")
        if n > len(self._free):
            raise OutOfPages(f"asked for {n} {self.what}s, {len(self._free)} free of {self.count}")
        out = [self._free.pop() for _ in range(n)]
        for i in out:
            self._held[i] = True
        return out

    def free(self, ids) -> None:
        for i in ids:
            if not (0 <= i < self.count):
                raise ValueError(f"{self.what} {i} does not exist")
            if not self._held[i]:
                raise ValueError(f"{self.what} {i} freed twice (or never handed out)")
            self._held[i] = False
            self._free.append(i)

    def is_held(self, i: int) -> bool:
        return self._held[i]

    def check(self) -> None:
        """Free and held ids partition [0, count); no id is free twice."""
        if len(set(self._free)) != len(self._free):
            raise AssertionError(f"a {self.what} is on the free list twice")
        for i in self._free:
            if self._held[i]:
                raise AssertionError(f"{self.what} {i} is both free and held")
        if sum(self._held) + len(self._free) != self.count:
            raise AssertionError(f"a {self.what} is lost: {sum(self._held)} held + {len(self._free)} free != {self.count}")
