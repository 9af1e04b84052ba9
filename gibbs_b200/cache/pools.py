"""Free lists of page ids and slot ids.  They hold no memory themselves; the
cache manager owns the tensors the ids index.  (MisterTK/gibbs keeps block ids
the same way, ``src/kv/mod.rs:332-430``, but there the ids are bookkeeping
only.)  Every misuse is an error: an id is never handed out twice, and giving
back an id that is not out raises."""
from __future__ import annotations


class PoolError(RuntimeError):
    pass


class IdPool:
    def __init__(self, size: int, what: str = "id"):
        if size < 0:
            raise ValueError(f"a pool of {size} {what}s")
        self.size, self.what = size, what
        self._free = list(range(size - 1, -1, -1))     # pop() hands out low ids first
        self._out = [False] * size

    @property
    def n_free(self) -> int:
        return len(self._free)

    @property
    def n_used(self) -> int:
        return self.size - len(self._free)

    def take(self):
        """An id that is not in use, or None when the pool is empty.  The id
        given back most recently is handed out first, so ids are reused soon."""
        if not self._free:
            return None
        i = self._free.pop()
        self._out[i] = True
        return i

    def take_many(self, n: int):
        """n ids, or None (and nothing taken) when fewer are free."""
        if n > len(self._free):
            return None
        return [self.take() for _ in range(n)]

    def give_back(self, i: int) -> None:
        if not 0 <= i < self.size:
            raise PoolError(f"{self.what} {i} is outside the pool of {self.size}")
        if not self._out[i]:
            raise PoolError(f"{self.what} {i} was given back twice (or never taken)")
        self._out[i] = False
        self._free.append(i)

    def check(self) -> None:
        """Invariant: every id is either free or out, never both, never neither."""
        free = set(self._free)
        if len(free) != len(self._free):
            raise PoolError(f"a {self.what} is on the free list twice")
        for i in range(self.size):
            if self._out[i] == (i in free):
                raise PoolError(f"{self.what} {i} is {'both free and out' if self._out[i] else 'lost'}")
