"""Free-list allocators for pages and for state slots.

Parity: src/llmserve/kvcache/paged.py:34-62 — a FIFO of integer ids; ``allocate`` takes from
the head, ``free`` validates (an id that is not held raises) and appends to the tail, so the
order in which ids are used again is deterministic.
"""

from __future__ import annotations

from collections import deque


class OutOfPages(RuntimeError):
    """The pool cannot give what a step asked for; nothing was changed."""


class IdAllocator:
    def __init__(self, count: int, what: str = "page"):
        if count < 0:
            raise ValueError(f"cannot make an allocator of {count} {what}s")
        self.count = int(count)
        self.what = what
        self._free: deque[int] = deque(range(self.count))
        self._used: set[int] = set()

    @property
    def num_free(self) -> int:
        return len(self._free)

    @property
    def num_used(self) -> int:
        return len(self._used)

    def allocate(self) -> int:
        if not self._free:
            raise OutOfPages(f"no free {self.what}")
        i = self._free.popleft()
        self._used.add(i)
        return i

    def free(self, ids) -> None:
        ids = list(ids)
        for i in ids:
            if i not in self._used:
                raise ValueError(f"double free or invalid {self.what} id {i}")
        if len(set(ids)) != len(ids):
            raise ValueError(f"a {self.what} id is freed twice in one call: {ids}")
        for i in ids:
            self._used.remove(i)
            self._free.append(i)

    def check(self) -> None:
        """No id lost, held twice, or both free and held."""
        free = list(self._free)
        assert len(set(free)) == len(free), f"a {self.what} is twice in the free list"
        assert not (set(free) & self._used), f"a {self.what} is both free and held"
        assert len(free) + len(self._used) == self.count, f"a {self.what} was lost"
