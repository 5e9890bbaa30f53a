"""A pool of numbered things (cache pages, state slots, request rows) with a last-in first-out free list.

LIFO on purpose: what a finished request gives back is what the next request gets, so that tests with few pages use
pages again at once.  Handing out an id twice or taking one back twice is an error, not a silent repair.
"""
from ..errors import CacheError


class Pool:
    def __init__(self, n, what="page"):
        self.n, self.what = int(n), what
        self.free_list = list(range(self.n - 1, -1, -1))        # pop() hands out 0 first
        self.held = [False] * self.n

    @property
    def n_free(self):
        return len(self.free_list)

    def take(self):
        if not self.free_list:
            raise CacheError(f"no free {self.what}")
        i = self.free_list.pop()
        if self.held[i]:
            raise CacheError(f"{self.what} {i} was on the free list while held")
        self.held[i] = True
        return i

    def give(self, i):
        if not 0 <= i < self.n or not self.held[i]:
            raise CacheError(f"{self.what} {i} given back but not held")
        self.held[i] = False
        self.free_list.append(i)

    def check(self):
        """Every id is either free once or held, never both, never neither."""
        if len(set(self.free_list)) != len(self.free_list):
            raise CacheError(f"a {self.what} is on the free list twice")
        for i in range(self.n):
            if self.held[i] == (i in set(self.free_list)):
                raise CacheError(f"{self.what} {i} is {'held and free' if self.held[i] else 'lost'}")
