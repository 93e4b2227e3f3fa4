"""Free list of one pool of pages, and free list of state slots."""

from __future__ import annotations


class PagePool:
    """Pages 0..n-1 handed out last-in-first-out, page 0 first (oxr_runtime/kv_cache.py:31,43-52): a page given
    back is the next one handed out, so reuse happens at once. ``allocate`` is all-or-nothing."""

    def __init__(self, num_pages: int):
        if num_pages < 0:
            raise ValueError("num_pages must not be negative")
        self.num_pages = num_pages
        self._free = list(range(num_pages - 1, -1, -1))
        self._held = [False] * num_pages

    @property
    def free(self) -> int:
        return len(self._free)

    def allocate(self, count: int) -> list[int] | None:
        if count < 0:
            raise ValueError("count must not be negative")
        if count > len(self._free):
            return None
        out = [self._free.pop() for _ in range(count)]
        for p in out:
            self._held[p] = True
        return out

    def release(self, pages: list[int]) -> None:
        for p in pages:
            if not 0 <= p < self.num_pages:
                raise ValueError(f"page {p} is not of this pool")
            if not self._held[p]:
                raise ValueError(f"page {p} is released twice")
            self._held[p] = False
        self._free.extend(reversed(pages))

    def held(self) -> list[int]:
        return [p for p, h in enumerate(self._held) if h]
