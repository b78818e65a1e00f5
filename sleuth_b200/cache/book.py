"""Host-side bookkeeping of the cache: sequence slots, pages, lengths and block tables.

Nothing here touches a GPU; the device storage (``cache/paged.py``) is addressed through the tables
kept here.

* A **slot** stands for one live sequence. It is taken when a batch starts and given back when the
  sequence ends; the next batch takes it again.
* Keys and values live in **pages** of 64 tokens. Each *group* of cache entries with the same needs
  (key/value heads, head size, window) has a page pool of its own and, per slot, a row of the
  group's **block table**: entry ``i`` of the row is the page that holds positions ``64*i .. 64*i+63``.
* A group with a **window** gives pages back as soon as every position on them has fallen out of the
  window of all future queries, so such a group holds about ``window`` tokens per sequence however
  long the sequence grows. Positions still map to table entries the same way.
* ``lengths[slot]`` is the number of tokens the sequence holds. Stale contents of a reused page are
  never read: every kernel reads positions below the length only (the reference relies on the same
  idea: entries past ``pos`` are simply overwritten, sleuth/forge/infer/kv_cache.py:52-64).

The reference's cache is one preallocated ``[batch, kv_heads, max_len, head_dim]`` pair per layer with
a single position shared by all rows (sleuth/forge/infer/kv_cache.py:25-70); slots, per-sequence
lengths, pages and groups are this library's own.
"""

from __future__ import annotations

import heapq

from dataclasses import dataclass

import numpy as np

PAGE_TOKENS = 64


class CacheFull(RuntimeError):
    """No free page or slot is left."""


class CacheMisuse(RuntimeError):
    """A slot or page was given back twice, or used while not held."""


def pages_for(tokens: int) -> int:
    return (tokens + PAGE_TOKENS - 1) // PAGE_TOKENS


class PagePool:
    """Free page numbers 0..n-1; the lowest are handed out first. Pages that were used before are so used again
    before untouched ones, and what is held stays together at the low end of the pool: a prompt whose pages lie
    scattered over a pool of many gigabytes was measured 5 % slower than one whose pages lie side by side."""

    def __init__(self, n_pages: int):
        self.n_pages = n_pages
        self._free = list(range(n_pages))          # a heap (ascending numbers are one)
        self._held = np.zeros(n_pages, dtype=bool)

    @property
    def free(self) -> int:
        return len(self._free)

    def take(self, k: int) -> list[int]:
        if k > len(self._free):
            raise CacheFull(f"the cache needs {k} more pages of {PAGE_TOKENS} tokens and {len(self._free)} of "
                            f"{self.n_pages} are free")
        out = [heapq.heappop(self._free) for _ in range(k)]
        self._held[out] = True
        return out

    def give(self, pages) -> None:
        for p in pages:
            if not self._held[p]:
                raise CacheMisuse(f"page {p} was given back while not held")
            self._held[p] = False
            heapq.heappush(self._free, p)


@dataclass
class GroupBook:
    window: int                 # 0 = keep every position
    pool: PagePool
    table: np.ndarray           # [max_slots, stride] int32, -1 = no page
    first_page: np.ndarray      # [max_slots] index of the first table entry still held


class CacheBook:
    """Slots, lengths and per-group block tables.

    windows: the window of each group (0 = none). n_pages: pages of each group's pool.
    stride: entries per block-table row = pages of the longest sequence allowed.
    """

    def __init__(self, windows: list[int], n_pages: int, max_slots: int, stride: int):
        self.max_slots = max_slots
        self.stride = stride
        self.max_len = stride * PAGE_TOKENS
        self.lengths = np.zeros(max_slots, dtype=np.int32)
        self._free_slots = list(range(max_slots - 1, -1, -1))
        self._live = np.zeros(max_slots, dtype=bool)
        self.groups = [GroupBook(w, PagePool(n_pages), np.full((max_slots, stride), -1, dtype=np.int32),
                                 np.zeros(max_slots, dtype=np.int64)) for w in windows]

    # ---- slots ----
    @property
    def free_slots(self) -> int:
        return len(self._free_slots)

    def live_slots(self) -> list[int]:
        return [int(i) for i in np.nonzero(self._live)[0]]

    def open(self, n: int) -> list[int]:
        if n > len(self._free_slots):
            raise CacheFull(f"{n} sequences were asked for and {len(self._free_slots)} of {self.max_slots} slots are free")
        slots = [self._free_slots.pop() for _ in range(n)]
        for s in slots:
            self._live[s] = True
            self.lengths[s] = 0
            for g in self.groups:
                g.first_page[s] = 0
        return slots

    def close(self, slots) -> None:
        for s in slots:
            self._check_live(s)
            for g in self.groups:
                row = g.table[s]
                held = row[row >= 0]
                g.pool.give(held.tolist())
                row[:] = -1
            self.lengths[s] = 0
            self._live[s] = False
            self._free_slots.append(s)

    def _check_live(self, s: int) -> None:
        if not (0 <= s < self.max_slots) or not self._live[s]:
            raise CacheMisuse(f"slot {s} is not held")

    # ---- growth ----
    def pages_needed(self, slots, new_lengths) -> list[int]:
        """Pages each group would have to take so that the sequences can grow to ``new_lengths``."""
        need = [0] * len(self.groups)
        for s, n in zip(slots, new_lengths):
            for gi, g in enumerate(self.groups):
                have = int((g.table[s] >= 0).sum())
                lo = int(g.first_page[s])
                need[gi] += max(0, pages_for(n) - lo - have)
        return need

    def peak_pages_needed(self, chunks) -> list[int]:
        """The most pages each group's pool must still give out at any moment while ``chunks`` run one after
        another, each a ``(slots, new_lengths)`` pair that is grown and then committed. A windowed group hands
        pages back as its sequences move on, so its peak can lie below what the final lengths alone suggest.
        Nothing is changed: the run is only played through on copies of the counts."""
        peaks = []
        for g in self.groups:
            first = {}
            have = {}
            out = peak = 0
            for slots, new_lengths in chunks:
                for s, n in zip(slots, new_lengths):
                    if s not in first:
                        first[s] = int(g.first_page[s])
                        have[s] = int((g.table[s] >= 0).sum())
                    take = max(0, pages_for(n) - first[s] - have[s])
                    have[s] += take
                    out += take
                peak = max(peak, out)
                if g.window:
                    for s, n in zip(slots, new_lengths):
                        keep_from = max(0, n - g.window + 1) // PAGE_TOKENS
                        if keep_from > first[s]:
                            back = min(have[s], keep_from - first[s])
                            have[s] -= back
                            out -= back
                            first[s] = keep_from
            peaks.append(peak)
        return peaks

    def grow(self, slots, new_lengths) -> None:
        """Take the pages for ``new_lengths`` (all or nothing) without changing the lengths yet."""
        for s, n in zip(slots, new_lengths):
            self._check_live(s)
            if n > self.max_len:
                raise CacheFull(f"a sequence of {n} tokens does not fit the longest allowed one ({self.max_len})")
            if n < self.lengths[s]:
                raise CacheMisuse(f"slot {s} holds {self.lengths[s]} tokens and cannot shrink to {n}")
        need = self.pages_needed(slots, new_lengths)
        for g, k in zip(self.groups, need):
            if k > g.pool.free:
                raise CacheFull(f"the cache needs {k} more pages of {PAGE_TOKENS} tokens and {g.pool.free} of "
                                f"{g.pool.n_pages} are free")
        for s, n in zip(slots, new_lengths):
            for g in self.groups:
                row = g.table[s]
                for i in range(int(g.first_page[s]), pages_for(n)):
                    if row[i] < 0:
                        row[i] = g.pool.take(1)[0]

    def commit(self, slots, new_lengths) -> None:
        """The step has been issued: set the lengths and let windowed groups give pages back."""
        for s, n in zip(slots, new_lengths):
            self.lengths[s] = n
            for g in self.groups:
                if g.window:
                    # the next query sits at position >= n and sees keys >= n - window + 1
                    keep_from = max(0, n - g.window + 1) // PAGE_TOKENS
                    lo = int(g.first_page[s])
                    if keep_from > lo:
                        row = g.table[s]
                        g.pool.give(row[lo:keep_from].tolist())
                        row[lo:keep_from] = -1
                        g.first_page[s] = keep_from

    def tables_for(self, slots, pages: int | None = None) -> list[np.ndarray]:
        """Per group the block-table rows of ``slots`` [n, stride] (or their first ``pages`` entries)."""
        idx = np.asarray(slots, dtype=np.int64)
        return [g.table[idx] if pages is None else g.table[idx, :pages] for g in self.groups]

    def pages_in_use(self) -> list[int]:
        return [g.pool.n_pages - g.pool.free for g in self.groups]
