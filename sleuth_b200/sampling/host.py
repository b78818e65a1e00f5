"""The host side of sampling: random numbers, the recent-token window and the n-gram ban list.

None of this touches a GPU. The uniform number of a draw is a pure function of (seed, request,
step), so the token a request gets does not depend on which other requests share its batch or on
the order in which batches run. (The reference draws from one ``torch.Generator`` per call,
sleuth/forge/infer/generate.py:71-75; batches are this library's own, hence the keyed generator.)
"""

from __future__ import annotations

import os

import numpy as np

_M64 = (1 << 64) - 1
_K1, _K2, _K3 = 0x9E3779B97F4A7C15, 0xBF58476D1CE4E5B9, 0x94D049BB133111EB
_BELOW_ONE = float(np.nextafter(np.float32(1.0), np.float32(0.0)))


def fresh_seed() -> int:
    return int.from_bytes(os.urandom(8), "little")


def uniform(seed: int, request: int, step: int) -> float:
    """A number in [0, 1) determined by its three arguments (splitmix64 of their mix)."""
    x = ((seed & _M64) * _K1 + ((request + 1) & _M64) * _K2 + ((step + 1) & _M64) * _K3) & _M64
    for _ in range(2):
        x = (x + _K1) & _M64
        x ^= x >> 30
        x = (x * _K2) & _M64
        x ^= x >> 27
        x = (x * _K3) & _M64
        x ^= x >> 31
    return min((x >> 11) * 2.0 ** -53, _BELOW_ONE)


def uniforms(seed: int, requests, step_of) -> np.ndarray:
    return np.asarray([uniform(seed, r, s) for r, s in zip(requests, step_of)], dtype=np.float32).clip(0.0, _BELOW_ONE)


class _Node:
    """A node of the phrase trie: children by token, and the tokens seen right after this phrase when it is n-1 long."""
    __slots__ = ("next", "after")

    def __init__(self):
        self.next: dict[int, "_Node"] = {}
        self.after: set[int] = set()


class NgramBlocker:
    """Bans the tokens that would complete an n-gram the sequence already holds (the prompt counts).

    The phrases of n-1 tokens seen so far form a trie; a node at depth n-1 keeps the tokens that have
    followed its phrase. ``_open`` holds, for each length 0..n-2, the node reached by the most recent
    tokens of that length, so a new token extends every open phrase by one step and the node that the
    last n-1 tokens reach is always at hand: one token costs n-1 dictionary steps, a query none.
    The rule itself is the reference's (sleuth/forge/infer/sampling.py:36-64): with n = 1 every token
    seen is banned, with n <= 0 nothing is."""

    def __init__(self, n: int, ids=()):
        self.n = int(n)
        self._root = _Node()
        self._open: list[_Node] = [self._root]      # _open[k]: the node of the last k tokens (k < n - 1)
        self._last: _Node | None = self._root if self.n == 1 else None   # the node of the last n-1 tokens
        for t in ids:
            self.add(t)

    def add(self, token: int) -> None:
        if self.n <= 0:
            return
        token = int(token)
        if self._last is not None:
            self._last.after.add(token)              # the last n-1 tokens were followed by this one
        if self.n == 1:
            return
        grown = [self._root]
        for node in self._open:                      # every open phrase takes the token
            child = node.next.get(token)
            if child is None:
                child = node.next[token] = _Node()
            grown.append(child)
        full = grown[self.n - 1] if len(grown) >= self.n else None
        self._open = grown[:self.n - 1]
        self._last = full

    def banned(self) -> list[int]:
        return sorted(self._last.after) if self.n > 0 and self._last is not None else []


def recent_window(context: list[int], repeat_last_n: int) -> list[int]:
    """The distinct tokens among the last ``repeat_last_n`` of the context (all of it for 0)
    (sleuth/forge/infer/sampling.py:121-123)."""
    tail = context[-repeat_last_n:] if repeat_last_n > 0 else context
    return sorted(set(tail))
