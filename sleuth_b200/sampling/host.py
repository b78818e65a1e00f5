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


class NgramBlocker:
    """Remembers, for every (n-1)-token phrase seen, the tokens that followed it, so that the token
    completing a seen n-gram can be banned. Incremental: each token costs one dictionary update.
    The prompt counts. (Behaviour of sleuth/forge/infer/sampling.py:36-64.)"""

    def __init__(self, n: int, ids=()):
        self.n = n
        self.ids: list[int] = []
        self.followers: dict[tuple, set] = {}
        for t in ids:
            self.add(t)

    def add(self, token: int) -> None:
        self.ids.append(int(token))
        if self.n > 0 and len(self.ids) >= self.n:
            key = tuple(self.ids[len(self.ids) - self.n:-1])
            self.followers.setdefault(key, set()).add(int(token))

    def banned(self) -> list[int]:
        if self.n <= 0 or len(self.ids) < self.n - 1:
            return []
        key = tuple(self.ids[len(self.ids) - (self.n - 1):]) if self.n > 1 else ()
        return sorted(self.followers.get(key, ()))


def recent_window(context: list[int], repeat_last_n: int) -> list[int]:
    """The distinct tokens among the last ``repeat_last_n`` of the context (all of it for 0)
    (sleuth/forge/infer/sampling.py:121-123)."""
    tail = context[-repeat_last_n:] if repeat_last_n > 0 else context
    return sorted(set(tail))
