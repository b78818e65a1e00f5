"""Device storage of the cache, laid out from what the model's parts ask for.

Each layer application has one cache *entry*. A part asks for what its entry needs through a request:

* ``KVRequest(kv_heads, head_dim, window)``: keys and values of every position (or of the last
  ``window`` positions). Entries with equal requests form a *group*; a group owns one tensor
  ``[entries, 2, pages, kv_heads, 64, head_dim]`` (index 1: 0 = keys, 1 = values), so a page number
  means the same place in every entry of the group and one block table serves them all.
* ``StateRequest(shape, dtype)``: a fixed-size state per sequence, ``[max_sequences, *shape]``, zeroed
  when a slot is taken. It is sized by the number of sequences that may be live at once, not by the
  number of pages: a state of a megabyte per sequence beside a cache of thousands of pages stays small. The Qwen3 decoder has none; a recurrent or convolutional mixer would keep
  its state here (the reference keeps such state beside the keys and values of the same batch row,
  sleuth/formats/qwen35.py:132-145, and a per-row token history, sleuth/forge/infer/kv_cache.py:37-43).
* ``None``: the entry holds nothing.

The head-major page layout lets a decode block stream one (sequence, kv head) as contiguous
``64 * head_dim`` runs. The cache dtype is the run dtype: bfloat16 on the fast path, as the reference's
cache on CUDA (sleuth/forge/infer/generate.py:94-95), float32 on the 32-bit path.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from .book import PAGE_TOKENS, CacheBook, pages_for


@dataclass(frozen=True)
class KVRequest:
    kv_heads: int
    head_dim: int
    window: int = 0


@dataclass(frozen=True)
class StateRequest:
    shape: tuple
    dtype: torch.dtype = torch.float32


@dataclass
class KVView:
    """What an attention part gets for its entry in one step."""
    k_pool: torch.Tensor        # [pages, kv_heads, 64, head_dim]
    v_pool: torch.Tensor
    group: int                  # which block table of the step's batch applies
    window: int
    writes: bool                # this application owns the entry and stores its keys and values


@dataclass
class StateView:
    state: torch.Tensor         # [max_slots, *shape]; index with the batch's slots


class PagedCache:
    """Pools and state regions for a list of requests (one per cache entry), plus the bookkeeping."""

    # Sequences live at once when the caller names no number and some entry keeps per-sequence state.
    DEFAULT_SEQUENCES_WITH_STATE = 256

    def __init__(self, requests: list, max_tokens: int, max_seq_len: int, dtype: torch.dtype, device,
                 max_sequences: int | None = None):
        """max_tokens: tokens all live sequences may hold together (pages of 64). max_sequences: how many
        sequences may be live at once (slots). Default: one per page, the most that can ever hold a token, unless
        some entry keeps a per-sequence state, which is allocated for every slot: then 256 at most."""
        self.dtype = dtype
        self.device = torch.device(device)
        self.n_pages = max(1, pages_for(max_tokens))
        self.stride = max(1, pages_for(max_seq_len))
        self.requests = list(requests)
        if max_sequences is None:
            has_state = any(isinstance(r, StateRequest) for r in self.requests)
            max_sequences = min(self.n_pages, self.DEFAULT_SEQUENCES_WITH_STATE) if has_state else self.n_pages
        if max_sequences < 1:
            raise ValueError(f"max_sequences must be at least 1, got {max_sequences}")
        self.max_slots = int(max_sequences)

        keys: list[KVRequest] = []
        self.entry_group: list[int | None] = []
        self.entry_index: list[int | None] = []
        members: list[list[int]] = []
        for e, r in enumerate(self.requests):
            if isinstance(r, KVRequest):
                if r not in keys:
                    keys.append(r)
                    members.append([])
                g = keys.index(r)
                self.entry_group.append(g)
                self.entry_index.append(len(members[g]))
                members[g].append(e)
            elif isinstance(r, StateRequest) or r is None:
                self.entry_group.append(None)
                self.entry_index.append(None)
            else:
                raise TypeError(f"cache entry {e}: unknown request {r!r}")
        self.group_requests = keys
        self.book = CacheBook([k.window for k in keys], self.n_pages, self.max_slots, self.stride)
        self.pools = [torch.zeros((len(m), 2, self.n_pages, k.kv_heads, PAGE_TOKENS, k.head_dim), dtype=dtype,
                                  device=self.device) for k, m in zip(keys, members)]
        self.states = {e: torch.zeros((self.max_slots, *r.shape), dtype=r.dtype, device=self.device)
                       for e, r in enumerate(self.requests) if isinstance(r, StateRequest)}

    @property
    def n_groups(self) -> int:
        return len(self.group_requests)

    def view(self, entry: int, writes: bool):
        r = self.requests[entry]
        if isinstance(r, KVRequest):
            g, i = self.entry_group[entry], self.entry_index[entry]
            return KVView(self.pools[g][i, 0], self.pools[g][i, 1], g, r.window, writes)
        if isinstance(r, StateRequest):
            return StateView(self.states[entry])
        return None

    def open(self, n: int) -> list[int]:
        slots = self.book.open(n)
        if self.states:
            idx = torch.tensor(slots, dtype=torch.long, device=self.device)
            for s in self.states.values():
                s.index_fill_(0, idx, 0)
        return slots

    def close(self, slots) -> None:
        self.book.close(slots)

    def nbytes(self) -> int:
        return (sum(p.numel() * p.element_size() for p in self.pools) +
                sum(s.numel() * s.element_size() for s in self.states.values()))
