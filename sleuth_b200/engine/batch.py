"""The description of one step's batch, on the host and on the device.

A step runs ``n`` sequences with ``counts[i]`` new tokens each (unequal), appended after the
``past[i]`` tokens the sequence already holds. On the device the kernels read flat int32 tables:

* ``token_ids[T]``, ``tok_seq[T]`` (index of the token's sequence in this batch), ``tok_pos[T]``
  (its absolute position), ``seq_start[n + 1]``, ``past[n]``, ``counts[n]``, ``slots[n]``
* ``rows[W]``: the token rows whose logits are wanted
* per cache group a block table ``[n, stride]``

All of it is packed into one pinned host buffer and sent with one copy. The host buffers form a
ring guarded by events, because a copy from pinned memory reads the buffer when it executes, not
when it is issued. The device buffer is a single one at a fixed address (copies and kernels are
ordered on the stream), which is what lets a captured decode step be replayed with new contents.
"""

from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np
import torch

_ALIGN = 64   # int32 elements (256 bytes) between regions


@dataclass
class StepBatch:
    n: int
    T: int
    stream: int
    token_ids: torch.Tensor
    tok_seq: torch.Tensor
    tok_pos: torch.Tensor
    seq_start: torch.Tensor
    past: torch.Tensor
    counts: torch.Tensor
    slots: torch.Tensor
    rows: torch.Tensor
    tables: list
    floats: torch.Tensor | None = None      # [n] float32 scratch for the sampler's uniform numbers
    ids_map: torch.Tensor | None = None     # decode steps: row t reads token_ids[ids_map[t]]
    host_counts: list = field(default_factory=list)
    host_past: list = field(default_factory=list)
    host_slots: list = field(default_factory=list)
    max_count: int = 1
    max_len: int = 0
    # the weight matrix that is read right after the part now running has finished (the next part's first product),
    # or None: the last kernel of a part may ask the L2 cache for it
    next_read: torch.Tensor | None = None


def _round(n: int) -> int:
    return (n + _ALIGN - 1) // _ALIGN * _ALIGN


class MetaStager:
    """Packs a step's tables, uploads them in one copy, and returns a ``StepBatch`` of device views."""

    RING = 4
    FEED = 1024      # int32 slots at the start of the buffer where decode steps find their tokens

    def __init__(self, device, n_groups: int, stride: int, capacity: int = 1 << 16):
        self.device = torch.device(device)
        self.n_groups, self.stride = n_groups, stride
        self.cap = 0
        self.dev = None
        self.hosts, self.events = [], []
        self.turn = 0
        self.generation = 0
        self.last_upload_bytes = 0
        self._grow(capacity)

    def _grow(self, capacity: int) -> None:
        """Replace the buffers by larger ones. The token feed at the start of the device buffer is carried over:
        in the pipelined loop the sampler has already left the next step's tokens there when an upload finds the
        buffer too small. Views of the old buffer that a caller still holds (``feed``) go stale; ``generation``
        tells (the stepper drops its recorded graphs on it, and ``Stepper.feed`` is looked up afresh each time)."""
        torch.cuda.synchronize(self.device)
        old = self.dev
        self.cap = capacity
        self.dev = torch.zeros(capacity, dtype=torch.int32, device=self.device)
        if old is not None:
            self.dev[:self.FEED].copy_(old[:self.FEED])
            torch.cuda.synchronize(self.device)
        self.hosts = [torch.zeros(capacity, dtype=torch.int32).pin_memory() for _ in range(self.RING)]
        self.events = [None] * self.RING
        self.generation += 1

    def layout(self, n: int, T: int, W: int, n_floats: int):
        """Offsets (in int32 elements) of every region for a batch of these sizes."""
        off, o = {}, self.FEED
        for name, size in (("token_ids", T), ("tok_seq", T), ("tok_pos", T), ("seq_start", n + 1), ("past", n),
                           ("counts", n), ("slots", n), ("rows", W), ("floats", n_floats), ("ids_map", n)):
            off[name] = (o, size)
            o += _round(max(size, 1))
        for g in range(self.n_groups):
            off[f"table{g}"] = (o, n * self.stride)
            o += _round(n * self.stride)
        return off, o

    @property
    def feed(self) -> torch.Tensor:
        """The device-side token feed: a decode step reads its tokens from here (through ``ids_map``), and the
        sampler may write the tokens it chooses straight into it for the next step."""
        return self.dev[:self.FEED]

    def upload(self, slots, pasts, counts, tokens: np.ndarray | None, rows: np.ndarray, tables: list[np.ndarray],
               floats: np.ndarray | None = None, stream: torch.cuda.Stream | None = None,
               feed_map: np.ndarray | None = None) -> StepBatch:
        """tokens: this step's token ids from the host. For a decode step (one token per sequence, at most FEED
        sequences) they go to the feed region; with ``tokens=None`` the feed is left as the sampler filled it and
        ``feed_map[i]`` says which feed slot holds sequence i's token."""
        n, W = len(slots), int(rows.shape[0])
        T = int(sum(counts))
        via_feed = feed_map is not None or (T == n and n <= self.FEED)
        if tokens is None and feed_map is None:
            raise ValueError("a step needs its tokens: from the host, or a map into the device-side feed")
        nf = 0 if floats is None else int(floats.shape[0])
        off, total = self.layout(n, T, W, nf)
        if total > self.cap:
            self._grow(max(total, 2 * self.cap))
        i = self.turn
        self.turn = (self.turn + 1) % self.RING
        if self.events[i] is not None:
            self.events[i].synchronize()
        host = self.hosts[i].numpy()

        counts_a = np.asarray(counts, dtype=np.int32)
        pasts_a = np.asarray(pasts, dtype=np.int32)
        starts = np.zeros(n + 1, dtype=np.int32)
        np.cumsum(counts_a, out=starts[1:])
        seq_of = np.repeat(np.arange(n, dtype=np.int32), counts_a)
        pos_of = np.arange(T, dtype=np.int32) - starts[seq_of] + pasts_a[seq_of]

        def put(name, arr):
            o, size = off[name]
            if size:
                host[o:o + size] = arr

        first = self.FEED                       # the copy starts here unless the host supplies feed contents
        if via_feed:
            if tokens is not None:
                host[:n] = tokens
                first = 0
            put("ids_map", np.arange(n, dtype=np.int32) if feed_map is None or tokens is not None else feed_map)
        else:
            put("token_ids", tokens)
        put("tok_seq", seq_of)
        put("tok_pos", pos_of)
        put("seq_start", starts)
        put("past", pasts_a)
        put("counts", counts_a)
        put("slots", np.asarray(slots, dtype=np.int32))
        put("rows", rows)
        if nf:
            o, size = off["floats"]
            host[o:o + size] = floats.astype(np.float32).view(np.int32)
        for g, t in enumerate(tables):
            o, size = off[f"table{g}"]
            host[o:o + size] = t.reshape(-1)

        st = stream if stream is not None else torch.cuda.current_stream(self.device)
        with torch.cuda.stream(st):
            self.dev[first:total].copy_(self.hosts[i][first:total], non_blocking=True)
            self.last_upload_bytes = 4 * (total - first)
            ev = torch.cuda.Event()
            ev.record(st)
        self.events[i] = ev

        def view(name):
            o, size = off[name]
            return self.dev[o:o + size]

        fl = view("floats").view(torch.float32) if nf else None
        return StepBatch(
            n=n, T=T, stream=st.cuda_stream, token_ids=self.feed if via_feed else view("token_ids"),
            ids_map=view("ids_map") if via_feed else None, tok_seq=view("tok_seq"),
            tok_pos=view("tok_pos"), seq_start=view("seq_start"), past=view("past"), counts=view("counts"),
            slots=view("slots"), rows=view("rows"),
            tables=[view(f"table{g}").view(n, self.stride) for g in range(self.n_groups)], floats=fl,
            host_counts=list(map(int, counts)), host_past=list(map(int, pasts)), host_slots=list(map(int, slots)),
            max_count=int(counts_a.max()) if n else 0, max_len=int((pasts_a + counts_a).max()) if n else 0)
