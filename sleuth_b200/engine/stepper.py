"""The step function: run the tokens a batch brings, from the cache, and return the wanted logits.

A step takes sequences that start together (their prompts, of unequal lengths) or go on together
(one token each); in fact each sequence may bring any number of tokens, and they are appended after
what its slot already holds. Only the given tokens are computed. Every sequence's keys and values go
to its own pages and every query reads its own sequence's pages, so no padding exists and nothing a
sequence computes depends on the others in the batch.

The reference's counterpart is ``Transformer.forward(idx, cache)`` with one shared position for a
rectangular batch and logits for every position (sleuth/forge/model/transformer.py:257-313,
sleuth/forge/infer/kv_cache.py:34,62-64); ragged batches, per-sequence positions and logits at chosen
rows only are this library's own.

Long steps are cut into chunks of at most ``max_step_tokens`` tokens; a chunk runs through all
layers before the next begins, so later chunks of a sequence find the earlier ones in the cache.
A step in which every sequence brings one token is replayed as a CUDA graph from its second
occurrence at a batch size on (the reference captures one decode step per length bucket,
sleuth/forge/infer/cuda_graph.py:96-129; here lengths live in device tables, so one graph per batch
size serves every length).
"""

from __future__ import annotations

from dataclasses import dataclass

import os

import numpy as np
import torch

from ..cache.book import CacheFull
from ..kernels import ops
from ..parts.base import Workspace
from .batch import MetaStager


@dataclass
class StepEntry:
    slot: int
    tokens: object              # sequence of token ids
    want: object = ()           # positions among ``tokens`` whose logits are wanted


class Stepper:
    def __init__(self, model, cache, device, max_len: int | None = None, max_step_tokens: int = 8192,
                 use_graphs: bool = True, max_graph_batch: int = 256):
        self.model, self.cache = model, cache
        self.max_len = cache.book.max_len if max_len is None else min(int(max_len), cache.book.max_len)
        self.device = torch.device(device)
        self.max_step_tokens = max_step_tokens
        self.use_graphs = use_graphs
        self.max_graph_batch = max_graph_batch
        self.ws = Workspace(self.device)
        self.meta = MetaStager(self.device, cache.n_groups, cache.stride)
        self._graphs: dict = {}
        self._seen_decode: set = set()
        self._seen_chunk: set = set()
        self._chunk_logits: torch.Tensor | None = None
        self.max_graph_rows = 64        # steps of many tokens are recorded only if they want at most this many rows of logits
        self.max_chunk_graphs = 16      # recordings of such steps kept at a time
        self._decode_logits: torch.Tensor | None = None
        self._graph_key = None
        self.check_kernels = os.environ.get("SLEUTH_B200_CHECK", "0") == "1"   # read the kernels' status word after each step
        self._status_host: torch.Tensor | None = None     # pinned copy of the kernels' status word, read one step late
        self._status_event = None
        self._graph_own: dict = {}          # own kernel launches captured in each graph
        self.graph_kernel_launches = 0      # own kernel launches replayed through graphs so far
        ops.lib()   # build or load the kernels now; fail here, loudly, if that is impossible

    # ------------------------------------------------------------------ public ----
    def step(self, entries: list[StepEntry], floats: np.ndarray | None = None) -> torch.Tensor:
        """Run one step. Returns float32 logits ``[sum(len(e.want)), vocab]`` in the order of the
        entries and of their ``want``. After a step of single tokens the result may be a view of a
        buffer that the next step overwrites."""
        if not entries:
            return torch.empty((0, self.model.vocab), dtype=torch.float32, device=self.device)
        self._raise_late_status()
        toks = [np.asarray(e.tokens, dtype=np.int64).reshape(-1) for e in entries]
        book = self.cache.book
        for e, t in zip(entries, toks):
            if t.size == 0:
                raise ValueError(f"slot {e.slot}: a step must bring at least one token for every sequence")
            if t.min() < 0 or t.max() >= self.model.vocab:
                raise ValueError(f"slot {e.slot}: token ids must lie in [0, {self.model.vocab})")
            for w in e.want:
                if not 0 <= int(w) < t.size:
                    raise ValueError(f"slot {e.slot}: wanted position {w} is outside its {t.size} tokens")
        slots = [int(e.slot) for e in entries]
        if len(set(slots)) != len(slots):
            raise ValueError("a step names a slot twice")
        finals = [int(book.lengths[s]) + int(t.size) for s, t in zip(slots, toks)]
        for s, n in zip(slots, finals):
            if n > self.max_len:
                raise CacheFull(f"slot {s} would hold {n} tokens; the longest sequence allowed is {self.max_len}")

        if all(t.size == 1 for t in toks):
            return self._decode(entries, slots, toks, floats)

        chunks = self._cut(toks)
        # All or nothing: a step that the cache cannot hold to its end is refused before its first chunk runs, so a
        # sequence is never left half-appended.
        lens = {s: int(book.lengths[s]) for s in slots}
        plan = []
        for chunk in chunks:
            c_slots = [slots[i] for i, _, _ in chunk]
            for (i, _, take), s in zip(chunk, c_slots):
                lens[s] += take
            plan.append((c_slots, [lens[s] for s in c_slots]))
        for g, need in zip(book.groups, book.peak_pages_needed(plan)):
            if need > g.pool.free:
                raise CacheFull(f"the step needs {need} more pages of 64 tokens and {g.pool.free} of {g.pool.n_pages} "
                                f"are free; nothing of it was run")

        n_want = sum(len(e.want) for e in entries)
        out = torch.empty((n_want, self.model.vocab), dtype=torch.float32, device=self.device)
        out_base, acc = [], 0
        for e in entries:
            out_base.append(acc)
            acc += len(e.want)
        for chunk in chunks:
            self._run_chunk(entries, slots, toks, chunk, out, out_base)
        if self.check_kernels:
            ops.gemm_tc_check(self.device)
        else:
            self._status_later()
        return out

    def _cut(self, toks) -> list:
        """The chunks of a step: lists of (entry index, first token, tokens) with at most ``max_step_tokens`` tokens
        each, entries in order, an entry that does not fit going on in the next chunk."""
        chunks, done = [], [0] * len(toks)
        while True:
            chunk, room = [], self.max_step_tokens
            for i, t in enumerate(toks):
                left = t.size - done[i]
                if left and room:
                    take = min(left, room)
                    chunk.append((i, done[i], take))
                    room -= take
            if not chunk:
                return chunks
            chunks.append(chunk)
            for i, start, take in chunk:
                done[i] = start + take

    # ------------------------------------------------------------ the kernels' status word ----
    def _status_later(self) -> None:
        """After a step of many tokens (the tcgen05 kernels serve those): start a copy of the kernels' status word
        to pinned memory. It is looked at when the next step begins, without waiting for the device, and at
        ``check_status``; a bounded wait that gave up inside a kernel is then reported one step late instead of never."""
        status = ops.tc_status(self.device)
        if status is None:
            return
        if self._status_host is None:
            self._status_host = torch.zeros(1, dtype=torch.int32).pin_memory()
        elif self._status_event is not None and not self._status_event.query():
            return                      # the earlier copy has not landed yet; it will tell the same story
        self._status_host.copy_(status, non_blocking=True)
        self._status_event = torch.cuda.Event()
        self._status_event.record()

    def _raise_late_status(self, wait: bool = False) -> None:
        ev = self._status_event
        if ev is None or not (wait or ev.query()):
            return
        ev.synchronize()
        self._status_event = None
        if int(self._status_host[0]):
            ops.gemm_tc_check(self.device)          # reads the word itself, clears it and raises

    def check_status(self) -> None:
        """Raise if a kernel's bounded wait gave up in any step so far (waits for the device)."""
        self._raise_late_status(wait=True)
        ops.gemm_tc_check(self.device)

    # ------------------------------------------------------------------ chunks ----
    def _run_chunk(self, entries, slots, toks, chunk, out, out_base) -> None:
        book = self.cache.book
        c_slots = [slots[i] for i, _, _ in chunk]
        c_past = [int(book.lengths[s]) for s in c_slots]
        c_counts = [take for _, _, take in chunk]
        new_lens = [p + c for p, c in zip(c_past, c_counts)]
        book.grow(c_slots, new_lens)
        tokens = np.concatenate([toks[i][start:start + take] for i, start, take in chunk]).astype(np.int32)
        rows, dest = [], []
        base = 0
        for i, start, take in chunk:
            for j, w in enumerate(entries[i].want):
                w = int(w)
                if start <= w < start + take:
                    rows.append(base + w - start)
                    dest.append(out_base[i] + j)
            base += take
        order = np.argsort(np.asarray(dest, dtype=np.int64), kind="stable") if dest else np.zeros(0, dtype=np.int64)
        rows_a = np.asarray(rows, dtype=np.int32)[order] if rows else np.zeros(0, dtype=np.int32)
        dest_a = np.asarray(dest, dtype=np.int64)[order] if dest else np.zeros(0, dtype=np.int64)
        b = self.meta.upload(c_slots, c_past, c_counts, tokens, rows_a, book.tables_for(c_slots))
        W = rows_a.shape[0]
        if self._chunk_by_graph(b, W, out, dest_a):
            pass
        elif W and np.array_equal(dest_a, np.arange(dest_a[0], dest_a[0] + W)):
            self.model.forward(b, self.cache, self.ws, out[int(dest_a[0]):int(dest_a[0]) + W])
        elif W:
            mark = self.ws.mark()
            tmp = self.ws.take((W, self.model.vocab), torch.float32)
            self.model.forward(b, self.cache, self.ws, tmp)
            out.index_copy_(0, torch.from_numpy(dest_a).to(self.device), tmp)
            self.ws.release(mark)
        else:
            self.model.forward(b, self.cache, self.ws, out[:0])
        book.commit(c_slots, new_lens)

    def _chunk_by_graph(self, b, W: int, out, dest_a) -> bool:
        """A step of many tokens whose shape (tokens, sequences, longest share, wanted rows) has been seen before is
        recorded once as a CUDA graph and replayed from then on: the host then no longer issues some two hundred
        launches per step, which for short prompts is most of the step's time. Lengths, positions and tables live
        in the device buffer that the upload refreshed, so one recording serves every step of that shape. The logits
        land in a buffer of the stepper's and are copied to ``out``. Returns False if the step was not run."""
        if not (self.use_graphs and getattr(self.model, "capturable", True) and 0 < W <= self.max_graph_rows):
            return False
        self._check_graph_key()
        gkey = ("chunk", b.T, b.n, b.max_count, W)
        graph = self._graphs.get(gkey)
        if graph is None and gkey not in self._seen_chunk:
            self._seen_chunk.add(gkey)
            if len(self._seen_chunk) > 4096:
                self._seen_chunk.clear()
            return False
        if self._chunk_logits is None or self._chunk_logits.shape[0] < W:
            self._chunk_logits = torch.empty((max(W, 8), self.model.vocab), dtype=torch.float32, device=self.device)
            for k in [k for k in self._graphs if isinstance(k[0], str)]:
                del self._graphs[k]
            graph = None
        logits = self._chunk_logits[:W]
        if graph is None:
            if sum(1 for k in self._graphs if isinstance(k[0], str)) >= self.max_chunk_graphs:
                for k in [k for k in self._graphs if isinstance(k[0], str)]:
                    del self._graphs[k]
            before = ops.lib().launches
            graph = self._graphs[gkey] = self._capture(b, logits)
            self._graph_own[gkey] = ops.lib().launches - before
            ops.lib().launches = before          # captured, not run
        graph.replay()
        self.graph_kernel_launches += self._graph_own[gkey]
        if np.array_equal(dest_a, np.arange(dest_a[0], dest_a[0] + W)):
            out[int(dest_a[0]):int(dest_a[0]) + W].copy_(logits)
        else:
            out.index_copy_(0, torch.from_numpy(dest_a).to(self.device), logits)
        return True

    def _check_graph_key(self) -> None:
        """Recordings hold addresses of the workspace and of the metadata buffer: when either was replaced, they go."""
        key = (self.ws.generation, self.meta.generation)
        if key != self._graph_key:
            self._graphs.clear()
            self._graph_key = key

    # ------------------------------------------------------------------ decode ----
    def _decode(self, entries, slots, toks, floats) -> torch.Tensor:
        tokens = np.asarray([int(t[0]) for t in toks], dtype=np.int32)
        logits = self._decode_core(slots, tokens, None, floats)
        n = len(slots)
        wanted = [i for i, e in enumerate(entries) if len(e.want)]
        if len(wanted) == n:
            return logits
        if not wanted:
            return logits[:0]
        return logits.index_select(0, torch.tensor(wanted, dtype=torch.long, device=self.device))

    def decode_fed(self, slots, feed_map) -> torch.Tensor:
        """One token for each of ``slots``, taken from the device-side feed: sequence i reads
        ``feed[feed_map[i]]``, where the sampler left the tokens it chose for the previous step's rows.
        Returns the logits of every row (a view that the next step overwrites)."""
        self._raise_late_status()
        book = self.cache.book
        slots = [int(s) for s in slots]
        if len(slots) > self.meta.FEED:
            raise ValueError(f"a device-fed step takes at most {self.meta.FEED} sequences")
        for s in slots:
            if int(book.lengths[s]) + 1 > self.max_len:
                raise CacheFull(f"slot {s} would hold {int(book.lengths[s]) + 1} tokens; the longest sequence allowed "
                                f"is {self.max_len}")
        return self._decode_core(slots, None, np.asarray(feed_map, dtype=np.int32), None)

    @property
    def feed(self) -> torch.Tensor:
        return self.meta.feed

    def _decode_core(self, slots, tokens, feed_map, floats) -> torch.Tensor:
        book = self.cache.book
        n = len(slots)
        past = [int(book.lengths[s]) for s in slots]
        new_lens = [p + 1 for p in past]
        book.grow(slots, new_lens)
        rows = np.arange(n, dtype=np.int32)
        if floats is None:
            floats = np.zeros(n, dtype=np.float32)
        b = self.meta.upload(slots, past, [1] * n, tokens, rows, book.tables_for(slots), floats=floats,
                             feed_map=feed_map)
        self.last_batch = b
        if self._decode_logits is None or self._decode_logits.shape[0] < n:
            cap = max(n, 8 if self._decode_logits is None else 2 * self._decode_logits.shape[0])
            self._decode_logits = torch.empty((cap, self.model.vocab), dtype=torch.float32, device=self.device)
            self._graphs.clear()
        logits = self._decode_logits[:n]

        self._check_graph_key()
        gkey = (n, b.ids_map is not None)
        graph = self._graphs.get(gkey)
        if graph is not None:
            graph.replay()
            self.graph_kernel_launches += self._graph_own[gkey]
        elif (self.use_graphs and getattr(self.model, "capturable", True) and n <= self.max_graph_batch
              and gkey in self._seen_decode):
            before = ops.lib().launches
            self._graphs[gkey] = self._capture(b, logits)
            self._graph_own[gkey] = ops.lib().launches - before
            ops.lib().launches = before          # captured, not run
            self._graphs[gkey].replay()
            self.graph_kernel_launches += self._graph_own[gkey]
        else:
            self.model.forward(b, self.cache, self.ws, logits)
            self._seen_decode.add(gkey)
        book.commit(slots, new_lens)
        return logits

    def _capture(self, b, logits):
        torch.cuda.synchronize(self.device)
        g = torch.cuda.CUDAGraph()
        self.ws.frozen = True
        try:
            with torch.cuda.graph(g):
                self.model.forward(b, self.cache, self.ws, logits)
        finally:
            self.ws.frozen = False
        return g
