"""The generation loop: requests in, tokens out, batch after batch.

For each batch: take a slot per request, run all prompts (unequal lengths) in one step, then one
token per live sequence per step. A sequence ends on a stop token (which is kept in its output), when
its context is full, or after ``max_new_tokens``; it leaves the batch at once, its slot and pages go
back, and the others continue unchanged. Requests that do not fit the first batch run in later
ones, which reuse the slots.

The single-sequence flow and its three stop reasons are the reference's
(sleuth/forge/infer/generate.py:49-136: prompt truncated to the last ``max_len - 1`` tokens :69-70,
empty prompt refused :64-65, stop token appended then "stop_token" :116-121, "context_full" when the
cache holds ``max_len`` tokens :122-124, first new token charged to the prefill :114-115). Batches of
unequal prompts and early finishers are this library's own.

The loop decides everything on the host and talks to the GPU through a small backend (``open``,
``close``, ``prefill``, ``decode``, ``choose``), so its decisions can be tested without one.
"""

from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Callable, Protocol, Sequence

from ..cache.book import pages_for
from ..sampling.config import SamplingConfig
from ..sampling.host import NgramBlocker, fresh_seed, recent_window, uniform


@dataclass
class GenerationResult:
    prompt_ids: list[int]
    new_ids: list[int]
    stop_reason: str                    # "stop_token" | "max_new_tokens" | "context_full"
    prefill_seconds: float
    decode_seconds: float
    stats: dict = field(default_factory=dict)

    @property
    def decode_tok_per_s(self) -> float:
        n = max(0, len(self.new_ids) - 1)   # the first new token comes from the prompt's step
        return n / self.decode_seconds if self.decode_seconds > 0 else 0.0

    @property
    def prefill_tok_per_s(self) -> float:
        return len(self.prompt_ids) / self.prefill_seconds if self.prefill_seconds > 0 else 0.0


class Backend(Protocol):
    max_len: int
    vocab: int
    total_pages: int

    def open(self, n: int) -> list[int]: ...
    def close(self, slots: Sequence[int]) -> None: ...
    def prefill(self, slots: Sequence[int], prompts: Sequence[Sequence[int]]): ...
    def decode(self, slots: Sequence[int], tokens: Sequence[int]): ...
    def choose(self, logits, cfg: SamplingConfig, uniforms, vocab_limit, recent, banned) -> list[int]: ...
    def free_pages(self) -> int: ...
    def pages_needed(self, slots: Sequence[int], new_lengths: Sequence[int]) -> int: ...
    def length(self, slot: int) -> int: ...
    def sync(self) -> None: ...
    # optional, for the pipelined loop (``pipelined = True``):
    #   choose_later(logits, cfg, uniforms, vocab_limit) -> callable giving the tokens once they are on the host;
    #       the tokens also stay on the device, row i of them in feed slot i
    #   decode_fed(slots, feed_map) -> logits: sequence i continues with the token in feed slot feed_map[i]


@dataclass
class _Live:
    request: int
    slot: int
    prompt: list[int]
    new: list[int] = field(default_factory=list)
    blocker: NgramBlocker | None = None


def plan_batches(prompt_lengths: Sequence[int], max_new_tokens: int, max_len: int, total_pages: int,
                 max_batch: int) -> list[list[int]]:
    """Split request indices, in order, into batches. A batch holds at most ``max_batch`` requests and
    only as many as the cache can hold at their longest (prompt plus new tokens, capped by the
    context); a request too long for that on its own still gets a batch to itself."""
    batches, cur, pages = [], [], 0
    for i, n in enumerate(prompt_lengths):
        need = pages_for(min(n + max_new_tokens, max_len))
        if cur and (len(cur) >= max_batch or pages + need > total_pages):
            batches.append(cur)
            cur, pages = [], 0
        cur.append(i)
        pages += need
    if cur:
        batches.append(cur)
    return batches


def generate_batches(backend: Backend, prompts: Sequence[Sequence[int]], max_new_tokens: int = 200,
                     sampling: SamplingConfig | None = None, stop_ids=None, vocab_limit: int | None = None,
                     seed: int | None = None, on_token: Callable[[int, int], None] | None = None,
                     max_batch: int = 64) -> list[GenerationResult]:
    """Generate for every prompt; results come back in the order of ``prompts``.

    on_token(request_index, token) is called for each new token as it is produced.
    Request ``i`` draws from the random stream (seed, i), whatever batch it lands in."""
    sampling = sampling or SamplingConfig()
    stop_ids = set(stop_ids or ())
    seed = fresh_seed() if seed is None else int(seed)
    cleaned = []
    for i, p in enumerate(prompts):
        p = [int(t) for t in p]
        if not p:
            raise ValueError(f"prompt {i} is empty: a prompt must contain at least one token")
        if len(p) >= backend.max_len:
            p = p[-(backend.max_len - 1):]      # keep the most recent context
        cleaned.append(p)
    results: list[GenerationResult | None] = [None] * len(cleaned)
    if max_new_tokens <= 0:
        return [GenerationResult(p, [], "max_new_tokens", 0.0, 0.0) for p in cleaned]
    # Penalties and n-gram bans need the newest token on the host before the next choice; everything else can run
    # one step ahead of the host (see _run_batch_pipelined).
    pipelined = getattr(backend, "pipelined", False) and not sampling.needs_context
    run = _run_batch_pipelined if pipelined else _run_batch
    for batch in plan_batches([len(p) for p in cleaned], max_new_tokens, backend.max_len, backend.total_pages,
                              max_batch):
        run(backend, batch, cleaned, results, max_new_tokens, sampling, stop_ids, vocab_limit, seed, on_token)
    return results  # type: ignore[return-value]


def _run_batch(backend, batch, prompts, results, max_new_tokens, sampling, stop_ids, vocab_limit, seed, on_token):
    slots = backend.open(len(batch))
    live = [_Live(r, s, prompts[r]) for r, s in zip(batch, slots)]
    if sampling.no_repeat_ngram > 0:
        for q in live:
            q.blocker = NgramBlocker(sampling.no_repeat_ngram, q.prompt)
    held = set(slots)
    try:
        backend.sync()
        t0 = time.perf_counter()
        logits = backend.prefill([q.slot for q in live], [q.prompt for q in live])
        t1 = t0
        for step in range(max_new_tokens):
            us = None if sampling.greedy else [uniform(seed, q.request, step) for q in live]
            recent = banned = None
            if sampling.repetition_penalty != 1.0:
                recent = [recent_window(q.prompt + q.new, sampling.repeat_last_n) for q in live]
            if sampling.no_repeat_ngram > 0:
                banned = [q.blocker.banned() for q in live]
            tokens = backend.choose(logits, sampling, us, vocab_limit, recent, banned)   # synchronises
            now = time.perf_counter()
            if step == 0:
                t1 = now                         # the prompt's step ends once the first tokens exist
            keep = []
            for q, tok in zip(live, tokens):
                q.new.append(tok)
                if q.blocker is not None:
                    q.blocker.add(tok)
                if on_token is not None:
                    on_token(q.request, tok)
                reason = None
                if tok in stop_ids:
                    reason = "stop_token"
                elif backend.length(q.slot) >= backend.max_len:
                    reason = "context_full"
                elif step + 1 >= max_new_tokens:
                    reason = "max_new_tokens"
                if reason is None:
                    keep.append(q)
                else:
                    _finish(backend, q, reason, results, t0, t1, now, held)
            # sequences that would need a page the cache no longer has end here
            while keep and backend.pages_needed([q.slot for q in keep],
                                                [backend.length(q.slot) + 1 for q in keep]) > backend.free_pages():
                q = max(keep, key=lambda q: backend.length(q.slot))
                keep.remove(q)
                _finish(backend, q, "context_full", results, t0, t1, now, held)
            live = keep
            if not live:
                break
            logits = backend.decode([q.slot for q in live], [q.new[-1] for q in live])
    finally:
        if held:
            backend.close(sorted(held))


def _run_batch_pipelined(backend, batch, prompts, results, max_new_tokens, sampling, stop_ids, vocab_limit, seed,
                         on_token):
    """The same decisions as ``_run_batch`` with the host one step behind the GPU.

    The chosen tokens stay on the device and the next step reads them there, so step k + 1 is launched before the
    host has seen the tokens of step k; the host then reads them while the GPU works. Whether a sequence goes on
    is known without its newest token except for one reason, a stop token: a sequence that has just produced one
    is therefore carried through one more step, whose result is thrown away. Its outputs, its stop reason and the
    other sequences' results are exactly those of the step-by-step loop."""
    slots = backend.open(len(batch))
    rows = [_Live(r, s, prompts[r]) for r, s in zip(batch, slots)]      # in the order of the pending tokens
    held = set(slots)
    done: set[int] = set()                                               # requests that have ended

    def uniforms(live, step):
        return None if sampling.greedy else [uniform(seed, q.request, step) for q in live]

    try:
        backend.sync()
        t0 = time.perf_counter()
        logits = backend.prefill([q.slot for q in rows], [q.prompt for q in rows])
        pending = backend.choose_later(logits, sampling, uniforms(rows, 0), vocab_limit)
        t1 = None
        k = 0                                   # index of the pending tokens among each sequence's new tokens
        while rows:
            # who is fed its pending token: decided from counts alone
            why_not = {}
            for q in rows:
                if q.request in done:
                    continue
                if backend.length(q.slot) >= backend.max_len:
                    why_not[q.request] = "context_full"
                elif k + 1 >= max_new_tokens:
                    why_not[q.request] = "max_new_tokens"
            cont = [q for q in rows if q.request not in done and q.request not in why_not]
            while cont and backend.pages_needed([q.slot for q in cont],
                                                [backend.length(q.slot) + 1 for q in cont]) > backend.free_pages():
                q = max(cont, key=lambda q: backend.length(q.slot))
                cont.remove(q)
                why_not[q.request] = "context_full"
            next_pending = None
            if cont:
                index = {q.request: i for i, q in enumerate(rows)}
                logits = backend.decode_fed([q.slot for q in cont], [index[q.request] for q in cont])
                next_pending = backend.choose_later(logits, sampling, uniforms(cont, k + 1), vocab_limit)
            # now the host catches up with the tokens of step k
            tokens = pending()
            now = time.perf_counter()
            if t1 is None:
                t1 = now
            for q, tok in zip(rows, tokens):
                if q.request in done:
                    continue                    # carried along after its stop token: not its token any more
                q.new.append(tok)
                if on_token is not None:
                    on_token(q.request, tok)
                reason = "stop_token" if tok in stop_ids else why_not.get(q.request)
                if reason is not None:
                    done.add(q.request)
                    _finish(backend, q, reason, results, t0, t1, now, held)
            rows, pending, k = cont, next_pending, k + 1
            if not any(q.request not in done for q in rows):
                break
    finally:
        if held:
            backend.close(sorted(held))


def _finish(backend, q: _Live, reason: str, results, t0, t1, now, held) -> None:
    results[q.request] = GenerationResult(q.prompt, q.new, reason, t1 - t0, now - t1,
                                          {"slot": q.slot})
    backend.close([q.slot])
    held.discard(q.slot)
