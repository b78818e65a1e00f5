"""Choosing next tokens on the GPU from a logits matrix, for a batch of rows at once.

Pipeline and option meanings are the reference's (sleuth/forge/infer/sampling.py:99-127): ban list,
repetition penalty, then greedy argmax for temperature <= 0, else temperature, top-k, top-p, min-p
and a draw. The kernels are in ``csrc/sampling.cu``.
"""

from __future__ import annotations

import numpy as np
import torch

from ..kernels import ops
from .config import SamplingConfig


class Sampler:
    def __init__(self, device, vocab: int):
        self.device = torch.device(device)
        self.vocab = vocab
        self._out = torch.zeros(1024, dtype=torch.int32, device=self.device)
        self._host = torch.zeros(1024, dtype=torch.int32).pin_memory()
        self._scratch = torch.zeros(ops.argmax_scratch_words(1024), dtype=torch.int32, device=self.device)

    def _fit(self, n: int) -> None:
        if n > self._out.numel():
            self._out = torch.zeros(2 * n, dtype=torch.int32, device=self.device)
            self._host = torch.zeros(2 * n, dtype=torch.int32).pin_memory()
            self._scratch = torch.zeros(ops.argmax_scratch_words(2 * n), dtype=torch.int32, device=self.device)

    def choose(self, logits: torch.Tensor, cfg: SamplingConfig, uniform: torch.Tensor | np.ndarray | None = None,
               vocab_limit: int | None = None, recent: list[list[int]] | None = None,
               banned: list[list[int]] | None = None, out: torch.Tensor | None = None) -> torch.Tensor:
        """Tokens for the rows of ``logits`` [n, vocab] as a device int32 tensor [n].

        ``logits`` is changed in place when a ban list or a repetition penalty applies. ``recent``
        and ``banned`` hold, per row, each token at most once."""
        n = logits.shape[0]
        self._fit(n)
        limit = min(vocab_limit or self.vocab, logits.shape[1])
        stream = ops.current_stream()
        rec_t = nrec_t = ban_t = nban_t = None
        if recent is not None and cfg.repetition_penalty != 1.0 and any(recent):
            rec_t, nrec_t = self._ragged(recent)
        if banned is not None and any(banned):
            # a ban that would forbid every token is ignored (sampling.py:118-120)
            banned = [b if len({t for t in b if t < limit}) < limit else [] for b in banned]
            if any(banned):
                ban_t, nban_t = self._ragged(banned)
        if rec_t is not None or ban_t is not None:
            ops.penalize(logits, limit, rec_t, nrec_t, cfg.repetition_penalty, ban_t, nban_t, stream)
        out = self._out[:n] if out is None else out[:n]
        if cfg.greedy:
            ops.argmax(logits, limit, out, self._scratch, stream)
        else:
            if uniform is None:
                raise ValueError("sampling with a temperature needs one uniform number per row")
            if not isinstance(uniform, torch.Tensor):
                uniform = self._upload(np.asarray(uniform, dtype=np.float32))
            ops.sample(logits, limit, cfg.temperature, cfg.top_k, cfg.top_p, cfg.min_p, uniform, out, stream)
        return out

    def _upload(self, values: np.ndarray) -> torch.Tensor:
        """The uniform numbers of a step on the device, through one of four pinned buffers: the copy is asynchronous,
        so a loop that runs ahead of the GPU is not held up; a buffer is reused only when its last copy is done."""
        n = values.size
        if not hasattr(self, "_u_ring") or self._u_ring[0][0].numel() < n:
            cap = max(1024, 2 * n)
            self._u_ring = [(torch.zeros(cap, dtype=torch.float32).pin_memory(),
                             torch.zeros(cap, dtype=torch.float32, device=self.device), torch.cuda.Event())
                            for _ in range(4)]
            self._u_turn, self._u_used = 0, [False] * 4
        host, dev, ev = self._u_ring[self._u_turn]
        if self._u_used[self._u_turn]:
            ev.synchronize()
        host[:n].copy_(torch.from_numpy(values.reshape(-1)))
        dev[:n].copy_(host[:n], non_blocking=True)
        ev.record(torch.cuda.current_stream(self.device))
        self._u_used[self._u_turn] = True
        self._u_turn = (self._u_turn + 1) % 4
        return dev[:n]

    def to_host(self, tokens: torch.Tensor) -> list[int]:
        n = tokens.numel()
        self._host[:n].copy_(tokens, non_blocking=True)
        torch.cuda.current_stream(self.device).synchronize()
        return self._host[:n].tolist()

    def to_host_later(self, tokens: torch.Tensor):
        """Start copying ``tokens`` to the host; returns a function that waits for the copy and gives the list.
        Up to four such copies may be pending."""
        n = tokens.numel()
        if not hasattr(self, "_ring"):
            self._ring, self._turn = [torch.zeros(4096, dtype=torch.int32).pin_memory() for _ in range(4)], 0
        buf = self._ring[self._turn]
        self._turn = (self._turn + 1) % len(self._ring)
        if n > buf.numel():
            raise ValueError(f"{n} tokens are more than a pending copy holds ({buf.numel()})")
        buf[:n].copy_(tokens, non_blocking=True)
        ev = torch.cuda.Event()
        ev.record(torch.cuda.current_stream(self.device))

        def wait() -> list[int]:
            ev.synchronize()
            return buf[:n].tolist()
        return wait

    def _ragged(self, lists: list[list[int]]):
        width = max(1, max(len(x) for x in lists))
        a = np.full((len(lists), width), -1, dtype=np.int32)
        for i, x in enumerate(lists):
            a[i, :len(x)] = x
        counts = np.asarray([len(x) for x in lists], dtype=np.int32)
        return torch.from_numpy(a).to(self.device), torch.from_numpy(counts).to(self.device)
