"""The Python entry point: a model folder in, an ``Engine`` that steps and generates out.

In the reference's manner (sleuth/models.py:44-79 ``load_any(path, device, dtype, max_seq_len)`` and
sleuth/forge/infer/generate.py:50-52 ``generate(model, prompt_ids, max_new_tokens, sampling, stop_ids,
vocab_limit, seed, on_token, cuda_graph)``)::

    engine = load("model-dir", dtype="bf16", max_seq_len=4096)
    result = generate(engine, prompt_ids, max_new_tokens=200, sampling=SamplingConfig(temperature=0))
    results = engine.generate([ids_a, ids_b, ...], ...)          # a batch of unequal prompts

The model class is chosen by ``config.json`` through the architecture registry. Everything runs on
one CUDA device; there is no CPU path.
"""

from __future__ import annotations

from pathlib import Path
from typing import Callable, Sequence

import numpy as np
import torch

from ..cache.paged import PagedCache
from ..config.base import read_config_json
from ..config.registry import parse_config
from ..parts.base import BuildContext
from ..kernels import ops
from ..sampling.config import SamplingConfig
from ..sampling.sampler import Sampler
from ..weights.loader import load_into
from ..weights.safetensors import Checkpoint
from .generate import GenerationResult, generate_batches
from .model import Model
from .stepper import StepEntry, Stepper

_DTYPES = {"bf16": torch.bfloat16, "bfloat16": torch.bfloat16, "fp32": torch.float32, "float32": torch.float32,
           "auto": torch.bfloat16, None: torch.bfloat16, torch.bfloat16: torch.bfloat16, torch.float32: torch.float32}


def resolve_dtype(dtype) -> torch.dtype:
    """"auto" and None mean bfloat16, the reference's default on CUDA (sleuth/models.py:39-41).
    float16 is not a run dtype here."""
    try:
        return _DTYPES[dtype]
    except KeyError:
        raise ValueError(f"dtype {dtype!r} is not supported: use 'bf16' (or 'bfloat16', 'auto') or 'fp32' "
                         f"(or 'float32')") from None


class Engine:
    """A loaded model with its cache, step function, sampler and generation loop."""

    def __init__(self, config, spec, model: Model, cache: PagedCache, device, dtype, max_seq_len: int,
                 unread_keys=(), use_graphs: bool = True, max_step_tokens: int = 8192):
        self.config, self.spec, self.model, self.cache = config, spec, model, cache
        self.device, self.dtype = torch.device(device), dtype
        self.unread_keys = list(unread_keys)
        self.max_len = int(max_seq_len)
        self.stepper = Stepper(model, cache, device, max_len=self.max_len, max_step_tokens=max_step_tokens,
                               use_graphs=use_graphs)
        self.sampler = Sampler(device, model.vocab)
        self.vocab = model.vocab
        self.total_pages = cache.n_pages

    # ------------------------------------------------------------------ loading ----
    @classmethod
    def from_pretrained(cls, folder, dtype="bf16", max_seq_len: int = 4096, max_tokens: int | None = None,
                        device="cuda:0", use_graphs: bool = True, max_step_tokens: int = 8192,
                        max_sequences: int | None = None) -> "Engine":
        """Load ``folder`` (``config.json`` + safetensors).

        max_seq_len: the longest sequence (prompt plus new tokens); capped by the model's
        ``max_position_embeddings`` (sleuth/formats/hf.py:96). max_tokens: how many tokens all live
        sequences may hold together (each rounded up to 64); sizes the cache. Default: 8 sequences
        of ``max_seq_len``. max_sequences: how many sequences may be live at once (sizes the slot tables and
        any per-sequence state; see ``PagedCache``)."""
        if not torch.cuda.is_available():
            raise RuntimeError("sleuth_b200 runs on an NVIDIA GPU only; torch.cuda.is_available() is False")
        run_dtype = resolve_dtype(dtype)
        device = torch.device(device)
        torch.cuda.set_device(device)
        folder = Path(folder)
        arch, cfg, unread = parse_config(read_config_json(folder))
        with Checkpoint(folder) as ckpt:
            spec = arch.model_spec(cfg, tensor_names=set(ckpt.names()))
            max_seq_len = max(1, min(int(max_seq_len), spec.max_positions))
            ctx = BuildContext(device=device, dtype=run_dtype, max_positions=-(-max_seq_len // 64) * 64)
            model = Model(spec, ctx)
            tensors = load_into(model.expected(), ckpt, run_dtype, device, ignored=spec.ignored_tensors)
            model.bind(tensors)
            del tensors
        if max_tokens is None:
            max_tokens = 8 * max_seq_len
        cache = PagedCache(model.cache_requests, max_tokens, max_seq_len, run_dtype, device, max_sequences)
        return cls(cfg, spec, model, cache, device, run_dtype, max_seq_len, unread, use_graphs, max_step_tokens)

    @classmethod
    def from_config(cls, config_json: dict, seed: int = 0, dtype="bf16", max_seq_len: int = 4096,
                    max_tokens: int | None = None, device="cuda:0", use_graphs: bool = True,
                    max_step_tokens: int = 8192, std: float = 0.02, max_sequences: int | None = None) -> "Engine":
        """A model with random weights drawn on the device from a ``config.json`` dictionary and a
        seed: matrices and biases ~ N(0, std), norm gains ~ 1 + N(0, std). Nothing is written to disk
        (``weights.write_random_model`` writes a folder instead, with a generator that is the same on
        every machine)."""
        if not torch.cuda.is_available():
            raise RuntimeError("sleuth_b200 runs on an NVIDIA GPU only; torch.cuda.is_available() is False")
        run_dtype = resolve_dtype(dtype)
        device = torch.device(device)
        torch.cuda.set_device(device)
        arch, cfg, unread = parse_config(config_json)
        spec = arch.model_spec(cfg)
        max_seq_len = max(1, min(int(max_seq_len), spec.max_positions))
        ctx = BuildContext(device=device, dtype=run_dtype, max_positions=-(-max_seq_len // 64) * 64)
        model = Model(spec, ctx)
        gen = torch.Generator(device=device)
        gen.manual_seed(int(seed))
        tensors = {}
        for name, d in sorted(model.expected().items()):
            if d.role == "table":
                tensors[name] = torch.zeros(d.shape, dtype=torch.int32, device=device)
                continue
            t = torch.randn(d.shape, generator=gen, device=device, dtype=torch.float32) * std
            if d.init == "gain":
                t += 1.0
            tensors[name] = t.to(run_dtype) if d.role == "matrix" else t
        model.bind(tensors)
        del tensors
        if max_tokens is None:
            max_tokens = 8 * max_seq_len
        cache = PagedCache(model.cache_requests, max_tokens, max_seq_len, run_dtype, device, max_sequences)
        return cls(cfg, spec, model, cache, device, run_dtype, max_seq_len, unread, use_graphs, max_step_tokens)

    # ------------------------------------------------------------------ stepping ----
    def open(self, n: int) -> list[int]:
        return self.cache.open(n)

    def close(self, slots: Sequence[int]) -> None:
        self.cache.close(slots)

    def step(self, entries) -> torch.Tensor:
        """entries: ``StepEntry`` objects or ``(slot, tokens, want)`` tuples. See ``Stepper.step``."""
        return self.stepper.step([e if isinstance(e, StepEntry) else StepEntry(*e) for e in entries])

    # ---- what the generation loop needs (the ``Backend`` protocol of engine/generate.py) ----
    def prefill(self, slots, prompts):
        return self.stepper.step([StepEntry(s, p, (len(p) - 1,)) for s, p in zip(slots, prompts)])

    def decode(self, slots, tokens):
        return self.stepper.step([StepEntry(s, (t,), (0,)) for s, t in zip(slots, tokens)])

    pipelined = True      # the generation loop may run one step ahead of the host (engine/generate.py)

    def choose_later(self, logits, cfg, uniforms, vocab_limit):
        """Choose into the device-side token feed and start copying the tokens to the host."""
        u = None if uniforms is None else np.asarray(uniforms, dtype=np.float32)
        if logits.shape[0] > self.stepper.feed.numel():
            tokens = self.sampler.choose(logits, cfg, u, vocab_limit)
        else:
            tokens = self.sampler.choose(logits, cfg, u, vocab_limit, out=self.stepper.feed)
        return self.sampler.to_host_later(tokens)

    def decode_fed(self, slots, feed_map):
        return self.stepper.decode_fed(slots, feed_map)

    def choose(self, logits, cfg, uniforms, vocab_limit, recent, banned) -> list[int]:
        u = None if uniforms is None else np.asarray(uniforms, dtype=np.float32)
        return self.sampler.to_host(self.sampler.choose(logits, cfg, u, vocab_limit, recent, banned))

    def free_pages(self) -> int:
        return min(g.pool.free for g in self.cache.book.groups) if self.cache.book.groups else 1 << 30

    def pages_needed(self, slots, new_lengths) -> int:
        need = self.cache.book.pages_needed(slots, new_lengths)
        return max(need) if need else 0

    def length(self, slot: int) -> int:
        return int(self.cache.book.lengths[slot])

    def sync(self) -> None:
        torch.cuda.synchronize(self.device)

    # ------------------------------------------------------------------ generation ----
    def generate(self, prompts, max_new_tokens: int = 200, sampling: SamplingConfig | None = None, stop_ids=None,
                 vocab_limit: int | None = None, seed: int | None = None,
                 on_token: Callable[[int, int], None] | None = None, cuda_graph: bool = True,
                 max_batch: int = 64) -> list[GenerationResult]:
        """Generate for a list of prompts (token id lists of unequal lengths).

        stop_ids default to the ``eos_token_id`` of ``config.json``. ``cuda_graph=False`` runs every
        decode step launch by launch."""
        if stop_ids is None:
            stop_ids = set(getattr(self.config, "stop_ids", ()))
        before = self.stepper.use_graphs
        self.stepper.use_graphs = before and cuda_graph
        max_batch = max(1, min(int(max_batch), self.cache.max_slots))
        self.pipelined = len(prompts) <= self.stepper.feed.numel() and max_batch <= self.stepper.feed.numel()
        try:
            results = generate_batches(self, prompts, max_new_tokens, sampling, stop_ids, vocab_limit, seed, on_token,
                                       max_batch)
        finally:
            self.stepper.use_graphs = before
        # every token has been read back, so the device is idle: one look at the status word that the tensor-memory
        # kernels write when a bounded wait gives up (their results would be wrong, and nothing else would say so)
        ops.gemm_tc_check(self.device)
        for r in results:
            r.stats.update(kv_cache_mb=round(self.cache.nbytes() / 1e6, 2), device=str(self.device),
                           dtype=str(self.dtype).replace("torch.", ""))
        return results


def load(path, dtype="bf16", max_seq_len: int = 4096, max_tokens: int | None = None, device="cuda:0",
         **kw) -> Engine:
    """Load a model folder; the counterpart of the reference's ``load_any`` (sleuth/models.py:44-79)."""
    return Engine.from_pretrained(path, dtype=dtype, max_seq_len=max_seq_len, max_tokens=max_tokens, device=device, **kw)


def generate(engine: Engine, prompt_ids: Sequence[int], max_new_tokens: int = 200,
             sampling: SamplingConfig | None = None, stop_ids=None, vocab_limit: int | None = None,
             seed: int | None = None, on_token: Callable[[int], None] | None = None,
             cuda_graph: bool = True) -> GenerationResult:
    """Generate after one prompt; the counterpart of the reference's ``generate``
    (sleuth/forge/infer/generate.py:50-52), same argument names and meanings."""
    cb = None if on_token is None else (lambda request, tok: on_token(tok))
    return engine.generate([list(prompt_ids)], max_new_tokens, sampling, stop_ids, vocab_limit, seed, cb,
                           cuda_graph)[0]
