"""Command line: ``python -m sleuth_b200 generate <model-dir> ...`` and ``python -m sleuth_b200 replay ...``.

``generate`` follows the reference's command of the same name (sleuth/cli.py:769-806 for the options,
:174-256 for the flow): same option names, defaults and meanings for ``--dtype``, ``--prompt``,
``--max-new-tokens``, ``--temperature`` (0.8), ``--top-k`` (0), ``--top-p`` (1.0), ``--min-p`` (0.05 on
the command line), ``--repetition-penalty``, ``--repeat-last-n``, ``--no-repeat-ngram``, ``--seed``
(sample i uses seed + i, cli.py:228), ``--samples``, ``--device``, ``--cuda-graph``; a throw-away
two-token run warms everything up before timing (cli.py:199-214); the closing line reports tokens,
stop reason, prompt time, decode speed and peak memory (cli.py:252-254).

Text needs a tokenizer, which lies outside this library (tokens in, tokens out): ``--prompt-ids``
takes comma- or space-separated token ids (several prompts separated by ``;`` run as one batch) and
the new ids are printed. ``--prompt`` works when the model folder has a ``tokenizer.json`` and the
``tokenizers``-free byte-level BPE reader is given by the user through ``--tokenizer``; otherwise it
explains what to pass instead. Options of the reference that belong to parts this library does not
have (``--step``, ``--draft*``, ``--keep-quantized``, ``--chat``) are not offered.
"""

from __future__ import annotations

import argparse
import sys


def _dtype_name(name: str) -> str:
    return {"auto": "bf16", "bf16": "bf16", "fp32": "fp32"}[name]


def _parse_ids(text: str) -> list[list[int]]:
    prompts = []
    for part in text.split(";"):
        ids = [int(t) for t in part.replace(",", " ").split()]
        if ids:
            prompts.append(ids)
    return prompts


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="sleuth_b200", description="Qwen3 generation on one B200")
    sub = ap.add_subparsers(dest="command", required=True)

    s = sub.add_parser("generate", help="generate tokens from a model folder (config.json + safetensors)")
    s.add_argument("path", help="a model folder with config.json and model.safetensors")
    s.add_argument("--dtype", choices=["auto", "fp32", "bf16"], default="auto",
                   help="auto = bf16; fp32 = true 32-bit arithmetic everywhere")
    s.add_argument("--prompt", default="", help="text prompt (needs --tokenizer)")
    s.add_argument("--prompt-ids", default="", help="token ids, e.g. '1 2 3' or '1,2,3; 7,8' for a batch of two")
    s.add_argument("--max-new-tokens", type=int, default=200)
    s.add_argument("--temperature", type=float, default=0.8)
    s.add_argument("--top-k", type=int, default=0)
    s.add_argument("--top-p", type=float, default=1.0)
    s.add_argument("--min-p", type=float, default=0.05)
    s.add_argument("--repetition-penalty", type=float, default=1.0,
                   help="above 1 makes recently used tokens less likely, e.g. 1.1-1.3 (1 = off)")
    s.add_argument("--repeat-last-n", type=int, default=64,
                   help="the repetition penalty looks at this many recent tokens (0 = the whole context)")
    s.add_argument("--no-repeat-ngram", type=int, default=0, metavar="N",
                   help="never repeat a phrase of N tokens (0 = off)")
    s.add_argument("--seed", type=int, default=None)
    s.add_argument("--samples", type=int, default=1)
    s.add_argument("--device", default="auto", help="auto = cuda:0")
    s.add_argument("--tokenizer", default=None, help="a Python 'module:function' returning (encode, decode) callables")
    s.add_argument("--cuda-graph", dest="cuda_graph", action="store_true", default=True,
                   help="replay each decode step as one CUDA graph (default)")
    s.add_argument("--no-cuda-graph", dest="cuda_graph", action="store_false", help="launch every kernel separately")
    s.add_argument("--stop-id", type=int, action="append", default=None,
                   help="stop at this token id (repeatable; default: eos_token_id of config.json)")
    s.add_argument("--max-seq-len", type=int, default=4096, help="longest sequence, prompt plus new tokens")
    s.set_defaults(fn=cmd_generate)

    r = sub.add_parser("replay", help="feed token traces through a model and write logits (see bin/trace_run)")
    r.add_argument("rest", nargs=argparse.REMAINDER)
    r.set_defaults(fn=cmd_replay)

    w = sub.add_parser("random-model", help="write a model folder with seeded random weights from a config.json")
    w.add_argument("config", help="path of a config.json")
    w.add_argument("out", help="folder to create")
    w.add_argument("--seed", type=int, default=0)
    w.add_argument("--dtype", choices=["bf16", "fp32"], default="bf16")
    w.set_defaults(fn=cmd_random_model)
    return ap


def _tokenizer(spec: str | None):
    if not spec:
        return None
    import importlib
    mod, _, fn = spec.partition(":")
    return getattr(importlib.import_module(mod), fn or "load")()


def cmd_generate(a) -> int:
    import torch

    from .engine.engine import load
    from .sampling.config import SamplingConfig

    tok = _tokenizer(a.tokenizer)
    if a.prompt_ids:
        prompts = _parse_ids(a.prompt_ids)
    elif tok is not None:
        prompts = [list(tok[0](a.prompt))]
    else:
        print("generate: give --prompt-ids (token ids), or --tokenizer module:function together with --prompt; "
              "this library goes from tokens to tokens and ships no tokenizer", file=sys.stderr)
        return 2
    device = "cuda:0" if a.device == "auto" else a.device
    engine = load(a.path, dtype=_dtype_name(a.dtype), max_seq_len=a.max_seq_len, device=device,
                  max_tokens=max(1, len(prompts)) * a.max_seq_len)
    sampling = SamplingConfig(a.temperature, a.top_k, a.top_p, a.min_p, a.repetition_penalty, a.repeat_last_n,
                              a.no_repeat_ngram)
    n_params = sum(int(torch.tensor(d.shape).prod()) for d in engine.model.expected().values())
    print(f"[{engine.spec.__class__.__name__} of {type(engine.config).__name__}, {n_params / 1e6:.2f}M params, "
          f"{engine.device}, {str(engine.dtype).replace('torch.', '')}]", file=sys.stderr, flush=True)
    stop_ids = set(a.stop_id) if a.stop_id is not None else None
    engine.generate([[prompts[0][0]] * 8], 2, sampling, seed=0, cuda_graph=a.cuda_graph)     # warm-up
    for i in range(a.samples):
        seed = None if a.seed is None else a.seed + i
        res = engine.generate(prompts, a.max_new_tokens, sampling, stop_ids=stop_ids, seed=seed, cuda_graph=a.cuda_graph)
        for r in res:
            if tok is not None:
                print(tok[1](r.new_ids), flush=True)
            else:
                print(" ".join(str(t) for t in r.new_ids), flush=True)
            mem = f", peak GPU memory {torch.cuda.max_memory_allocated(engine.device) / 2**30:.2f} GiB"
            print(f"[{len(r.new_ids)} tokens, stop: {r.stop_reason}, prompt {len(r.prompt_ids)} tokens in "
                  f"{r.prefill_seconds * 1000:.0f} ms, decode {r.decode_tok_per_s:,.1f} tok/s{mem}]",
                  file=sys.stderr, flush=True)
        if i + 1 < a.samples:
            print("-" * 40, flush=True)
    return 0


def cmd_replay(a) -> int:
    from .replay import main as replay_main
    return replay_main(a.rest)


def cmd_random_model(a) -> int:
    import json

    import torch

    from .weights.random_init import write_random_model
    cfg = json.load(open(a.config))
    out = write_random_model(a.out, cfg, seed=a.seed, dtype=torch.bfloat16 if a.dtype == "bf16" else torch.float32)
    print(out)
    return 0


def main(argv=None) -> int:
    a = build_parser().parse_args(argv)
    return a.fn(a)
