#!/usr/bin/env python3
"""Decode and prefill throughput of the Qwen3-0.6B-shaped model on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

Prints ONE JSON line. ``value`` is decoded tokens per second at batch 8 (2,048-token prompts, context
growing towards 4,096), timed on the device with CUDA events over exactly K decode steps after W
warm-up steps; a step is one decode step of the whole batch including the choice of the next tokens.
``e2e`` is the same through the Python entry point (``Engine.generate``: host token lists in, host
token lists out, one host-to-device copy of the step's tables and one device-to-host read of the
chosen tokens per step). ``prefill`` is one 2,048-token prompt; ``roofline`` relates the decode step to the
memory bandwidth. ``points`` holds decode at batch 1 (device-timed and through ``generate``) and 64, the
4B-shaped configuration (16 ragged prompts of 64..2,048 tokens, 256 steps through ``generate``, greedy and
at temperature 0.8) and the 8B-shaped one (untied, batch 64, 4,096-token prompts), each with its fraction
of the memory bandwidth; ``fp32`` is the true 32-bit path at the 0.6B sizes (decode at batch 8, one
2,048-token prompt) against its own rooflines. Weights are random (N(0, 0.02)), token ids are seeded
uniform: there is no dataset. ``--skip-other-configs`` leaves the 32-bit block and the larger shapes out.

``--impl reference`` runs tbertha35/Sleuth itself (installed under baseline/_ref) on the same shapes
through its own model, cache and sampling code: its eager batch-8 loop after one untimed pass, best of
three, and for batch 1 its own ``generate()`` with and without its CUDA-graph decoder.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

CONFIG = {  # BASELINE.json configs[2]: Qwen3-0.6B-shaped
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "vocab_size": 151936, "hidden_size": 1024,
    "intermediate_size": 3072, "num_hidden_layers": 28, "num_attention_heads": 16, "num_key_value_heads": 8,
    "head_dim": 128, "rope_theta": 1000000.0, "rms_norm_eps": 1e-6, "attention_bias": False,
    "tie_word_embeddings": True, "max_position_embeddings": 40960,
}
PROMPT, CONTEXT, BATCH = 2048, 4096, 8
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


def peaks() -> dict:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            d = json.load(open(path))
            out = {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]), "source": "measured"}
            if "bf16_tflops_sustained" in d:
                out["bf16_tflops_sustained"] = float(d["bf16_tflops_sustained"])
            return out
        except (KeyError, ValueError, TypeError):
            pass
    return dict(FALLBACK_PEAKS)


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a timed region runs."""

    FIELDS = ["clocks.sm", "clocks.max.sm", "clocks_event_reasons.hw_slowdown",
              "clocks_event_reasons.hw_thermal_slowdown", "clocks_event_reasons.sw_thermal_slowdown",
              "clocks_event_reasons.sw_power_cap"]

    def __init__(self):
        self.rows, self.proc, self.thread = [], None, None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", "--query-gpu=" + ",".join(self.FIELDS),
                                          "--format=csv,noheader,nounits", "-lms", "200"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.time(), [c.strip() for c in line.split(",")]))

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self, windows, slack: float = 0.0) -> dict:
        """Over the samples taken inside the timed regions (every 200 ms: a query costs the GPU's driver a moment, and
        at 100 ms the end-to-end figure lost up to 6 %); if a short run caught none inside, over those within half a
        second of a region, and the result says so."""
        sm, mx, reasons = [], [], set()
        for t, cols in self.rows:
            if len(cols) != len(self.FIELDS) or not any(a - slack <= t <= b + slack for a, b in windows):
                continue
            try:
                sm.append(float(cols[0]))
                mx.append(float(cols[1]))
            except ValueError:
                continue
            for name, val in zip(self.FIELDS[2:], cols[2:]):
                if val.lower().startswith("active"):
                    reasons.add(name.split(".")[-1])
        if not sm:
            if slack == 0.0:
                near = self.summary(windows, slack=0.5)
                near["note"] = "no sample fell inside a timed region; these lie within 0.5 s of one"
                return near
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm)}


def layer_matrix_params(c) -> int:
    d, hd = c["hidden_size"], c["head_dim"]
    H, K, I = c["num_attention_heads"], c["num_key_value_heads"], c["intermediate_size"]
    return d * (H + 2 * K) * hd + H * hd * d + 3 * d * I


def prefill_flops(c, T: int) -> float:
    L, H, hd = c["num_hidden_layers"], c["num_attention_heads"], c["head_dim"]
    gemm = 2.0 * T * layer_matrix_params(c) * L + 2.0 * c["hidden_size"] * c["vocab_size"]
    attn = 2.0 * H * hd * T * T * L          # QK^T and PV over the causal half
    return gemm + attn


def kv_bytes_per_token(c, itemsize=2) -> int:
    return 2 * c["num_key_value_heads"] * c["head_dim"] * itemsize * c["num_hidden_layers"]


# ------------------------------------------------------------------------------- ours ----

def decode_run(engine, batch: int, steps: int, warmup: int, seed: int, windows=None, prompt_len: int = PROMPT):
    """Prefill ``batch`` prompts of ``prompt_len`` tokens, then time ``steps`` decode steps on the device."""
    import numpy as np
    import torch

    from sleuth_b200.kernels import ops
    from sleuth_b200.sampling.config import SamplingConfig
    rng = np.random.default_rng(seed)
    V = engine.vocab
    prompts = [rng.integers(0, V, size=prompt_len).tolist() for _ in range(batch)]
    feed = rng.integers(0, V, size=(warmup + steps, batch))
    greedy = SamplingConfig(temperature=0.0)
    slots = engine.open(batch)
    try:
        logits = engine.prefill(slots, prompts)
        engine.sampler.choose(logits, greedy)
        for k in range(warmup):
            logits = engine.decode(slots, feed[k].tolist())
            engine.sampler.choose(logits, greedy)
        torch.cuda.synchronize()
        lib = ops.lib()
        own0, g0 = lib.launches, engine.stepper.graph_kernel_launches
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t_a = time.time()
        start.record()
        for k in range(warmup, warmup + steps):
            logits = engine.decode(slots, feed[k].tolist())
            engine.sampler.choose(logits, greedy)
        end.record()
        torch.cuda.synchronize()
        t_b = time.time()
        if windows is not None:
            windows.append((t_a, t_b))
        ms = start.elapsed_time(end) / steps
        launches = (lib.launches - own0) + (engine.stepper.graph_kernel_launches - g0)
        ctx_first = prompt_len + warmup + 1
        mean_ctx = ctx_first + (steps - 1) / 2.0
    finally:
        engine.close(slots)
    return ms, launches, mean_ctx


def prefill_run(engine, warmup: int, iters: int, seed: int, windows=None):
    import numpy as np
    import torch
    rng = np.random.default_rng(seed)
    prompt = rng.integers(0, CONFIG["vocab_size"], size=PROMPT).tolist()
    times = []
    for i in range(warmup + iters):
        slots = engine.open(1)
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t_a = time.time()
        a.record()
        engine.prefill(slots, [prompt])
        b.record()
        torch.cuda.synchronize()
        t_b = time.time()
        engine.close(slots)
        if i >= warmup:
            times.append(a.elapsed_time(b))
            if windows is not None:
                windows.append((t_a, t_b))
    return statistics.median(times)


def e2e_run(engine, batch: int, steps: int, seed: int, windows=None):
    """The same decode through ``Engine.generate``: host token lists in and out."""
    import numpy as np

    from sleuth_b200.sampling.config import SamplingConfig
    rng = np.random.default_rng(seed)
    prompts = [rng.integers(0, CONFIG["vocab_size"], size=PROMPT).tolist() for _ in range(batch)]
    import gc
    engine.generate(prompts, max_new_tokens=4, sampling=SamplingConfig(temperature=0.0), stop_ids=())   # warm-up
    # the timed region is some twenty milliseconds of host-driven steps: a collection of the interpreter's garbage
    # inside it would be a twentieth of it, so it runs before
    gc.collect()
    gc.disable()
    try:
        t_a = time.time()
        res = engine.generate(prompts, max_new_tokens=steps + 1, sampling=SamplingConfig(temperature=0.0), stop_ids=())
        t_b = time.time()
    finally:
        gc.enable()
    if windows is not None:
        windows.append((t_a, t_b))
    decoded = sum(len(r.new_ids) - 1 for r in res)
    seconds = max(r.decode_seconds for r in res)
    return decoded / seconds, engine.stepper.meta.last_upload_bytes, 4 * batch


CONFIG4 = dict(CONFIG, hidden_size=2560, num_hidden_layers=36, num_attention_heads=32, num_key_value_heads=8,
               intermediate_size=9728)                                    # BASELINE.json configs[3]: Qwen3-4B-shaped
CONFIG5 = dict(CONFIG, hidden_size=4096, num_hidden_layers=36, num_attention_heads=32, num_key_value_heads=8,
               intermediate_size=12288, tie_word_embeddings=False)        # configs[4]: Qwen3-8B-shaped, untied


def release(engine) -> None:
    """Give an engine's device memory back before the next, larger one is made."""
    import gc

    import torch
    engine.stepper._graphs.clear()
    del engine
    gc.collect()
    torch.cuda.empty_cache()


def config4_points(windows, new_tokens: int = 257) -> dict:
    """BASELINE.json configs[3]: 4B-shaped, a ragged batch of 16 prompts with seeded lengths in [64, 2048], then 256
    decode steps each, greedy and at temperature 0.8, through ``Engine.generate`` (host tokens in and out)."""
    import numpy as np

    from sleuth_b200.engine.engine import Engine
    from sleuth_b200.sampling.config import SamplingConfig
    rng = np.random.default_rng(16)
    lengths = rng.integers(64, 2049, size=16)
    prompts = [rng.integers(0, CONFIG4["vocab_size"], size=int(n)).tolist() for n in lengths]
    engine = Engine.from_config(CONFIG4, seed=4, dtype="bf16", max_seq_len=CONTEXT, max_tokens=16 * (2048 + 256 + 64))
    out = {}
    try:
        for key, sampling in (("cfg4_b16_greedy_e2e", SamplingConfig(temperature=0.0)),
                              ("cfg4_b16_t0.8_e2e", SamplingConfig(temperature=0.8))):
            engine.generate(prompts, max_new_tokens=4, sampling=sampling, stop_ids=(), seed=1)       # warm-up
            t_a = time.time()
            res = engine.generate(prompts, max_new_tokens=new_tokens, sampling=sampling, stop_ids=(), seed=1)
            windows.append((t_a, time.time()))
            out[key] = round(sum(len(r.new_ids) - 1 for r in res) / max(r.decode_seconds for r in res), 1)
        mean_ctx = float(lengths.mean()) + new_tokens / 2.0
        step_bytes = engine.model.weight_bytes() + 16 * mean_ctx * kv_bytes_per_token(CONFIG4)
        out["cfg4_hbm_frac"] = round(step_bytes * out["cfg4_b16_greedy_e2e"] / 16 / 1e9 / peaks()["hbm_gbs"], 4)
    finally:
        release(engine)
    return out


def config5_points(windows, steps: int, warmup: int, layers: int) -> dict:
    """BASELINE.json configs[4]: 8B-shaped, untied, batch 64, 4,096-token prompts, decode steps from there on."""
    from sleuth_b200.engine.engine import Engine
    cfg = dict(CONFIG5, num_hidden_layers=layers)
    engine = Engine.from_config(cfg, seed=5, dtype="bf16", max_seq_len=8192, max_tokens=64 * (4096 + 128))
    try:
        ms, _, mean_ctx = decode_run(engine, 64, steps, warmup, seed=5, windows=windows, prompt_len=4096)
        step_bytes = engine.model.weight_bytes() + 64 * mean_ctx * kv_bytes_per_token(cfg)
        return {"cfg5_b64": round(64 * 1000.0 / ms, 1), "cfg5_b64_ms": round(ms, 3),
                "cfg5_hbm_frac": round(step_bytes / (ms * 1e-3) / 1e9 / peaks()["hbm_gbs"], 4)}
    finally:
        release(engine)


def fp32_block(windows, steps: int, warmup: int, sm_mhz: float) -> dict:
    """The true 32-bit path at the benchmark's sizes: decode at batch 8 and one 2,048-token prompt. Its rooflines:
    the decode step reads every weight and the live cache once, both twice as wide as in bfloat16; the prompt's
    products run as plain fused multiply-adds, whose peak is 128 lanes x 2 flops x SMs x clock (no tensor-core mode
    is used on this path)."""
    import torch

    from sleuth_b200.engine.engine import Engine
    engine = Engine.from_config(CONFIG, seed=0, dtype="fp32", max_seq_len=CONTEXT, max_tokens=BATCH * CONTEXT)
    try:
        ms, _, mean_ctx = decode_run(engine, BATCH, steps, warmup, seed=1, windows=windows)
        pre_ms = prefill_run(engine, warmup=1, iters=3, seed=2, windows=windows)
        step_bytes = engine.model.weight_bytes() + BATCH * mean_ctx * kv_bytes_per_token(CONFIG, itemsize=4)
        sms = torch.cuda.get_device_properties(0).multi_processor_count
        ffma_tflops = sms * 128 * 2 * sm_mhz * 1e6 / 1e12
        pre_tflops = prefill_flops(CONFIG, PROMPT) / (pre_ms * 1e-3) / 1e12
        return {"decode_b8": round(BATCH * 1000.0 / ms, 1), "decode_ms": round(ms, 3),
                "decode_hbm_frac": round(step_bytes / (ms * 1e-3) / 1e9 / peaks()["hbm_gbs"], 4),
                "prefill_ms": round(pre_ms, 2), "prefill_tok_s": round(PROMPT / (pre_ms * 1e-3), 1),
                "ffma_peak_tflops": round(ffma_tflops, 1), "prefill_ffma_frac": round(pre_tflops / ffma_tflops, 4)}
    finally:
        release(engine)


def run_ours(args) -> dict:
    import torch

    from sleuth_b200.engine.engine import Engine
    pk = peaks()
    steps, warmup = args.steps, args.warmup
    if warmup + steps + 1 > CONTEXT - PROMPT:
        steps = CONTEXT - PROMPT - warmup - 1
    layers = args.layers or CONFIG["num_hidden_layers"]
    cfg = dict(CONFIG, num_hidden_layers=layers)
    engine = Engine.from_config(cfg, seed=0, dtype="bf16", max_seq_len=CONTEXT, max_tokens=64 * CONTEXT)
    clocks = ClockSampler()
    clocks.start()
    windows = []
    try:
        ms, launches, mean_ctx = decode_run(engine, BATCH, steps, warmup, seed=1, windows=windows)
        value = BATCH * 1000.0 / ms
        e2e, h2d, d2h = e2e_run(engine, BATCH, steps, seed=1, windows=windows)
        pre_ms = prefill_run(engine, warmup=5, iters=15, seed=2, windows=windows)
        ms1, _, _ = decode_run(engine, 1, steps, warmup, seed=3, windows=windows)
        ms64, _, _ = decode_run(engine, 64, steps, warmup, seed=4, windows=windows)
        e2e1, _, _ = e2e_run(engine, 1, min(steps, 128), seed=3, windows=windows)
        weight_bytes = engine.model.weight_bytes()
        release(engine)
        engine = None
        extra, fp32 = {}, None
        if not args.skip_other_configs:
            side = min(steps, 20)
            fp32 = fp32_block(windows, side, warmup, sm_mhz=peaks_clock())
            extra.update(config4_points(windows))
            extra.update(config5_points(windows, side, warmup, args.layers5 or CONFIG5["num_hidden_layers"]))
    finally:
        clocks.stop()
    step_bytes = weight_bytes + BATCH * mean_ctx * kv_bytes_per_token(cfg)
    achieved = step_bytes / (ms * 1e-3) / 1e9
    flops = prefill_flops(cfg, PROMPT)
    pre_tflops = flops / (pre_ms * 1e-3) / 1e12
    out = {
        "metric": "decode tok/s at batch 8 (Qwen3-0.6B shape, 2,048-token prompts, context to 4,096)",
        "value": round(value, 1), "unit": "tok/s", "n_gpus": 1, "steps": steps, "warmup": warmup,
        "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "baseline_note": BASELINE_NOTE,
        "dtype": "bf16", "data": "synthetic (seeded uniform token ids, random N(0,0.02) weights)", "impl": "ours",
        "config": {"model": "Qwen3-0.6B-shaped", "layers": layers, "layers_of_config": CONFIG["num_hidden_layers"],
                   "hidden": CONFIG["hidden_size"], "heads": CONFIG["num_attention_heads"],
                   "kv_heads": CONFIG["num_key_value_heads"], "head_dim": CONFIG["head_dim"],
                   "intermediate": CONFIG["intermediate_size"], "vocab": CONFIG["vocab_size"], "global_batch": BATCH,
                   "prompt_len": PROMPT, "seq_len": CONTEXT, "mean_context": round(mean_ctx, 1),
                   "parallelism": "single GPU", "l2": "inputs larger than L2 (weights 1.19 GB + cache per step)",
                   "peaks": pk["source"],
                   "cfg4": "4B-shaped: 36 layers, hidden 2560, 32/8 heads of 128, intermediate 9728; 16 prompts of 64..2048 tokens, 256 steps",
                   "cfg5": f"8B-shaped, untied: {args.layers5 or 36} of 36 layers, hidden 4096, 32/8 heads of 128, intermediate 12288; batch 64, 4096-token prompts",
                   "fp32": "the same 0.6B sizes and batch on the true 32-bit path"},
        "clocks": clocks.summary(windows),
        "e2e": {"value": round(e2e, 1), "unit": "tok/s", "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h)},
        "gpu_launches": int(launches),
        "prefill": {"value": round(PROMPT / (pre_ms * 1e-3), 1), "tokens": PROMPT, "ms": round(pre_ms, 3),
                    "frac": round(pre_tflops / pk["bf16_tflops"], 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
        "points": {"decode_b1": round(1000.0 / ms1, 1), "decode_b64": round(64 * 1000.0 / ms64, 1),
                   "decode_b1_e2e": round(e2e1, 1), **extra},
    }
    if fp32 is not None:
        out["fp32"] = fp32
    return out


BASELINE_NOTE = ("the reference publishes one figure for this model, 19 tok/s at batch 1, eager, on an RTX 5060 Ti: "
                 "other GPU, other batch, so no ratio is formed; compare with --impl reference on the same box")


def peaks_clock() -> float:
    """SM clock (MHz) for the FFMA peak: the measured maximum if the peaks file has it, else the nominal 1,965."""
    try:
        return float(json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))["sm_max_mhz"])
    except (OSError, KeyError, ValueError, TypeError):
        return 1965.0


def run_part(args) -> dict:
    """One part of the benchmark on its own, small enough to sit under a profiler."""
    from sleuth_b200.engine.engine import Engine
    layers = args.layers or CONFIG["num_hidden_layers"]
    cfg = dict(CONFIG, num_hidden_layers=layers)
    engine = Engine.from_config(cfg, seed=0, dtype="bf16", max_seq_len=CONTEXT, max_tokens=max(args.batch, 1) * CONTEXT)
    if args.only == "decode":
        ms, launches, mean_ctx = decode_run(engine, args.batch, args.steps, args.warmup, seed=1)
        return {"part": "decode", "batch": args.batch, "layers": layers, "ms_per_step": round(ms, 4),
                "tok_per_s": round(args.batch * 1000.0 / ms, 1), "mean_context": mean_ctx, "own_launches": launches}
    ms = prefill_run(engine, warmup=args.warmup, iters=max(1, args.steps), seed=2)
    return {"part": "prefill", "layers": layers, "tokens": PROMPT, "ms": round(ms, 3),
            "tflops": round(prefill_flops(cfg, PROMPT) / (ms * 1e-3) / 1e12, 1)}


# -------------------------------------------------------------------------- reference ----

def run_reference(args) -> dict:
    ref = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref, "sleuth")):
        return {"impl": "reference", "unavailable": "baseline/_ref holds no install of the reference (pip --target failed or was not run)"}
    sys.path.insert(0, ref)
    try:
        import numpy as np
        import torch
        from sleuth.forge.infer.kv_cache import KVCache
        from sleuth.forge.infer.sampling import SamplingConfig, sample_next
        from sleuth.forge.model.config import ModelConfig
        from sleuth.forge.model.transformer import Transformer
    except Exception as e:  # noqa: BLE001
        return {"impl": "reference", "unavailable": f"the reference does not import here: {type(e).__name__}: {e}"[:300]}
    c = CONFIG
    steps, warmup = args.steps, args.warmup
    if warmup + steps + 1 > CONTEXT - PROMPT:
        steps = CONTEXT - PROMPT - warmup - 1
    torch.manual_seed(0)
    mc = ModelConfig(vocab_size=c["vocab_size"], d_model=c["hidden_size"], n_layers=c["num_hidden_layers"],
                     n_heads=c["num_attention_heads"], head_size=c["head_dim"], n_kv_heads=c["num_key_value_heads"],
                     ffn_type="swiglu", ffn_hidden=c["intermediate_size"], norm_eps=c["rms_norm_eps"],
                     rope_theta=c["rope_theta"], max_seq_len=CONTEXT, qk_norm=True, tie_embeddings=True, pad_vocab_to=1)
    model = Transformer(mc).to(device="cuda", dtype=torch.bfloat16).eval()
    rng = np.random.default_rng(1)
    prompts = torch.tensor(rng.integers(0, c["vocab_size"], size=(BATCH, PROMPT)), device="cuda")
    feed = rng.integers(0, c["vocab_size"], size=(warmup + steps, BATCH))
    greedy = SamplingConfig(temperature=0.0)
    clocks = ClockSampler()
    clocks.start()
    windows = []
    try:
        with torch.no_grad():
            def decode(e2e: bool, timed_steps: int):
                cache = KVCache.for_model(model, batch=BATCH, max_len=CONTEXT, dtype=torch.bfloat16)
                logits = model(prompts, cache=cache).logits[:, -1]
                nxt = sample_next(logits, greedy)
                for k in range(warmup):
                    logits = model(torch.tensor(feed[k], device="cuda").view(BATCH, 1), cache=cache).logits[:, -1]
                    nxt = sample_next(logits, greedy)
                torch.cuda.synchronize()
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                t_a = time.time()
                a.record()
                host = feed[warmup].tolist()
                for k in range(warmup, warmup + timed_steps):
                    ids = torch.tensor(host if e2e else feed[k].tolist(), device="cuda").view(BATCH, 1)
                    logits = model(ids, cache=cache).logits[:, -1]
                    nxt = sample_next(logits, greedy)
                    if e2e:
                        host = nxt.tolist()
                b.record()
                torch.cuda.synchronize()
                t_b = time.time()
                windows.append((t_a, t_b))
                return (a.elapsed_time(b) / timed_steps) if not e2e else (t_b - t_a) * 1000.0 / timed_steps

            # The reference's own method (sleuth/forge/experiment.py:87-121): a warm-up run first, then the best of
            # three. The first pass through this loop pays one-time costs (library handles, kernel selection,
            # allocator growth) that a 20-step window does not amortise; it is run once untimed.
            decode(False, min(steps, 8))
            ms = min(decode(False, steps) for _ in range(3))
            ms_e2e = min(decode(True, steps) for _ in range(3))
            one = prompts[:1]
            times = []
            for i in range(6):
                cache = KVCache.for_model(model, batch=1, max_len=CONTEXT, dtype=torch.bfloat16)
                torch.cuda.synchronize()
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
                model(one, cache=cache).logits[:, -1]
                b.record()
                torch.cuda.synchronize()
                if i:
                    times.append(a.elapsed_time(b))
            pre_ms = statistics.median(times)
        # Batch 1 through the reference's public entry point at its best: generate(..., cuda_graph=True), which
        # replays one recorded graph per token (sleuth/forge/infer/generate.py:49-136, cuda_graph.py:52-144), and
        # eagerly for comparison; greedy, 128 new tokens, warm-up then best of three, as its decode_speed does.
        from sleuth.forge.infer.generate import generate as ref_generate
        prompt1 = prompts[0].tolist()
        b1 = {}
        for key, graph in (("decode_b1_graph", True), ("decode_b1_eager", False)):
            try:
                t_a = time.time()
                runs = [ref_generate(model, prompt1, 129, greedy, cuda_graph=graph) for _ in range(4)][1:]
                windows.append((t_a, time.time()))
                b1[key] = round(max(r.decode_tok_per_s for r in runs), 1)
            except Exception as e:  # noqa: BLE001
                b1[key] = None
                b1[key + "_error"] = f"{type(e).__name__}: {e}"[:200]
    finally:
        clocks.stop()
    pk = peaks()
    value = BATCH * 1000.0 / ms
    return {
        "metric": "decode tok/s at batch 8 (Qwen3-0.6B shape, 2,048-token prompts, context to 4,096)",
        "value": round(value, 1), "unit": "tok/s", "n_gpus": 1, "steps": steps, "warmup": warmup,
        "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "baseline_note": BASELINE_NOTE,
        "dtype": "bf16", "data": "synthetic (seeded uniform token ids, reference's own random init)",
        "impl": "reference",
        "config": {"model": "Qwen3-0.6B-shaped", "layers": c["num_hidden_layers"], "global_batch": BATCH,
                   "prompt_len": PROMPT, "seq_len": CONTEXT, "parallelism": "single GPU",
                   "path": "Transformer.forward + KVCache + sample_next, eager (its generate() is batch 1 only)",
                   "method": "one untimed pass, then best of 3 (its own decode_speed: warm-up, best of 3)",
                   "points": "batch 1: its generate(), greedy, 128 tokens, with and without its CUDA-graph decoder"},
        "clocks": clocks.summary(windows),
        "e2e": {"value": round(BATCH * 1000.0 / ms_e2e, 1), "unit": "tok/s", "h2d_bytes_per_step": 8 * BATCH,
                "d2h_bytes_per_step": 8 * BATCH},
        "gpu_launches": 0,
        "prefill": {"value": round(PROMPT / (pre_ms * 1e-3), 1), "tokens": PROMPT, "ms": round(pre_ms, 3),
                    "frac": round(prefill_flops(c, PROMPT) / (pre_ms * 1e-3) / 1e12 / pk["bf16_tflops"], 4)},
        "points": b1,
    }


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2040)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--layers", type=int, default=0, help="fewer layers than the configuration (0 = all)")
    ap.add_argument("--only", choices=["all", "decode", "prefill"], default="all",
                    help="run one part only, for profiling (prints that part's numbers, not the full record)")
    ap.add_argument("--batch", type=int, default=BATCH, help="batch of --only decode")
    ap.add_argument("--print-config", action="store_true", help="print the benchmark model's config.json and exit")
    ap.add_argument("--skip-other-configs", action="store_true",
                    help="leave out the 32-bit block and the 4B- and 8B-shaped points (a quicker run)")
    ap.add_argument("--layers5", type=int, default=0, help="layers of the 8B-shaped point (0 = all 36)")
    args = ap.parse_args()
    if args.print_config:
        print(json.dumps(CONFIG))
        return 0
    if args.gpus != 1:
        print(f"bench.py measures one GPU only: this library runs on a single GPU, --gpus {args.gpus} is not supported")
        return 2
    if args.warmup < 3:
        args.warmup = 3
    if args.only != "all" and args.impl == "ours":
        out = run_part(args)
    else:
        out = run_reference(args) if args.impl == "reference" else run_ours(args)
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
