#!/usr/bin/env python3
"""Makes tests/golden/*.npz: logits of tbertha35/Sleuth's own model code on the tiny random models.

Run once on a machine where the reference can be imported (CPU is enough):

    PYTHONPATH=<path to tbertha35/Sleuth> python tests/golden/make_golden.py

For each tiny configuration it writes the seeded random model folder with this repository's writer,
loads it into the reference's ``Transformer`` in float32 and stores the logits of one seeded prompt.
Configurations A and B go through the reference's own folder loader
(sleuth/formats/hf.py:268-306). Configuration C has sliding-window layers, which that loader does
not map from config.json (hf.py:95-98 only shortens the context), so its model is built from the
reference's ``ModelConfig(layer_types=..., sliding_window=...)`` and filled through the loader's name
map (hf.py:131-145). tests/test_plain.py compares the plain implementation with these files.
"""

import json
import os
import sys
import tempfile

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "..", ".."))
sys.path.insert(0, os.path.join(HERE, ".."))

import tiny  # noqa: E402
from sleuth_b200.weights.random_init import write_random_model  # noqa: E402
from sleuth_b200.weights.safetensors import read_safetensors  # noqa: E402

from sleuth.forge.model.config import ModelConfig  # noqa: E402
from sleuth.forge.model.transformer import Transformer  # noqa: E402
from sleuth.formats.hf import load_hf_model, our_name  # noqa: E402

PROMPT_LEN = {"A": 17, "B": 40, "C": 100, "D": 70}


def prompt(name):
    rng = np.random.default_rng(tiny.SEEDS[name])
    return rng.integers(0, tiny.CONFIGS[name]["vocab_size"], size=PROMPT_LEN[name]).tolist()


def reference_model(name, folder):
    cfg = tiny.CONFIGS[name]
    if "layer_types" not in cfg:
        model, info = load_hf_model(folder, dtype=torch.float32, max_seq_len=cfg["max_position_embeddings"])
        assert info["n_unused"] == 0
        return model
    mc = ModelConfig(vocab_size=cfg["vocab_size"], d_model=cfg["hidden_size"], n_layers=cfg["num_hidden_layers"],
                     n_heads=cfg["num_attention_heads"], n_kv_heads=cfg["num_key_value_heads"], head_size=cfg["head_dim"],
                     ffn_type="swiglu", ffn_hidden=cfg["intermediate_size"], norm_eps=cfg["rms_norm_eps"],
                     rope_theta=cfg["rope_theta"], max_seq_len=cfg["max_position_embeddings"], qk_norm=True,
                     tie_embeddings=cfg["tie_word_embeddings"], qkv_bias=cfg["attention_bias"], pad_vocab_to=1,
                     layer_types=["sliding" if t == "sliding_attention" else "full" for t in cfg["layer_types"]],
                     sliding_window=cfg["sliding_window"])
    model = Transformer(mc).eval()
    params = dict(model.named_parameters())
    with torch.no_grad():
        for k, t in read_safetensors(os.path.join(folder, "model.safetensors")).items():
            params[our_name(k)].copy_(t)
    return model


def main():
    for name in tiny.CONFIGS:
        with tempfile.TemporaryDirectory() as d:
            write_random_model(d, tiny.CONFIGS[name], seed=tiny.SEEDS[name], dtype=torch.float32)
            model = reference_model(name, d)
            ids = prompt(name)
            with torch.no_grad():
                logits = model(torch.tensor([ids])).logits[0].float().numpy()
        keep = logits if name in ("A",) else logits[-12:]
        np.savez_compressed(os.path.join(HERE, f"{name}.npz"), prompt=np.asarray(ids, dtype=np.int32),
                            rows=np.arange(len(ids))[-len(keep):].astype(np.int32), logits=keep.astype(np.float32))
        print(name, logits.shape, "->", keep.shape, float(np.abs(logits).max()))


if __name__ == "__main__":
    main()
