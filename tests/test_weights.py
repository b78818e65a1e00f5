"""Weights: safetensors reading and writing, refusal of corrupt files, by-name loading errors, random folders."""

import json
import struct

import pytest
import torch

import tiny
from sleuth_b200.config import parse_config
from sleuth_b200.engine.model import declare_model
from sleuth_b200.weights import (Checkpoint, SafetensorsError, SafetensorsFile, WeightError, check, read_safetensors,
                                 write_random_model, write_safetensors)


def test_round_trip_dtypes_and_layout(tmp_path):
    t = {"a": torch.randn(3, 5), "b": torch.randn(4).to(torch.bfloat16), "c": torch.arange(6, dtype=torch.int32).view(2, 3),
         "e": torch.empty(0, 7), "s": torch.tensor(2.5), "nc": torch.randn(4, 6).t()}
    p = tmp_path / "x.safetensors"
    write_safetensors(t, p, metadata={"k": "v"})
    back = read_safetensors(p)
    assert list(back) == list(t)
    for k in t:
        assert back[k].dtype == t[k].dtype and torch.equal(back[k], t[k].contiguous())
    raw = p.read_bytes()
    (n,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + n])
    assert n % 8 == 0 and header["__metadata__"] == {"k": "v"} and header["a"]["data_offsets"] == [0, 60]
    assert header["b"]["dtype"] == "BF16" and header["b"]["data_offsets"] == [60, 68]
    with SafetensorsFile(p) as f:
        assert f.metadata == {"k": "v"} and f.describe("c") == (torch.int32, (2, 3))


def test_hand_written_file(tmp_path):
    header = json.dumps({"w": {"dtype": "F32", "shape": [2], "data_offsets": [0, 8]}}).encode()
    p = tmp_path / "h.safetensors"
    p.write_bytes(struct.pack("<Q", len(header)) + header + struct.pack("<ff", 1.5, -2.0))
    assert read_safetensors(p)["w"].tolist() == [1.5, -2.0]


@pytest.mark.parametrize("damage", ["short", "header_len", "not_json", "dtype", "offsets", "overlap", "truncated"])
def test_corrupt_files_are_refused(tmp_path, damage):
    def make(header: dict, data: bytes, n=None):
        h = json.dumps(header).encode()
        return struct.pack("<Q", len(h) if n is None else n) + h + data

    good = {"w": {"dtype": "F32", "shape": [2], "data_offsets": [0, 8]}}
    blob = {
        "short": b"abc",
        "header_len": make(good, b"\0" * 8, n=10 ** 9),
        "not_json": struct.pack("<Q", 4) + b"{{{{" + b"\0" * 8,
        "dtype": make({"w": {"dtype": "Q4", "shape": [2], "data_offsets": [0, 8]}}, b"\0" * 8),
        "offsets": make({"w": {"dtype": "F32", "shape": [3], "data_offsets": [0, 8]}}, b"\0" * 8),
        "overlap": make({"w": {"dtype": "F32", "shape": [2], "data_offsets": [0, 8]},
                         "v": {"dtype": "F32", "shape": [2], "data_offsets": [4, 12]}}, b"\0" * 12),
        "truncated": make(good, b"\0" * 4),
    }[damage]
    p = tmp_path / "bad.safetensors"
    p.write_bytes(blob)
    with pytest.raises(SafetensorsError):
        SafetensorsFile(p)


def test_random_folder_is_reproducible_and_loads_by_name(tmp_path):
    a = write_random_model(tmp_path / "a", tiny.B, seed=5, dtype=torch.float32)
    b = write_random_model(tmp_path / "b", tiny.B, seed=5, dtype=torch.float32)
    c = write_random_model(tmp_path / "c", tiny.B, seed=6, dtype=torch.bfloat16)
    ta, tb, tc = (read_safetensors(d / "model.safetensors") for d in (a, b, c))
    assert all(torch.equal(ta[k], tb[k]) for k in ta) and not torch.equal(ta["lm_head.weight"], tc["lm_head.weight"].float())
    assert tc["lm_head.weight"].dtype == torch.bfloat16
    assert json.loads((a / "config.json").read_text())["num_key_value_heads"] == 3
    arch, cfg, _ = parse_config(json.loads((a / "config.json").read_text()))
    expected = declare_model(arch.model_spec(cfg))
    assert set(expected) == set(ta)
    gain = ta["model.layers.0.self_attn.q_norm.weight"]
    assert abs(float(gain.mean()) - 1.0) < 0.05 and float(gain.std()) > 0.005       # gains are 1 + noise
    assert "model.layers.0.self_attn.q_proj.bias" in ta and ta["model.layers.1.mlp.down_proj.weight"].shape == (96, 160)
    with Checkpoint(a) as ck:
        check(expected, ck)


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    d = write_random_model(tmp_path / "m", tiny.A, seed=1, dtype=torch.float32)
    t = read_safetensors(d / "model.safetensors")
    del t["model.layers.1.mlp.up_proj.weight"]
    del t["model.norm.weight"]
    t["model.layers.0.self_attn.q_proj.bias"] = torch.zeros(64)          # attention_bias is false
    t["model.layers.0.self_attn.k_proj.weight"] = torch.zeros(32, 60)
    t["rubbish"] = torch.zeros(1)
    t["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(8)   # ignored, as in the reference
    write_safetensors(t, d / "model.safetensors")
    arch, cfg, _ = parse_config(tiny.A)
    spec = arch.model_spec(cfg)
    with Checkpoint(d) as ck, pytest.raises(WeightError) as e:
        check(declare_model(spec), ck, spec.ignored_tensors)
    err = e.value
    assert err.missing == ["model.layers.1.mlp.up_proj.weight", "model.norm.weight"]
    assert err.unexpected == ["model.layers.0.self_attn.q_proj.bias", "rubbish"]
    assert err.wrong_shape == [("model.layers.0.self_attn.k_proj.weight", (32, 60), (32, 64))]
    msg = str(err)
    for word in ("missing (2)", "unexpected (2)", "rubbish", "wrong shape", "[32, 60]", "[32, 64]"):
        assert word in msg


def test_tied_model_ignores_a_stored_lm_head_and_untied_needs_it(tmp_path):
    d = write_random_model(tmp_path / "m", tiny.A, seed=1, dtype=torch.float32)
    t = read_safetensors(d / "model.safetensors")
    t["lm_head.weight"] = t["model.embed_tokens.weight"].clone()
    write_safetensors(t, d / "model.safetensors")
    arch, cfg, _ = parse_config(tiny.A)
    with Checkpoint(d) as ck:
        spec = arch.model_spec(cfg, tensor_names=set(ck.names()))
        check(declare_model(spec), ck, spec.ignored_tensors)
    arch, cfg, _ = parse_config(dict(tiny.A, tie_word_embeddings=False))
    with Checkpoint(d) as ck:
        spec = arch.model_spec(cfg, tensor_names=set(ck.names()))
        assert not spec.head.tied
        check(declare_model(spec), ck, spec.ignored_tensors)


def test_integer_weight_where_a_float_is_needed(tmp_path):
    d = write_random_model(tmp_path / "m", tiny.A, seed=1, dtype=torch.float32)
    t = read_safetensors(d / "model.safetensors")
    t["model.norm.weight"] = torch.ones(64, dtype=torch.int32)
    write_safetensors(t, d / "model.safetensors")
    arch, cfg, _ = parse_config(tiny.A)
    with Checkpoint(d) as ck, pytest.raises(WeightError, match="wrong dtype: model.norm.weight"):
        check(declare_model(arch.model_spec(cfg)), ck)


def test_sharded_checkpoint(tmp_path):
    d = write_random_model(tmp_path / "m", tiny.A, seed=1, dtype=torch.float32)
    t = read_safetensors(d / "model.safetensors")
    names = list(t)
    (d / "model.safetensors").unlink()
    half = len(names) // 2
    write_safetensors({k: t[k] for k in names[:half]}, d / "model-00001-of-00002.safetensors")
    write_safetensors({k: t[k] for k in names[half:]}, d / "model-00002-of-00002.safetensors")
    wm = {k: "model-00001-of-00002.safetensors" for k in names[:half]}
    wm.update({k: "model-00002-of-00002.safetensors" for k in names[half:]})
    (d / "model.safetensors.index.json").write_text(json.dumps({"metadata": {}, "weight_map": wm}))
    with Checkpoint(d) as ck:
        assert set(ck.names()) == set(names) and torch.equal(ck.tensor(names[-1]), t[names[-1]])
