"""The command line: option parsing and refusals on the CPU, and on a GPU the whole flow of
``python -m sleuth_b200 random-model`` and ``python -m sleuth_b200 generate`` as a user runs it (a subprocess),
compared with the plain implementation's greedy tokens. The flow is the reference's ``generate`` command
(sleuth/cli.py:174-256: load, warm-up, generate, one line of tokens per result on stdout, a bracketed
summary line on stderr; options sleuth/cli.py:769-806)."""

from __future__ import annotations

import json
import os
import subprocess
import sys

import pytest

import tiny
from plain import qwen3_plain as plain

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_prompt_ids_are_parsed_as_a_batch():
    from sleuth_b200.cli import _parse_ids
    assert _parse_ids("1 2 3") == [[1, 2, 3]]
    assert _parse_ids("1,2,3; 7,8") == [[1, 2, 3], [7, 8]]
    assert _parse_ids(" 4 ,5;;6 ; ") == [[4, 5], [6]]
    assert _parse_ids("") == []
    with pytest.raises(ValueError):
        _parse_ids("1 two 3")


def test_generate_options_carry_the_reference_defaults():
    from sleuth_b200.cli import build_parser
    a = build_parser().parse_args(["generate", "some/folder"])
    # sleuth/cli.py:769-806: temperature 0.8, top-k off, top-p off, min-p 0.05 on the command line, 200 new tokens,
    # penalty off over the last 64 tokens, no n-gram ban, one sample, random seed, dtype and device automatic
    assert (a.temperature, a.top_k, a.top_p, a.min_p) == (0.8, 0, 1.0, 0.05)
    assert (a.max_new_tokens, a.repetition_penalty, a.repeat_last_n, a.no_repeat_ngram) == (200, 1.0, 64, 0)
    assert (a.samples, a.seed, a.dtype, a.device, a.prompt, a.prompt_ids) == (1, None, "auto", "auto", "", "")
    assert a.cuda_graph is True and a.stop_id is None and a.max_seq_len == 4096
    b = build_parser().parse_args(["generate", "m", "--no-cuda-graph", "--stop-id", "3", "--stop-id", "9", "--dtype", "fp32",
                                   "--temperature", "0", "--seed", "4", "--samples", "2"])
    assert b.cuda_graph is False and b.stop_id == [3, 9] and b.dtype == "fp32" and b.temperature == 0.0 and b.seed == 4
    with pytest.raises(SystemExit):
        build_parser().parse_args(["generate", "m", "--dtype", "fp16"])       # float16 is no run dtype here
    with pytest.raises(SystemExit):
        build_parser().parse_args(["generate"])                               # the model folder is required


def test_generate_without_a_prompt_explains_and_returns_2(capsys):
    from sleuth_b200.cli import main
    assert main(["generate", "no/such/folder"]) == 2                         # refused before anything is loaded
    err = capsys.readouterr().err
    assert "--prompt-ids" in err and "--tokenizer" in err
    assert main(["generate", "no/such/folder", "--prompt", "text without a tokenizer"]) == 2


def test_random_model_writes_a_folder_that_reads_back(tmp_path):
    from sleuth_b200.cli import main
    cfg = tmp_path / "config.json"
    cfg.write_text(json.dumps(tiny.A))
    assert main(["random-model", str(cfg), str(tmp_path / "m"), "--seed", "5", "--dtype", "fp32"]) == 0
    got_cfg, w = plain.read_model(tmp_path / "m")
    assert got_cfg["hidden_size"] == tiny.A["hidden_size"] and "model.embed_tokens.weight" in w
    assert "lm_head.weight" not in w                                          # tied


@pytest.mark.gpu
def test_generate_command_end_to_end(tmp_path):
    env = dict(os.environ, PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""))
    cfg_path = tmp_path / "config.json"
    cfg_path.write_text(json.dumps(tiny.B))
    folder = tmp_path / "model"
    r = subprocess.run([sys.executable, "-m", "sleuth_b200", "random-model", str(cfg_path), str(folder), "--seed", "8",
                        "--dtype", "fp32"], env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr
    assert r.stdout.strip() == str(folder)
    cfg, w = plain.read_model(folder)
    prompts = [[5, 17, 3, 250, 9], [400, 2], [77]]
    text = "; ".join(",".join(map(str, p)) for p in prompts)
    r = subprocess.run([sys.executable, "-m", "sleuth_b200", "generate", str(folder), "--prompt-ids", text, "--temperature", "0",
                        "--max-new-tokens", "8", "--dtype", "fp32", "--max-seq-len", "128"],
                       env=env, capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stderr
    lines = [ln for ln in r.stdout.splitlines() if ln.strip()]
    assert [[int(t) for t in ln.split()] for ln in lines] == [plain.greedy_generate(cfg, w, p, 8) for p in prompts]
    summaries = [ln for ln in r.stderr.splitlines() if ln.startswith("[8 tokens, stop: max_new_tokens, prompt ")]
    assert len(summaries) == 3 and all("tok/s" in ln and "peak GPU memory" in ln for ln in summaries)
    assert any("float32" in ln and "params" in ln and "cuda:0" in ln for ln in r.stderr.splitlines())     # the header line
    # a stop token ends a request early and is kept; two samples are separated by a rule
    stop = plain.greedy_generate(cfg, w, prompts[0], 8)[2]
    r = subprocess.run([sys.executable, "-m", "sleuth_b200", "generate", str(folder), "--prompt-ids", "5 17 3 250 9",
                        "--temperature", "0", "--max-new-tokens", "8", "--dtype", "fp32", "--stop-id", str(stop), "--samples", "2",
                        "--max-seq-len", "128", "--no-cuda-graph"], env=env, capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stderr
    out = [ln for ln in r.stdout.splitlines() if ln.strip()]
    want = plain.greedy_generate(cfg, w, prompts[0], 8, stop_ids={stop})
    assert out[0].split() == [str(t) for t in want] and out[1] == "-" * 40 and out[2] == out[0]
    assert "stop: stop_token" in r.stderr
