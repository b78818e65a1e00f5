"""The plain implementation itself: against the reference's committed outputs, and its own properties."""

import os

import numpy as np
import pytest
import torch

import tiny
from plain import qwen3_plain as plain

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_plain_matches_the_reference_model(name, model_folders):
    g = np.load(os.path.join(GOLDEN, f"{name}.npz"))
    cfg, w = plain.read_model(model_folders[name])
    mine = plain.logits(cfg, w, g["prompt"].tolist())[g["rows"].tolist()]
    np.testing.assert_allclose(mine.numpy(), g["logits"], rtol=1e-4, atol=3e-6)


def test_float64_and_float32_agree(model_folders):
    cfg, w = plain.read_model(model_folders["B"])
    ids = list(range(3, 40))
    a, b = plain.logits(cfg, w, ids), plain.logits(cfg, w, ids, work=torch.float64)
    assert (a.double() - b).abs().max() < 5e-6


def test_causality(model_folders):
    cfg, w = plain.read_model(model_folders["A"])
    ids = [3, 9, 200, 17, 4, 4, 90, 1]
    a = plain.logits(cfg, w, ids)
    ids[5] = 77
    b = plain.logits(cfg, w, ids)
    assert torch.equal(a[:5], b[:5]) and not torch.allclose(a[5:], b[5:])


def test_window_hides_old_keys(model_folders):
    cfg, w = plain.read_model(model_folders["C"])
    ids = list(np.random.default_rng(0).integers(0, 311, size=90))
    a = plain.logits(cfg, w, ids)
    changed = list(ids)
    changed[3] = (ids[3] + 1) % 311
    b = plain.logits(cfg, w, changed)
    # layers 1 and 3 slide over 40 keys, layers 0 and 2 see everything: the change still reaches the end
    assert not torch.allclose(a[-1], b[-1])
    every = dict(cfg, layer_types=["sliding_attention"] * 4)
    a2, b2 = plain.logits(every, w, ids), plain.logits(every, w, changed)
    assert not torch.allclose(a2[20], b2[20])
    # with every layer sliding, information moves at most 4 * 39 positions: far enough away nothing changes
    long_ids = ids + ids
    long_changed = list(long_ids)
    long_changed[3] = changed[3]
    a3, b3 = plain.logits(every, w, long_ids), plain.logits(every, w, long_changed)
    assert torch.equal(a3[3 + 4 * 39 + 1:], b3[3 + 4 * 39 + 1:]) and not torch.equal(a3[3 + 39], b3[3 + 39])


def test_mask_matches_the_reference_rule():
    m = plain.causal_mask(6, 3)
    assert m[5].tolist() == [False, False, False, True, True, True] and m[1].tolist() == [True, True] + [False] * 4
    assert plain.causal_mask(4, 0).tolist() == torch.tril(torch.ones(4, 4, dtype=torch.bool)).tolist()


def test_greedy_keeps_the_stop_token(model_folders):
    cfg, w = plain.read_model(model_folders["A"])
    free = plain.greedy_generate(cfg, w, [5, 6, 7], 5)
    stopped = plain.greedy_generate(cfg, w, [5, 6, 7], 5, stop_ids={free[1]})
    assert stopped == free[:free.index(free[1]) + 1]
