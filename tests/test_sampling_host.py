"""Host-side sampling state and the plain sampling pipeline on hand-made rows."""

import torch

from plain import qwen3_plain as plain
from sleuth_b200.sampling import NgramBlocker, SamplingConfig, recent_window, uniform
import pytest


def test_uniform_is_a_function_of_its_arguments():
    a = [uniform(1, r, s) for r in range(4) for s in range(50)]
    assert a == [uniform(1, r, s) for r in range(4) for s in range(50)]
    assert len(set(a)) == len(a) and all(0.0 <= u < 1.0 for u in a)
    assert abs(sum(a) / len(a) - 0.5) < 0.08
    assert uniform(2, 0, 0) != uniform(1, 0, 0)


def test_ngram_blocker():
    b = NgramBlocker(3, [5, 6, 7, 5, 6])
    assert b.banned() == [7]
    b.add(9)
    assert b.banned() == []
    b.add(5)
    b.add(6)
    assert b.banned() == [7, 9]
    assert NgramBlocker(0, [1, 2]).banned() == []
    one = NgramBlocker(1, [4, 4, 8])
    assert one.banned() == [4, 8]


def test_recent_window():
    assert recent_window([1, 2, 3, 2, 9], 3) == [2, 3, 9] and recent_window([1, 2, 3, 2, 9], 0) == [1, 2, 3, 9]


def test_sampling_config_refuses_nonsense():
    for bad in (dict(top_p=0.0), dict(top_k=-1), dict(min_p=1.5), dict(repetition_penalty=0.0)):
        with pytest.raises(ValueError):
            SamplingConfig(**bad)
    assert SamplingConfig(temperature=0.0).greedy and SamplingConfig().temperature == 0.8


def test_plain_pipeline_on_small_rows():
    lo = torch.finfo(torch.float32).min
    row = torch.tensor([2.0, 1.0, 0.5, -1.0])
    assert plain.final_logits(row, 0.0).tolist() == row.tolist()
    assert plain.final_logits(row, 1.0, top_k=2).tolist() == [2.0, 1.0, lo, lo]
    p = torch.softmax(row, 0)
    kept = plain.final_logits(row, 1.0, top_p=float(p[0]) + 1e-3)
    assert kept.tolist() == [2.0, 1.0, lo, lo]              # the mass before token 1 is below p, before token 2 above
    assert plain.final_logits(row, 1.0, top_p=1e-6).tolist() == [2.0, lo, lo, lo]      # the best always stays
    assert plain.final_logits(row, 1.0, min_p=0.3).tolist() == [2.0, 1.0, lo, lo]      # e^-1 = .37 stays, e^-1.5 = .22 goes
    pen = plain.final_logits(row, 0.0, repetition_penalty=2.0, recent=[0, 3, 3])
    assert pen.tolist() == [1.0, 1.0, 0.5, -2.0]
    assert plain.final_logits(row, 0.0, banned=[0, 1]).argmax() == 2
    assert plain.final_logits(row, 0.0, banned=[0, 1, 2, 3]).tolist() == row.tolist()   # a ban on everything is ignored
    assert plain.final_logits(row, 0.5).tolist() == [4.0, 2.0, 1.0, -2.0]
    assert plain.draw(torch.tensor([0.0, 0.0]), 0.49) == 0 and plain.draw(torch.tensor([0.0, 0.0]), 0.51) == 1
