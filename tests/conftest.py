"""Shared test set-up: the ``gpu`` marker, import paths, the tiny configurations and model folders."""

from __future__ import annotations

import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.dirname(os.path.abspath(__file__))):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs an NVIDIA GPU (run with -m gpu on a B200)")


def pytest_collection_modifyitems(config, items):
    import torch
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device here")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def model_folders(tmp_path_factory):
    """Model folders of the tiny configurations, float32 weights, made once per session."""
    import torch

    import tiny
    from sleuth_b200.weights.random_init import write_random_model
    out = {}
    for name, cfg in tiny.CONFIGS.items():
        d = tmp_path_factory.mktemp(f"model_{name}")
        write_random_model(d, cfg, seed=tiny.SEEDS[name], dtype=torch.float32)
        out[name] = str(d)
    return out


def pytest_terminal_summary(terminalreporter):
    """The largest differences from the plain implementation that the GPU tests saw (tests/closeness.py)."""
    import closeness
    closeness.report(terminalreporter.write_line)
