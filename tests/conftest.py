"""Shared test configuration: markers, repo-root import path, golden loader."""
from __future__ import annotations

import os
import sys

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (sm_100a)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


def load_golden(name: str) -> dict:
    with np.load(os.path.join(GOLDEN, name)) as data:
        return {k: torch.from_numpy(np.asarray(data[k])) for k in data.files}


def rel_l2(actual: torch.Tensor, expected: torch.Tensor) -> float:
    a, e = actual.detach().double().cpu(), expected.detach().double().cpu()
    return float((a - e).norm() / e.norm().clamp_min(1e-12))
