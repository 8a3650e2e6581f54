"""Shared pytest set-up: the ``gpu`` marker, import paths, golden-fixture access."""
from __future__ import annotations

import os
import sys

import numpy as np
import pytest
import torch

os.environ.setdefault("RACE_B200_CHECK_STATUS", "1")
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN_PATH = os.path.join(ROOT, "tests", "golden", "race_golden.npz")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def golden():
    return np.load(GOLDEN_PATH)


def draw_kvq(M, B, T, H, dk, dtype, seed=0):
    """Inputs drawn the way the reference's tests draw them (src/test_equivalence.py:21-24):
    one generator seeded 0, order K, V, Q."""
    g = torch.Generator().manual_seed(seed)
    return [torch.randn((M, B, T, H, dk), generator=g, dtype=dtype) for _ in range(3)]
