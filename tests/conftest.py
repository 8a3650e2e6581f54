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


GLOBAL_CASES = ["g_k4l4", "g_k2l2", "g_k6l8_d128", "g_k3l2_d32", "g_k4l4_t700"]


@pytest.fixture(scope="session")
def golden_global():
    """Global-normalisation vectors written by tests/golden/make_golden_global.py from the reference's
    race_causal_reference."""
    return np.load(os.path.join(ROOT, "tests", "golden", "race_global_golden.npz"))


def global_case(golden_global, name):
    """(pQ [N,T,L,R], pK, V [N,T,d], out [N,T,d]) of one stored case, streams flattened."""
    B, H, T, d, L, R = (int(x) for x in golden_global[f"{name}/cfg"])
    t = {k: torch.from_numpy(golden_global[f"{name}/{k}"]) for k in ("phi_q", "phi_k", "v", "out")}
    return (t["phi_q"].reshape(B * H, T, L, R), t["phi_k"].reshape(B * H, T, L, R),
            t["v"].reshape(B * H, T, d), t["out"].reshape(B * H, T, d))


def draw_kvq(M, B, T, H, dk, dtype, seed=0):
    """Inputs drawn the way the reference's tests draw them (src/test_equivalence.py:21-24):
    one generator seeded 0, order K, V, Q."""
    g = torch.Generator().manual_seed(seed)
    return [torch.randn((M, B, T, H, dk), generator=g, dtype=dtype) for _ in range(3)]
