"""Shared test plumbing: import paths, the `gpu` marker, golden fixtures."""

import sys
from pathlib import Path

import numpy as np
import pytest

REPO = Path(__file__).resolve().parent.parent
for p in (REPO, REPO / "sparse-attention-hub_b200"):
    if str(p) not in sys.path:
        sys.path.insert(0, str(p))

GOLDEN = REPO / "tests" / "golden"


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


def load_golden(name: str):
    return dict(np.load(GOLDEN / f"{name}.npz"))


@pytest.fixture(scope="session")
def golden():
    return load_golden
