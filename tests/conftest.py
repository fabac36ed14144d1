"""Shared fixtures: the `gpu` marker, the golden-vector loader, and the import
of the (hyphen-named) product package."""
from __future__ import annotations

import importlib
import os
import sys

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG_NAME = "rag-cache-engineering-qwen35-9b-flute_b200"
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


def load_pkg():
    """Import the product package (its directory name is not an identifier)."""
    return importlib.import_module(PKG_NAME)


@pytest.fixture(scope="session")
def pkg():
    return load_pkg()


class Golden:
    """Read access to tests/golden/reference_vectors.npz; 16-bit float tensors
    are stored as raw bit patterns under '<key>__bf16' / '<key>__f16'."""

    def __init__(self, path):
        self.z = np.load(path)
        self.keys = set(self.z.files)

    def has(self, key):
        return key in self.keys or key + "__bf16" in self.keys or key + "__f16" in self.keys

    def np(self, key):
        return self.z[key]

    def t(self, key):
        if key in self.keys:
            return torch.from_numpy(self.z[key])
        if key + "__bf16" in self.keys:
            return torch.from_numpy(self.z[key + "__bf16"].view(np.int16)).view(torch.bfloat16)
        if key + "__f16" in self.keys:
            return torch.from_numpy(self.z[key + "__f16"].view(np.int16)).view(torch.float16)
        raise KeyError(key)

    def opt(self, key):
        return self.t(key) if self.has(key) else None


@pytest.fixture(scope="session")
def golden():
    return Golden(os.path.join(ROOT, "tests", "golden", "reference_vectors.npz"))


@pytest.fixture(scope="session")
def golden_embedding():
    return Golden(os.path.join(ROOT, "tests", "golden", "embedding_vectors.npz"))


def pytest_terminal_summary(terminalreporter):
    """Observed maxima of the parity checks (bound: 1e-2 unless the test says otherwise), the
    five largest and the count, so a regression shows before it crosses the bound."""
    try:
        from helpers import OBSERVED
    except Exception:
        return
    if not OBSERVED:
        return
    worst = sorted(OBSERVED.items(), key=lambda kv: -kv[1])[:5]
    terminalreporter.write_line(f"observed max-relative errors of {len(OBSERVED)} tests; largest:")
    for name, e in worst:
        terminalreporter.write_line(f"  {e:.3e}  {name}")
