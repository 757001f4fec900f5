"""Shared pytest configuration: the ``gpu`` marker, import paths and the golden fixtures."""

import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

REFERENCE_ROOT = os.environ.get("LQ_REFERENCE_ROOT", "/root/reference")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def pytest_collection_modifyitems(config, items):
    """GPU-marked tests are skipped, never silently passed, when no device is present."""
    try:
        import torch
        have = torch.cuda.is_available()
    except Exception:  # pragma: no cover
        have = False
    if have:
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for it in items:
        if "gpu" in it.keywords:
            it.add_marker(skip)


class Golden:
    """Name-spaced view on tests/golden/lqq_golden.npz (arrays computed by the reference)."""

    def __init__(self, path):
        self._z = np.load(path)
        self.cases = sorted({k.split("/")[0] for k in self._z.files})

    def get(self, case, key):
        return self._z[f"{case}/{key}"]

    def has(self, case, key):
        return f"{case}/{key}" in self._z.files


@pytest.fixture(scope="session")
def golden():
    return Golden(os.path.join(ROOT, "tests", "golden", "lqq_golden.npz"))


def have_reference():
    return os.path.isdir(os.path.join(REFERENCE_ROOT, "liquidgemm"))
