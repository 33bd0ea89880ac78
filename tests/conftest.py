"""pytest configuration: the `gpu` marker and shared helpers.

`-m "not gpu"` tests run on CPU (oracle vs golden vectors, host logic, library
symbols).  `-m gpu` tests call the C-ABI on a B200 and compare with the oracle.
"""
from __future__ import annotations

import importlib
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 GPU; calls the CUDA kernels through the C-ABI")


def pkg(sub: str = ""):
    """Import a module of the hyphen-named package."""
    return importlib.import_module("inference-server_b200" + (("." + sub) if sub else ""))


def golden(name: str):
    return np.load(os.path.join(GOLDEN, name))


@pytest.fixture(scope="session")
def ops():
    import torch

    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    pkg("_lib").load()  # raises if the library is missing: no silent fallback
    return pkg("ops")


def rel_err(a, b) -> float:
    """max |a - b| / max |b| over the whole tensor (fp32)."""
    import torch

    a = a.detach().float().cpu()
    b = b.detach().float().cpu()
    return float((a - b).abs().max() / b.abs().max().clamp_min(1e-30))
