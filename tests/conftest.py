"""Shared pytest configuration: the ``gpu`` marker and golden-fixture loading."""
from __future__ import annotations

import sys
from pathlib import Path

import numpy as np
import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

GOLDEN = Path(__file__).resolve().parent / "golden"


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


def load_golden(name: str) -> dict:
    """Load a fixture written by tests/golden/make_golden.py; ``__bf16`` arrays come back as
    torch.bfloat16 tensors, float/int arrays as torch tensors, scalars as Python numbers."""
    out = {}
    with np.load(GOLDEN / f"{name}.npz") as z:
        for key in z.files:
            arr = z[key]
            if key.endswith("__bf16"):
                out[key[: -len("__bf16")]] = torch.from_numpy(arr.view(np.int16).copy()).view(torch.bfloat16)
            elif arr.ndim == 0:
                out[key] = arr.item()
            else:
                out[key] = torch.from_numpy(arr.copy())
    return out


def rel_l2(a: torch.Tensor, b: torch.Tensor) -> float:
    a = a.double().flatten()
    b = b.double().flatten()
    denom = b.norm().item()
    return (a - b).norm().item() / (denom if denom > 0 else 1.0)


def max_abs(a: torch.Tensor, b: torch.Tensor) -> float:
    return (a.double() - b.double()).abs().max().item() if a.numel() else 0.0
