"""pytest configuration: the `gpu` marker, import paths and golden-fixture loading."""
from __future__ import annotations

import sys
from pathlib import Path

import numpy as np
import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
for p in (ROOT, ROOT / "mini-attention_b200"):
    if str(p) not in sys.path:
        sys.path.insert(0, str(p))

GOLDEN = ROOT / "tests" / "golden"
_DT = {"torch.float16": torch.float16, "torch.bfloat16": torch.bfloat16, "torch.float32": torch.float32}

# north-star tolerances on max |out - reference|
TOL = {torch.float16: 2e-3, torch.bfloat16: 1e-2}


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200, sm_100a)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


def load_golden(name: str) -> dict:
    """Load a fixture written by tests/golden/make_golden.py; 16-bit tensors come back exact."""
    out = {}
    with np.load(GOLDEN / f"{name}.npz") as z:
        for key in z.files:
            if key.endswith("__dtype"):
                continue
            arr = z[key]
            dt_key = key + "__dtype"
            if dt_key in z.files:
                dt = _DT[str(z[dt_key])]
                if dt in (torch.float16, torch.bfloat16):
                    out[key] = torch.from_numpy(arr.view(np.int16).copy()).view(dt)
                else:
                    out[key] = torch.from_numpy(arr.copy())
            else:
                out[key] = arr.item() if arr.shape == () else arr
    return out


def golden_names():
    return sorted(p.stem for p in GOLDEN.glob("*.npz"))
