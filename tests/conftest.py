"""Shared fixtures: the ``gpu`` marker, golden-fixture loading, seeded inputs."""

from __future__ import annotations

import pathlib
import sys

import numpy as np
import pytest
import torch

ROOT = pathlib.Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

GOLDEN = ROOT / "tests" / "golden"


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


def load_golden(name):
    """A golden fixture as a dict of torch tensors (``inputs_checksum`` stays a float)."""
    with np.load(GOLDEN / f"{name}.npz") as z:
        out = {k: torch.from_numpy(z[k]) if z[k].ndim else float(z[k]) for k in z.files}
    return out


def golden_checksum(*tensors):
    """Same fingerprint ``tests/golden/make_golden.py`` stores beside every fixture."""
    acc = 0.0
    for i, t in enumerate(tensors):
        t = t.double().flatten()
        ramp = torch.arange(1, t.numel() + 1, dtype=torch.float64) / t.numel()
        acc += (i + 1) * float((t * ramp).sum())
    return acc


def golden_state(B, H, DK, DV, seed, std):
    gen = torch.Generator(device="cpu").manual_seed(1000 + seed)
    return torch.randn(B, H, DK, DV, generator=gen) * std


def note(test, **values):
    """Append measured error figures to the file named by ``GDN2_TEST_NOTES`` (one JSON object per line), so a
    run leaves a record of how far inside its tolerances every comparison landed. No-op without the variable."""
    import json
    import os

    path = os.environ.get("GDN2_TEST_NOTES")
    if path:
        with open(path, "a") as f:
            f.write(json.dumps({"test": test, **{k: (float(v) if hasattr(v, "__float__") else v) for k, v in values.items()}}) + "\n")
