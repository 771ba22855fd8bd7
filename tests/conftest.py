"""Shared pytest configuration: registers the ``gpu`` marker, puts the repository root on
``sys.path`` and offers helpers to load the golden fixtures."""
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
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


def load_golden(name):
    return dict(np.load(os.path.join(GOLDEN, f"{name}.npz")))


def bf16_from_bits(bits):
    return torch.from_numpy(np.asarray(bits).astype(np.int16)).view(torch.bfloat16)


GOLDEN_CASES = ["mlp_tile16_d64", "mlp_tile16_d128_cs16", "mlp_blk128_d256"]
