# SPDX-License-Identifier: MIT
"""pytest configuration: the `gpu` marker and shared helpers.

Tests without the marker run on a machine with no GPU (CPU tensors, gloo
ranks).  Tests with it need a B200; those that need several skip themselves
when the box has fewer."""
import os
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs at least one CUDA device (B200, sm_100a)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


def rel_l2(a, b):
    a, b = a.float(), b.float()
    return ((a - b).norm() / b.norm().clamp_min(1e-12)).item()


@pytest.fixture(scope="session")
def ext():
    import barlink_sm86_b200 as bl

    return bl.load_extension()
