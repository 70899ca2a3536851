"""Shared fixtures.  GPU tests are marked `gpu`; everything else must pass on a CPU-only box."""
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "oracle"))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (sm_100a) GPU")


@pytest.fixture(scope="session")
def oracle():
    import oracle as o  # oracle/oracle.py
    o.build()
    return o


@pytest.fixture(scope="session")
def xf():
    import xefuse_loader
    return xefuse_loader.load()


@pytest.fixture(scope="session")
def capi(xf):
    xf.build()
    return xf.capi


@pytest.fixture(scope="session")
def cuda():
    import torch
    if not torch.cuda.is_available():
        pytest.fail("a `gpu` test was selected but no CUDA device is visible")
    return torch.device("cuda:0")


def bf16_bits(t):
    """torch bf16 tensor -> numpy uint16 bit patterns."""
    import torch
    return t.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16)


def bits_to_f32(u):
    return (u.astype(np.uint32) << 16).view(np.float32)
