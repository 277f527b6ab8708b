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
    config.addinivalue_line("markers", "gpu: needs a CUDA device (sm_100a)")


def load_golden(name):
    with np.load(os.path.join(GOLDEN, name + ".npz")) as z:
        return {k: z[k] for k in z.files}


@pytest.fixture(scope="session")
def golden():
    return load_golden


@pytest.fixture(scope="session")
def dev():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return torch.device("cuda:0")


@pytest.fixture(scope="session")
def lib():
    # Built by __graft_entry__.build(); a missing library is an error, never a skip.
    from custom_matmul_kernels_b200.custom_kernel import load_library
    return load_library()


def tol_ratio(got, want, rtol=1e-5, atol=1e-4):
    """max |got - want| / (atol + rtol |want|): <= 1 means inside the stated tolerance."""
    got = got.detach().double().cpu()
    want = want.detach().double().cpu()
    return float(((got - want).abs() / (atol + rtol * want.abs())).max())
