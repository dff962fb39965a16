import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import __graft_entry__ as entry  # noqa: E402


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200 with -m gpu)")


@pytest.fixture(scope="session")
def oracle():
    return entry.load_oracle()


@pytest.fixture(scope="session")
def pkg():
    return entry.load_package()


@pytest.fixture(scope="session")
def synth(pkg):
    from glmflash_b200 import synth as s
    return s


@pytest.fixture(scope="session")
def cuda(pkg):
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    pkg.lib()          # raises if the extension is missing: GPU tests never fall back to anything else
    return torch.device("cuda:0")


def rel_err(got, want):
    """(max |got-want| / max |want|, ||got-want|| / ||want||): the two error figures every parity test states."""
    got = np.asarray(got, dtype=np.float64)
    want = np.asarray(want, dtype=np.float64)
    d = got - want
    return float(np.abs(d).max() / max(np.abs(want).max(), 1e-30)), float(np.linalg.norm(d) / max(np.linalg.norm(want), 1e-30))


TOL = 1e-3   # the tolerance of the benchmark definition: layer outputs within 1e-3 relative error, fp32 accumulation
