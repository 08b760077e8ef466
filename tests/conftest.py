import os
import sys

import pytest

ROOT = os.path.abspath(os.path.join(os.path.dirname(__file__), ".."))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


@pytest.fixture(scope="session")
def golden():
    import numpy as np
    return np.load(os.path.join(ROOT, "tests", "golden", "attention_golden.npz"))


@pytest.fixture(scope="session")
def engine():
    """The engine context on cuda:0.  Fails (does not skip) when the library is missing."""
    import torch
    from logos_b200.engine import Engine
    assert torch.cuda.is_available(), "gpu tests need a CUDA device"
    eng = Engine(0)
    yield eng
    eng.close()


@pytest.fixture(scope="session")
def engine_general():
    """A context that never takes the tensor-core prefill kernel (exact fp32 arithmetic path)."""
    import torch
    from logos_b200.engine import Engine
    from logos_b200 import lib as L
    assert torch.cuda.is_available(), "gpu tests need a CUDA device"
    eng = Engine(0)
    eng.set_option(L.OPT_FORCE_GENERAL, 1)
    yield eng
    eng.close()
