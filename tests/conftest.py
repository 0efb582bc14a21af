"""Test configuration: the ``gpu`` marker (tests that need a B200) and shared fixtures."""
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200 with -m gpu)")


def golden(name):
    return np.load(os.path.join(GOLDEN, name))


@pytest.fixture(scope="session")
def config0():
    """Benchmark configuration 0 at full shape: (weights tuple, x bf16 bits [16,6144], logits [16,128]) from seed 0."""
    from oracle import moe_oracle as orc
    weights, gen = orc.make_weights(seed=0)
    xb, lg = orc.make_inputs(gen, 16)
    return weights, xb, lg
