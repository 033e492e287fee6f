import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line('markers', 'gpu: needs a CUDA device (B200, sm_100a)')


@pytest.fixture(scope='session')
def oracle():
    from oracle import c_oracle
    c_oracle.build()
    return c_oracle


@pytest.fixture(scope='session')
def golden():
    import numpy as np
    path = os.path.join(ROOT, 'tests', 'golden', 'golden_small.npz')
    return np.load(path)
