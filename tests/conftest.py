import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(autouse=True)
def _reset_dc_state():
    """Class-level registries of the module API are process-global; start every test clean."""
    yield
    try:
        from deltacnn_b200 import DCThreshold, DCConv2d, DCBackend
        from deltacnn_b200.sparse_layers import DCAdd, DCSparsify, DCActivation, DCDensify, DCModule
        DCThreshold.reset()
        DCThreshold.t_default = 0.0
        DCConv2d.backend = DCBackend.deltacnn
        DCConv2d.conv_idx = -1
        DCConv2d.fuse_blocks = False
        DCConv2d.fuse_heads = True
        DCAdd.idx = DCSparsify.idx = DCActivation.idx = DCDensify.idx = -1
        DCModule.temp_buffers = []
    except Exception:
        pass
