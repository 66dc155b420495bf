"""Test configuration: the ``gpu`` marker and shared fixtures.

Tests marked ``gpu`` need a CUDA device and the compiled kernels; everything else runs on the CPU.
Model folders are made in temporary folders and never committed.
"""

import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def pytest_collection_modifyitems(config, items):
    import torch

    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(autouse=True)
def _seed_from_the_tests_name(request):
    """Every test draws its random inputs from a generator seeded by its own name, so that what a test sees
    does not depend on which tests ran before it, and a failure can be reproduced alone."""
    import zlib

    import torch

    torch.manual_seed(zlib.crc32(request.node.nodeid.encode()))   # seeds the CPU and every CUDA generator
    yield


@pytest.fixture(scope="session")
def model_dirs(tmp_path_factory):
    """{config name: model folder} for the tiny test configurations, random weights."""
    import helpers

    out = {}
    for name in helpers.TINY:
        d = tmp_path_factory.mktemp(f"model_{name}")
        helpers.make_model_dir(name, str(d))
        out[name] = str(d)
    return out
