"""Test configuration: the ``gpu`` marker and import paths."""

import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "tests", "golden")):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")
    config.addinivalue_line("markers", "small_kernels: leave the light kernels for short-window causal prefill on")


def pytest_collection_modifyitems(config, items):
    try:
        import torch

        have_gpu = torch.cuda.is_available()
    except Exception:  # noqa: BLE001
        have_gpu = False
    if have_gpu:
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(autouse=True)
def _large_kernels_by_default(request):
    """The GPU parity tests of causal prefill were written against the tcgen05 kernels, some of them on inputs whose
    key window is short enough that the operators would hand them to the light kernels for such windows. They keep
    testing the large kernels: the light ones are switched off around every GPU test and have tests of their own
    (tests/test_small_gpu.py, which asks for them with the ``small_kernels`` marker)."""
    if "gpu" not in request.keywords:
        yield
        return
    from cleave_b200 import ops

    old = ops.set_small_problem_limit(256 if "small_kernels" in request.keywords else 0)
    try:
        yield
    finally:
        ops.set_small_problem_limit(old)
