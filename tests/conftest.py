"""Shared pytest setup: the ``gpu`` marker, import paths, and the oracle."""
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200, sm_100a)")


def pytest_collection_modifyitems(config, items):
    # No test here needs minutes: a per-test limit (pytest-timeout, when installed) turns a
    # stuck host call into one failed test instead of a run that never ends.
    if config.pluginmanager.hasplugin("timeout"):
        for item in items:
            if item.get_closest_marker("timeout") is None:
                item.add_marker(pytest.mark.timeout(300))
    # GPU tests skip themselves on a machine without a device, so that the CPU
    # suite can be run with or without "-m 'not gpu'".
    try:
        import torch
        has_gpu = torch.cuda.is_available()
    except Exception:  # pragma: no cover - torch is part of the image
        has_gpu = False
    if has_gpu:
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def oracle():
    """The CPU restatement of the reference (test infrastructure)."""
    from oracle import oracle as orc
    orc.build()
    orc.lib()
    return orc


@pytest.fixture(scope="session")
def pkg():
    """The product package (directory ``oxide-train_b200``)."""
    import __graft_entry__ as entry
    return entry.load_package()
