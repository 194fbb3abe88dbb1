"""Shared pytest configuration: the `gpu` marker and the import path of the repository root."""
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def _cuda_present() -> bool:
    try:
        import torch
        return torch.cuda.is_available()
    except Exception:
        return False


def pytest_collection_modifyitems(config, items):
    if _cuda_present():
        return
    skip = pytest.mark.skip(reason="no CUDA device in this process")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


def pytest_terminal_summary(terminalreporter):
    """The raw max-abs error and the reference-style deviation (max |a - e| / max |e|,
    Tests/HydraMetalTests/AttentionKernelTests.swift:29-37) of every full-size parity case."""
    try:
        from tests import hydra_testlib as tl
    except Exception:
        return
    if not tl.MARGINS:
        return
    terminalreporter.write_line("parity margins against the oracle (bound: max-abs 1e-2):")
    for name, worst, dev, count in tl.MARGINS:
        terminalreporter.write_line(f"  {name}: max-abs {worst:.3e}, deviation {dev:.3e} over {count} values")
