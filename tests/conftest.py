import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.dirname(os.path.abspath(__file__))):
    if p not in sys.path:
        sys.path.insert(0, p)


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


def pytest_terminal_summary(terminalreporter):
    """The measured errors against the plain implementation, worst first within each dtype."""
    try:
        from helpers import WORST
    except ImportError:
        return
    for dtype in ("bfloat16", "float32", ""):
        rows = sorted(((e, t) for t, e in WORST.items() if (dtype in t if dtype else not ("bfloat16" in t or "float32" in t))),
                      reverse=True)[:6]
        dtype = dtype or "other tests"
        if rows:
            terminalreporter.write_line(f"worst relative errors against the plain implementation, {dtype}:")
            for e, t in rows:
                terminalreporter.write_line(f"  {e:.3e}  {t}")
