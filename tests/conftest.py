import os
import sys

import pytest

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


def pytest_collection_modifyitems(config, items):
    try:
        import torch
        have = torch.cuda.is_available()
    except Exception:
        have = False
    if have:
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


def pytest_terminal_summary(terminalreporter):
    """The largest logit errors (relative to the largest logit) that assert_close saw, by precision."""
    try:
        import helpers
    except Exception:
        return
    for dtype, (ratio, what) in sorted(helpers.worst.items()):
        terminalreporter.write_line(f"largest logit error seen, {dtype}: {ratio:.3e} of max |logit| ({what}); "
                                    f"bound {helpers.TOL[dtype]:.1e}")
