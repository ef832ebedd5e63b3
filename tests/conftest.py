import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
TESTS = os.path.dirname(os.path.abspath(__file__))
if TESTS not in sys.path:
    sys.path.insert(0, TESTS)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def pytest_collection_modifyitems(config, items):
    # the test of the allocation-free entry point runs after every other test
    items.sort(key=lambda item: 1 if "test_zz_" in item.nodeid else 0)


def pytest_terminal_summary(terminalreporter):
    """How close the compared logits were, next to the limit each was held to."""
    import helpers
    if not helpers.MEASURED:
        return
    terminalreporter.section("worst |diff| / max |logit| of the compared logits")
    for what, (worst, tol) in sorted(helpers.MEASURED.items(), key=lambda kv: -kv[1][0] / kv[1][1]):
        terminalreporter.write_line(f"{worst:9.2e}  of limit {tol:7.1e}  ({100 * worst / tol:5.1f} %)  {what}")
