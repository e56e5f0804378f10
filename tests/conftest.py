"""Shared pytest configuration: markers, repo-root import path, golden-fixture loader."""

import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

TESTS = os.path.dirname(os.path.abspath(__file__))
if TESTS not in sys.path:
    sys.path.insert(0, TESTS)

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")
    config.addinivalue_line("markers", "slow: takes more than a few seconds")


def pytest_collection_modifyitems(config, items):
    try:
        import torch

        has_cuda = torch.cuda.is_available()
    except Exception:
        has_cuda = False
    if has_cuda:
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def golden():
    def load(name):
        return np.load(os.path.join(GOLDEN, name + ".npz"))

    return load


@pytest.fixture(autouse=True)
def _name_parity_records(request):
    import parity_util

    parity_util.set_current_test(request.node.nodeid)
    yield


def pytest_terminal_summary(terminalreporter):
    import parity_util

    if not parity_util.RECORDS:
        return
    terminalreporter.section("measured norm-wise errors (max|got-ref| / max|ref|)")
    worst = {}
    for test, what, rel, tol in parity_util.RECORDS:
        key = (test, what)
        if key not in worst or rel > worst[key][0]:
            worst[key] = (rel, tol)
    for (test, what), (rel, tol) in sorted(worst.items(), key=lambda kv: -kv[1][0])[:40]:
        terminalreporter.write_line(f"{rel:9.2e}  (bound {tol:.0e})  {test} :: {what}")
