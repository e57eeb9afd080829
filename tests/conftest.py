import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "tests", "golden")):
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


# Parity figures measured by the GPU tests against the reference's fixtures (code bits that differ,
# scores that differ, overlap of the attended sets): collected here and printed after the run, so that
# the numbers behind the asserted bounds are in the log.
PARITY_REPORT = []


@pytest.fixture
def parity_report():
    def add(name, **figures):
        PARITY_REPORT.append((name, figures))
    return add


def pytest_terminal_summary(terminalreporter):
    if not PARITY_REPORT:
        return
    terminalreporter.section("parity against the reference's fixtures (measured)")
    for name, figures in PARITY_REPORT:
        terminalreporter.write_line(name + ": " + ", ".join(f"{k}={v}" for k, v in figures.items()))
