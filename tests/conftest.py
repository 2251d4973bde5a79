"""Shared test plumbing: path set-up, the `gpu` marker, and helpers that build inputs with the
CPU oracle's seeded generator."""
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "suzuqu-engine-4exp_b200")):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def oracle():
    from oracle import q4_oracle
    q4_oracle.lib()
    return q4_oracle
