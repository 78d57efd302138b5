"""Test configuration: markers, import paths and shared fixtures."""

import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
for entry in (str(ROOT), str(ROOT / "tests" / "golden")):
    if entry not in sys.path:
        sys.path.insert(0, entry)

import cfm_b200  # noqa: E402,F401  (registers the package alias `cfm_b200`)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def oracle():
    """The CPU oracle module, compiled on first use."""
    from oracle import reader_oracle

    reader_oracle.load()
    return reader_oracle
