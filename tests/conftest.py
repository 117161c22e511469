"""Test configuration: markers and import paths.

The package source root (the directory holding `custom/`, `models/` and
`backend/`, named like the reference's top-level packages) is put on sys.path so
that tests read like the reference's own: `from custom import ...`.
"""
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG_ROOT = os.path.join(ROOT, "fp4-training_b200")
for p in (ROOT, PKG_ROOT):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")
