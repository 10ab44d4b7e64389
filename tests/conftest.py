"""Shared pytest setup: registers the ``gpu`` marker and puts the product directory on sys.path."""
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
PKG = ROOT / "qwen3_5-triton-inference-engine_b200"
for p in (str(ROOT), str(PKG)):
    if p not in sys.path:
        sys.path.insert(0, p)

GOLDEN = ROOT / "tests" / "golden"


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def golden():
    import torch

    def load(name):
        return torch.load(GOLDEN / f"{name}.pt", map_location="cpu")

    return load
