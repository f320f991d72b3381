from __future__ import annotations

import sys
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
for p in (str(ROOT), str(ROOT / "tests")):
    if p not in sys.path:
        sys.path.insert(0, p)

GOLDEN = ROOT / "tests" / "golden"


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def lib():
    from spikeinfer_b200 import build

    build.build()
    from spikeinfer_b200 import _lib

    return _lib.load()


@pytest.fixture(scope="session")
def golden():
    def load(name: str):
        return torch.load(GOLDEN / f"{name}.pt", weights_only=False)

    return load


@pytest.fixture(scope="session")
def dev(lib):
    return torch.device("cuda:0")


def to_dev(case: dict, device) -> dict:
    return {k: (v.to(device) if isinstance(v, torch.Tensor) else v) for k, v in case.items()}
