"""Shared pytest set-up: markers, import path, the golden fixture and the oracle."""

from __future__ import annotations

import io
import lzma
import sys
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def golden():
    raw = lzma.decompress((ROOT / "tests" / "golden" / "reference_golden.pt.xz").read_bytes())
    return torch.load(io.BytesIO(raw), weights_only=False)


@pytest.fixture(scope="session")
def oracle():
    from oracle import fos_oracle

    fos_oracle.lib()
    return fos_oracle


def has_cuda() -> bool:
    return torch.cuda.is_available()
