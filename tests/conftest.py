"""Shared test configuration.

``-m "not gpu"`` tests cover the oracle against the golden vectors, the host
logic and the C-ABI exports; ``-m gpu`` tests are the parity tests proper and
need a CUDA device.
"""

from __future__ import annotations

from pathlib import Path
import sys

import pytest

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config: pytest.Config) -> None:
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200)")


def pytest_collection_modifyitems(config: pytest.Config, items: list[pytest.Item]) -> None:
    import torch

    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="CUDA is required")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)
