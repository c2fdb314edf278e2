"""pytest configuration: registers the ``gpu`` marker and puts the repo root on
``sys.path`` so that ``slinoss_b200`` and ``oracle`` import from the tree."""

from __future__ import annotations

import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200)")
