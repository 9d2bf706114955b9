import sys
from pathlib import Path

import pytest

import os

# Every device block of every GPU test carries 4 KiB guard bands, which the contexts check when they are closed (the library's
# stand-in for a device memory checker; include/otter_b200.h, ott_debug_guard_bands). OTT_DEBUG_GUARD_BYTES=0 switches it off.
os.environ.setdefault("OTT_DEBUG_GUARD_BYTES", "4096")

sys.path.insert(0, str(Path(__file__).resolve().parent))
sys.path.insert(0, str(Path(__file__).resolve().parent.parent))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the GPU box with -m gpu)")
