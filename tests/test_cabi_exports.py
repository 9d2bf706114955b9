"""The C-ABI library loads without a GPU and exports every symbol include/otter_b200.h declares."""
import ctypes as C
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


@pytest.fixture(scope="module")
def lib():
    from tensor_b200.build import build
    build()
    from tensor_b200 import capi
    return capi.library()


def declared_symbols():
    names = set()
    for header in sorted((ROOT / "include").glob("*.h")):
        text = re.sub(r"/\*.*?\*/", "", header.read_text(), flags=re.S)
        names |= set(re.findall(r"\b(ott_[a-z0-9_]+)\s*\(", text))
    return sorted(names)


def test_header_and_binding_list_agree(lib):
    from tensor_b200 import capi
    assert declared_symbols() == sorted(capi.SIGNATURES)


def test_every_declared_symbol_is_exported(lib):
    for name in declared_symbols():
        assert hasattr(lib, name), name


def test_no_gpu_means_failure_not_fallback(lib):
    n = C.c_int(-1)
    rc = lib.ott_cuda_device_count(C.byref(n))
    if rc == 0 and n.value > 0:
        pytest.skip("a GPU is present")
    h = C.c_void_p()
    assert lib.ott_ctx_create(0, C.byref(h)) != 0 and not h.value
    assert lib.ott_nhwc_channels(58) == 64 and lib.ott_nhwc_channels(3) == 16 and lib.ott_nhwc_channels(64) == 64
