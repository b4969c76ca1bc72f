"""The shared library loads without a GPU and exports every function include/dsb200.h declares; the
host-only entry points (sizes, argument checks that fail before any CUDA call) behave."""
import ctypes as C
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "dsb200.h")


@pytest.fixture(scope="module")
def lib():
    from ds_splat_b200 import _capi, build
    if not os.path.exists(_capi.LIB_PATH):
        build.build()
    return _capi.lib()


def declared_functions():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(dsb_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_what_python_binds():
    from ds_splat_b200 import _capi
    assert set(_capi.EXPORTS) <= set(declared_functions())


def test_every_declared_symbol_is_exported(lib):
    names = declared_functions()
    assert len(names) >= 18
    for name in names:
        assert hasattr(lib, name), f"{name} declared in dsb200.h but not exported by libdsb200.so"


def test_host_only_calls(lib):
    assert lib.dsb_version() >= 100
    assert lib.dsb_launch_count() >= 0
    a, b = lib.dsb_sort_workspace_bytes(1), lib.dsb_sort_workspace_bytes(10_000_000)
    assert 0 < a < b
    assert lib.dsb_plan_workspace_bytes(1_000_000) > lib.dsb_sort_workspace_bytes(1_000_000)


def test_argument_errors_are_reported_not_crashed(lib):
    from ds_splat_b200 import _capi
    cam = _capi.DsbCamera()  # all zero: invalid image size
    rc = lib.dsb_blend_forward(C.byref(cam), None, None, None, None, None, None, None, None)
    assert rc == -1
    assert b"image size" in lib.dsb_last_error()
    rc = lib.dsb_sort_pairs(None, None, 10, 40, 32, None, 0, None, None)
    assert rc == -1 and b"bit range" in lib.dsb_last_error()
    rc = lib.dsb_sort_pairs(None, None, 1 << 31, 0, 8, None, 0, None, None)
    assert rc == -4  # DSB_ERR_TOO_MANY_PAIRS
    in_alt = C.c_int32(7)
    assert lib.dsb_sort_pairs(None, None, 0, 0, 8, None, 0, C.byref(in_alt), None) == 0 and in_alt.value == 0
