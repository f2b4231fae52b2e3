"""No GPU needed: the C-ABI library loads and exports every symbol that include/tagi_b200.h declares, the Python
binding lists them all, and host-only entry points behave."""
import ctypes as C
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "tagi_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(tagi_[a-z0-9_]+)\s*\(", text)))


@pytest.fixture(scope="module")
def cdll():
    from cutagi_b200 import build, capi
    if not os.path.exists(capi.LIB_PATH):
        build.build()
    return C.CDLL(capi.LIB_PATH)


def test_header_declares_the_expected_entry_points():
    syms = declared_symbols()
    for s in ("tagi_linear_fwd", "tagi_linear_bwd_state", "tagi_linear_bwd_param", "tagi_conv2d_fwd",
              "tagi_conv2d_bwd_state", "tagi_conv2d_bwd_param", "tagi_last_error_string"):
        assert s in syms


def test_library_exports_every_declared_symbol(cdll):
    missing = [s for s in declared_symbols() if not hasattr(cdll, s)]
    assert not missing, f"declared in include/tagi_b200.h but not exported: {missing}"


def test_python_binding_covers_every_symbol():
    from cutagi_b200 import capi
    bound = set(capi._SIGNATURES) | {"tagi_last_error_string", "tagi_conv2d_workspace_bytes", "tagi_scratch_bytes"}
    assert set(declared_symbols()) <= bound


def test_host_only_entry_points(cdll):
    from cutagi_b200.capi import TagiError, conv_out_size, lib
    assert lib.tagi_version() >= 100
    assert conv_out_size(3, 1, 32, 32, 1, 1) == (32, 32)
    with pytest.raises(TagiError) as e:
        conv_out_size(3, 2, 8, 8, 0, 0)
    assert e.value.code == 1
    # host-only sizing of the Conv2d scratch: positive for a valid geometry, 0 for an inconsistent one
    from cutagi_b200.capi import ConvGeom as CG
    good = CG(64, 64, 56, 56, 64, 56, 56, 3, 1, 1, 1, 0)
    assert lib.tagi_conv2d_workspace_bytes(C.byref(good)) > 0
    bad = CG(1, 1, 8, 8, 1, 5, 5, 3, 1, 0, 0, 0)
    assert lib.tagi_conv2d_workspace_bytes(C.byref(bad)) == 0
    lib.tagi_set_impl(1)
    assert lib.tagi_get_impl() == 1
    lib.tagi_set_impl(0)
    with pytest.raises(TagiError):
        lib.tagi_set_impl(9)


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    from cutagi_b200 import capi
    monkeypatch.setattr(capi, "LIB_PATH", str(tmp_path / "nope.so"))
    monkeypatch.setattr(capi, "_lib", None)
    with pytest.raises(ImportError):
        capi.load()
