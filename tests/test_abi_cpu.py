"""The drop-in boundary without a GPU: the library builds for sm_100a, loads,
exports every symbol the header declares, and refuses to run without a device."""
import ctypes as C
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    from coalsack_b200.build import build_library
    build_library()
    from coalsack_b200 import _lib
    return _lib.load()


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "csk_moe.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(csk_moe_[a-z0-9_]+)\s*\(", text)))


def test_header_and_binding_agree(lib):
    from coalsack_b200 import _lib
    decl = declared_symbols()
    assert len(decl) >= 20
    assert sorted(_lib.SYMBOLS) == decl


def test_library_exports_every_declared_symbol(lib):
    raw = C.CDLL(lib._name)
    for name in declared_symbols():
        assert hasattr(raw, name), name


def test_struct_sizes_match_header():
    from coalsack_b200._lib import Config, Timings
    assert C.sizeof(Config) == 12 * 4 + 8
    assert C.sizeof(Timings) == 6 * 4 + 2 * 4


def test_no_gpu_means_loud_failure(lib):
    if lib.csk_moe_device_ok(0):
        pytest.skip("a GPU is present")
    from coalsack_b200 import CskError, MoeLayer
    with pytest.raises(CskError) as ei:
        MoeLayer(4, 2, 64, 64)
    assert "no CPU fallback" in str(ei.value)


def test_config_validation_messages(lib):
    from coalsack_b200._lib import Config
    h = C.c_void_p()
    bad = Config(4, 2, 48, 64, 0, 1, 0, 0, 0, 0, 0, 0, 8)
    assert lib.csk_moe_create(C.byref(bad), C.byref(h)) == -1
    assert b"hidden_dim must be a multiple of 32" in lib.csk_moe_last_error(None)
    bad = Config(4, 9, 64, 64, 0, 1, 0, 0, 0, 0, 0, 0, 8)
    assert lib.csk_moe_create(C.byref(bad), C.byref(h)) == -1
    bad = Config(4, 2, 64, 64, 0, 1, 0, 0, 0, 3, 2, 0, 8)
    assert lib.csk_moe_create(C.byref(bad), C.byref(h)) == -1
    assert b"expert range" in lib.csk_moe_last_error(None)


def test_product_does_not_touch_the_oracle():
    """Nothing in the package or the C ABI may import, link or run the CPU checker."""
    pkg = os.path.join(ROOT, "coalsack_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h", ".cpp")):
                text = open(os.path.join(dirpath, f)).read()
                assert "import oracle" not in text and "from oracle" not in text, f
                assert "libcsk_oracle" not in text and "libcsk_ref" not in text, f
