"""CPU-side checks of the drop-in boundary: the library builds, loads, and exports every symbol the
public header declares (no compute calls -- those need a GPU)."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def built_lib():
    from litert_b200 import build

    return build.build_kernels()


def _declared(header):
    text = open(os.path.join(ROOT, "include", header)).read()
    return sorted(set(re.findall(r"\b(b200_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol(built_lib):
    lib = ctypes.CDLL(built_lib)
    names = _declared("litert_b200.h")
    assert len(names) >= 15
    for name in names:
        assert hasattr(lib, name), f"{name} declared in include/litert_b200.h but not exported"


def test_ctypes_binding_covers_the_header():
    from litert_b200 import _lib

    assert sorted(_lib.SIGNATURES) == _declared("litert_b200.h")
    lib = _lib.load()
    assert lib.b200_abi_version() == 1


def test_size_queries_need_no_gpu():
    from litert_b200 import _lib

    lib = _lib.load()
    assert lib.b200_packed_w8_bytes(14336, 4096) == 14336 * 4096
    assert lib.b200_packed_w8_bytes(130, 100) == 2 * 1 * 16384  # padded to whole tiles
    assert lib.b200_packed_w4_bytes(16384, 2048) == (16384 // 128) * (2048 // 256) * (16384 + 2048)
    assert lib.b200_zero_workspace_bytes() > 256 * 128 * 64 * 4
    assert lib.b200_fc_scratch_bytes(1, 4096) >= 8 * 4096
    assert lib.b200_fc_scratch_bytes(0, 4096) == 0
    assert lib.b200_sdpa_workspace_bytes(16, 8, 1, 256, 8192) > 0


def test_argument_errors_are_reported_not_fatal():
    from litert_b200 import _lib

    lib = _lib.load()
    rc = lib.b200_pack_w8(None, 4, 4, None, None, None)
    assert rc == 1
    assert b"b200_pack_w8" in lib.b200_last_error()
    rc = lib.b200_sdpa_decode(None, None, None, None, None, None, None, None, 1, 8, 3, 64, 128, 0, 0, 0.0, 0.0, None,
                              0, None)
    assert rc == 1
