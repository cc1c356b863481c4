"""The C-ABI library builds for sm_100a, loads without a GPU and exports every symbol the public
header declares. Only host-side entry points are called here; nothing touches a device."""

import ctypes
import re
from pathlib import Path

import pytest

from sparsebench_b200 import _build, _lib

HEADER = Path(__file__).resolve().parent.parent / "include" / "sparsebench_b200.h"


def declared_symbols() -> list[str]:
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    return sorted(set(re.findall(r"\b(sb_[a-z0-9_]+)\s*\(", text)))


@pytest.fixture(scope="module")
def lib() -> ctypes.CDLL:
    _build.build()  # no-op when the library is newer than its sources
    return _lib.load()


def test_header_declares_the_whole_path() -> None:
    names = declared_symbols()
    for required in ("sb_arch_probe", "sb_route", "sb_sdd", "sb_dsd", "sb_combine", "sb_last_error"):
        assert required in names


@pytest.mark.parametrize("name", declared_symbols())
def test_library_exports_declared_symbol(lib: ctypes.CDLL, name: str) -> None:
    assert getattr(lib, name) is not None
    assert name in _lib.SIGNATURES, f"{name} is declared in the header but has no ctypes prototype"


def test_every_bound_symbol_is_declared() -> None:
    assert sorted(_lib.SIGNATURES) == declared_symbols()


def test_host_only_entry_points(lib: ctypes.CDLL) -> None:
    assert re.fullmatch(r"\d+\.\d+\.\d+", lib.sb_version().decode())
    assert lib.sb_status_string(0) == b"ok"
    assert lib.sb_status_string(1) == b"invalid argument"
    # Worst-case sizes, as the reference host code computes them (csrc/routing.cu:213-217).
    rb, rows, fb = ctypes.c_int64(), ctypes.c_int64(), ctypes.c_int64()
    assert lib.sb_route_sizes(8192, 64, 4096, 128, ctypes.byref(rb), ctypes.byref(rows), ctypes.byref(fb)) == 0
    assert (rb.value, rows.value, fb.value) == (127, 16256, 32)
    assert lib.sb_route_sizes(200, 8, 32, 16, ctypes.byref(rb), ctypes.byref(rows), ctypes.byref(fb)) == 0
    assert (rb.value, rows.value, fb.value) == ((200 + 8 * 15) // 16, (200 + 8 * 15) // 16 * 16, 2)


@pytest.mark.parametrize(("args", "text"), [
    ((2, 2000, 32, 16), "num_experts"),
    ((2, 8, 30, 16), "multiple"),
    ((2, 8, 32, 0), "block_size"),
    ((2**31, 8, 128, 128), "too large"),
    ((2_000_000, 1024, 2**20, 128), "too large"),
])
def test_route_sizes_rejects_like_the_reference(lib: ctypes.CDLL, args, text: str) -> None:
    # reference: csrc/routing.cu:205-224
    assert lib.sb_route_sizes(*args, None, None, None) == 1
    assert text in lib.sb_last_error().decode()


def test_route_workspace_is_zero_for_the_single_launch_shape(lib: ctypes.CDLL) -> None:
    assert lib.sb_route_workspace_bytes(8192, 64) == 0
    assert lib.sb_route_workspace_bytes(131_072, 1024) == 0
    assert lib.sb_route_workspace_bytes(131_073, 1024) == ((131_073 + 2047) // 2048) * 1025 * 4
    assert lib.sb_route_workspace_bytes(300_000, 1024) == ((300_000 + 2047) // 2048) * 1025 * 4


def test_null_and_shape_errors_are_reported_before_any_launch(lib: ctypes.CDLL) -> None:
    assert lib.sb_arch_probe(None, 0, None) == 1 and b"must be positive" in lib.sb_last_error()
    assert lib.sb_sdd(None, None, None, None, None, None, 4, 96, 256, 2, 1, 1, 0, None, None, None) == 1
    one = ctypes.c_void_p(256)  # never dereferenced: the size checks come first
    assert lib.sb_sdd(one, one, one, one, one, one, 4, 96, 256, 2, 1, 1, 0, None, None, None) == 1
    assert b"multiple of 64" in lib.sb_last_error()
    assert lib.sb_sdd(one, one, one, one, one, one, 4, 128, 128, 2, 1, 1, 0, None, None, None) == 1
    assert b"multiple of 256" in lib.sb_last_error()
    assert lib.sb_dsd(one, 4, one, 256, 100, one, one, 2, 128, 0, None, one, None, 0, None, None) == 1
    assert b"multiple of 128" in lib.sb_last_error()
    assert lib.sb_dsd(one, 4, one, 256, 128, one, one, 2, 32, 0, None, one, None, 0, None, None) == 1
    assert b"64 or 128" in lib.sb_last_error()
    assert lib.sb_combine(one, one, one, 0, one, 4, 2, 12, None) == 1
    assert b"multiple of 8" in lib.sb_last_error()
