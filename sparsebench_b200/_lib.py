"""ctypes binding of the C ABI declared in include/sparsebench_b200.h.

There is no fallback: if the library is missing or a symbol is absent, loading raises. The
library is only built on demand on a machine that has nvcc and no GPU work pending; on a GPU box
the prebuilt file next to this module is used.
"""

from __future__ import annotations

import ctypes
import os
from ctypes import c_char_p, c_int, c_int32, c_int64, c_size_t, c_void_p
from pathlib import Path

from sparsebench_b200 import _build

_P = c_void_p

# name -> (restype, argtypes), in the order of the header.
SIGNATURES: dict[str, tuple[object, list[object]]] = {
    "sb_last_error": (c_char_p, []),
    "sb_status_string": (c_char_p, [c_int]),
    "sb_version": (c_char_p, []),
    "sb_arch_probe": (c_int, [_P, c_int64, _P]),
    "sb_route_sizes": (c_int, [c_int64, c_int32, c_int64, c_int64, _P, _P, _P]),
    "sb_route_workspace_bytes": (c_size_t, [c_int64, c_int32]),
    "sb_route": (c_int, [_P, c_int, c_int64, c_int32, c_int32, c_int32, c_int32, c_int32,
                         _P, _P, _P, _P, _P, _P, _P, _P, _P, _P]),
    "sb_route_static_scratch": (c_int, [_P, c_int, c_int64, c_int32, c_int32, c_int32, c_int32, c_int32,
                                        _P, _P, _P, _P, _P, _P, _P, _P, _P]),
    "sb_sdd": (c_int, [_P, _P, _P, _P, _P, _P, c_int64, c_int32, c_int32, c_int32, c_int32, c_int, c_int, _P, _P, _P]),
    "sb_gemm_pair_clusters": (c_int, []),
    "sb_dsd": (c_int, [_P, c_int64, _P, c_int64, c_int32, _P, _P, c_int32, c_int32, c_int, _P, _P, _P, c_int32, _P, _P]),
    "sb_combine": (c_int, [_P, _P, _P, c_int, _P, c_int64, c_int32, c_int32, _P]),
    "sb_router_topk": (c_int, [_P, c_int, c_int64, c_int32, c_int32, _P, c_int, _P, _P]),
    "sb_route_from_logits_fused": (c_int, [c_int64, c_int32, c_int32]),
    "sb_route_from_logits": (c_int, [_P, c_int, c_int64, c_int32, c_int32, c_int32, c_int32, c_int32, _P, _P,
                                     _P, _P, _P, _P, _P, _P, _P, _P, _P]),
    "sb_remap_rows": (c_int, [_P, _P, c_int, _P, c_int64, c_int64, c_int64, _P]),
    "sb_combine_assigned": (c_int, [_P, _P, _P, c_int, _P, c_int, _P, _P, c_int64, c_int64, c_int32, _P]),
    "sb_token_rounding_capacity": (c_int64, [c_int64, c_int32, c_int32, c_int32]),
    "sb_token_rounding_workspace_bytes": (c_size_t, [c_int64, c_int32, c_int32]),
    "sb_token_rounding": (c_int, [_P, c_int64, c_int32, c_int32, c_int32, _P, _P, _P, _P, _P, _P]),
    "sb_ep_plan": (c_int, [_P, _P, _P, c_int64, c_int32, c_int32, c_int32, _P, _P, _P, _P]),
    "sb_ep_slot_experts": (c_int, [_P, c_int32, c_int32, c_int32, _P, _P]),
    "sb_gather_rows": (c_int, [_P, _P, _P, c_int64, c_int32, _P]),
    "sb_ep_push_rows": (c_int, [_P, _P, _P, c_int32, c_int32, c_int32, c_int32, _P]),
    "sb_ep_push_counts": (c_int, [_P, _P, c_int32, c_int32, c_int32, _P]),
    "sb_ep_barrier": (c_int, [_P, _P, _P, c_int32, c_int32, _P, _P]),
    "sb_ep_dispatch_segments": (c_int32, [c_int32]),
    "sb_ep_dispatch_schedule_ints": (c_int64, [c_int64]),
    "sb_ep_owner_layout": (c_int, [_P, c_int32, c_int32, c_int32, c_int32, c_int32, c_int32,
                                   _P, _P, _P, _P, _P, _P, _P, _P, _P, _P]),
    "sb_ep_push_rows_flagged": (c_int, [_P, _P, _P, _P, _P, _P, _P, c_int32, c_int32, c_int32, c_int32, c_int32, _P]),
    "sb_ep_sdd_dispatch": (c_int, [_P, _P, _P, _P, _P, _P, c_int32, c_int32, c_int32, _P, _P, _P, _P, _P, _P, _P, _P, _P,
                                   c_int32, c_int32, c_int32, c_int32, c_int32, _P, _P]),
    "sb_ep_dsd_push": (c_int, [_P, c_int64, _P, c_int64, c_int32, _P, _P, c_int32, _P, _P, c_int32, c_int32, c_int32,
                               _P, _P]),
}

_lib: ctypes.CDLL | None = None


class SparseBenchError(RuntimeError):
    """An entry point of libsparsebench_b200 returned a non-zero status."""


def library_path() -> Path:
    """The in-tree build, or the file SPARSEBENCH_B200_LIB names (to try another build of the same ABI)."""
    override = os.environ.get("SPARSEBENCH_B200_LIB")
    return Path(override) if override else _build.LIB_PATH


def load() -> ctypes.CDLL:
    """Loads the library once and declares every prototype. Raises if it cannot."""
    global _lib
    if _lib is not None:
        return _lib
    path = library_path()
    if not path.exists():
        raise RuntimeError(
            f"{path} is missing: build it with `python -m sparsebench_b200._build` (needs nvcc). "
            "This package has no CPU or PyTorch fallback."
        )
    lib = ctypes.CDLL(str(path))
    for name, (restype, argtypes) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if the symbol is missing
        fn.restype = restype
        fn.argtypes = argtypes
    _lib = lib
    return lib


def check(status: int) -> None:
    """Raises SparseBenchError with the library's text if status != 0."""
    if status != 0:
        lib = load()
        text = lib.sb_last_error().decode() or lib.sb_status_string(status).decode()
        raise SparseBenchError(text)
