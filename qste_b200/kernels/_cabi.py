"""ctypes binding of libqste_b200.so (the C ABI declared in include/qste_b200.h).

The library is the only kernel backend this package has.  If it is missing or
fails to load, every kernel call raises: there is no CPU or pure-torch path to
fall back to.
"""

from __future__ import annotations

import ctypes
from pathlib import Path

LIBRARY = Path(__file__).resolve().parent.parent / "libqste_b200.so"

# every symbol include/qste_b200.h declares
SYMBOLS = (
    "qste_b200_abi_version",
    "qste_b200_status_string",
    "qste_b200_last_cuda_error",
    "qste_b200_launch_count",
    "qste_b200_last_forward_kernel",
    "qste_b200_set_reserved_sms",
    "qste_b200_pack_coordinate",
    "qste_b200_pack_affine_rows",
    "qste_b200_pack_bits",
    "qste_b200_apply_bits",
    "qste_b200_unpack_rows",
    "qste_b200_packed_linear_affine_workspace",
    "qste_b200_packed_linear_affine",
    "qste_b200_packed_transpose_workspace",
    "qste_b200_packed_transpose",
    "qste_b200_evidence_from_packed_workspace",
    "qste_b200_evidence_from_packed",
    "qste_b200_linear_backward_evidence_workspace",
    "qste_b200_linear_backward_evidence",
    "qste_b200_linear_backward_workspace",
    "qste_b200_linear_backward",
    "qste_b200_linear_backward_staged",
    "qste_b200_packed_row_inner",
    "qste_b200_packed_embedding",
    "qste_b200_smooth_forward",
    "qste_b200_smooth_backward",
    "qste_b200_coordinate_update_workspace",
    "qste_b200_coordinate_update",
    "qste_b200_coordinate_update_static",
)

STATUS_SHAPE, STATUS_DTYPE, STATUS_UNSUPPORTED = -1, -2, -6

_p = ctypes.c_void_p
_i64 = ctypes.c_int64
_int = ctypes.c_int
_f64 = ctypes.c_double
_size = ctypes.c_size_t

_SIGNATURES = {
    "qste_b200_abi_version": (_int, []),
    "qste_b200_status_string": (ctypes.c_char_p, [_int]),
    "qste_b200_last_cuda_error": (ctypes.c_char_p, []),
    "qste_b200_launch_count": (ctypes.c_ulonglong, []),
    "qste_b200_last_forward_kernel": (ctypes.c_char_p, []),
    "qste_b200_set_reserved_sms": (_int, [_int]),
    "qste_b200_pack_coordinate": (_int, [_p, _i64, _i64, _p, _p]),
    "qste_b200_pack_affine_rows": (_int, [_p, _int, _i64, _i64, _p, _p, _p, _p]),
    "qste_b200_pack_bits": (_int, [_p, _i64, _i64, _p, _p]),
    "qste_b200_apply_bits": (_int, [_p, _int, _p, _i64, _i64, _p, _p]),
    "qste_b200_unpack_rows": (_int, [_p, _i64, _i64, _p, _int, _int, _p]),
    "qste_b200_packed_linear_affine_workspace": (_size, [_i64, _i64, _i64, _int, _int]),
    "qste_b200_packed_linear_affine": (
        _int, [_p, _int, _i64, _p, _p, _p, _i64, _i64, _p, _int, _int, _p, _size, _p]),
    "qste_b200_packed_transpose_workspace": (_size, [_i64, _i64, _i64, _int, _int]),
    "qste_b200_packed_transpose": (
        _int, [_p, _int, _i64, _p, _p, _i64, _i64, _p, _int, _int, _p, _size, _p]),
    "qste_b200_evidence_from_packed_workspace": (_size, [_i64, _i64, _i64, _int, _int]),
    "qste_b200_evidence_from_packed": (
        _int, [_p, _int, _i64, _i64, _p, _p, _i64, _p, _int, _p, _size, _p]),
    "qste_b200_linear_backward_evidence_workspace": (_size, [_i64, _i64, _i64, _int, _int]),
    "qste_b200_linear_backward_evidence": (
        _int, [_p, _int, _i64, _i64, _p, _p, _i64, _p, _p, _p, _p, _p, _int, _p, _size, _p]),
    "qste_b200_linear_backward_workspace": (_size, [_i64, _i64, _i64, _int]),
    "qste_b200_linear_backward": (
        _int, [_p, _int, _i64, _i64, _p, _p, _i64, _p, _p, _p, _int, _p, _p, _p, _p, _size, _p]),
    "qste_b200_linear_backward_staged": (
        _int, [_p, _int, _i64, _i64, _p, _p, _i64, _p, _p, _p, _int, _p, _p, _p, _p, _p, _size, _p]),
    "qste_b200_packed_row_inner": (_int, [_p, _p, _i64, _i64, _p, _p]),
    "qste_b200_packed_embedding": (_int, [_p, _i64, _p, _p, _i64, _i64, _p, _int, _p, _p]),
    "qste_b200_smooth_forward": (_int, [_p, _int, _i64, _i64, _int, _f64, _p, _p, _p, _p]),
    "qste_b200_smooth_backward": (_int, [_p, _int, _p, _p, _i64, _i64, _p, _p]),
    "qste_b200_coordinate_update_workspace": (_size, [_i64, _i64, _i64]),
    "qste_b200_coordinate_update": (
        _int, [_p, _p, _p, _p, _p, _p, _p, _i64, _i64, _f64, _f64, _f64, _f64, _i64, _i64, _i64,
               _p, _p, _p, _p, _size, _p]),
    "qste_b200_coordinate_update_static": (
        _int, [_p, _p, _p, _p, _p, _p, _p, _i64, _i64, _f64, _f64, _f64, _f64, _i64, _i64, _i64,
               _p, _p, _p, _p]),
}

_library = None
_failure: str | None = None


def load():
    """The loaded library.  Raises RuntimeError when it cannot be loaded."""

    global _library, _failure
    if _library is not None:
        return _library
    if _failure is not None:
        raise RuntimeError(_failure)
    if not LIBRARY.exists():
        _failure = (
            f"{LIBRARY} is missing: build it with `python -m qste_b200.csrc.build` "
            "(needs nvcc).  qste_b200 has no other kernel backend."
        )
        raise RuntimeError(_failure)
    try:
        library = ctypes.CDLL(str(LIBRARY))
        for name in SYMBOLS:
            function = getattr(library, name)
            function.restype, function.argtypes = _SIGNATURES[name]
    except (OSError, AttributeError) as error:
        _failure = f"cannot load {LIBRARY}: {error}"
        raise RuntimeError(_failure) from error
    _library = library
    return library


def failure() -> str | None:
    try:
        load()
    except RuntimeError as error:
        return str(error)
    return None


def check(status: int, name: str) -> None:
    if status == 0:
        return
    library = load()
    text = library.qste_b200_status_string(int(status)).decode()
    detail = library.qste_b200_last_cuda_error().decode()
    message = f"qste_b200 {name} failed: {text}" + (f" [{detail}]" if detail and status == -5 else "")
    if status in (STATUS_SHAPE, STATUS_DTYPE):
        raise RuntimeError(message)
    raise RuntimeError(message)
