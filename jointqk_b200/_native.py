"""ctypes binding of ``libjointqk_b200.so`` (declared in ``include/jointqk_b200.h``).

The library is the only implementation of the hot path.  If it cannot be loaded the import
of this module raises; nothing falls back to torch or to the CPU.
"""

from __future__ import annotations

import ctypes as C
from pathlib import Path

from . import build as _build

_c_i32p = C.POINTER(C.c_int32)


class JqkHeadTables(C.Structure):
    """Mirror of ``struct jqk_head_tables``."""

    _fields_ = [
        ("n_heads", C.c_int32),
        ("d", C.c_int32),
        ("words_per_record", C.c_int32),
        ("n_wide", C.c_int32),
        ("desc", C.c_void_p),
        ("col_meta", C.c_void_p),
        ("table_fields", C.c_void_p),
        ("fwd_cols", C.c_void_p),
        ("thresholds", C.c_void_p),
        ("cb_cols", C.c_void_p),
        ("qproj_cols", C.c_void_p),
        ("inv_rows", C.c_void_p),
        ("fwd_limbs", C.c_void_p),
        ("unit_pre", C.c_void_p),
        ("center", C.c_void_p),
        ("center_cols", C.c_void_p),
        ("unit_thr", C.c_float * 64),
        ("unit_aff", C.c_float * 2),
        ("wide_thr", C.c_void_p),
        ("wide_cb", C.c_void_p),
        ("unit_wide_thr", C.c_void_p),
        ("decodable", C.c_int32),
        ("value_decodable", C.c_int32),
    ]


# name -> (restype, argtypes); this table is also what the symbol-export test checks.
SIGNATURES = {
    "jqk_version": (C.c_int32, []),
    "jqk_head_tables_bytes": (C.c_size_t, []),
    "jqk_last_error": (C.c_char_p, []),
    "jqk_compress_paged": (C.c_int32, [
        C.POINTER(JqkHeadTables), C.c_void_p, C.c_int32, C.c_int64, C.c_int64, C.c_int64, C.c_int32,
        C.c_void_p, C.c_void_p, C.c_int32, C.c_void_p, C.c_int32, C.c_int32, C.c_void_p, C.c_void_p,
        C.c_void_p]),
    "jqk_decompress_paged": (C.c_int32, [
        C.POINTER(JqkHeadTables), C.c_int32, C.c_void_p, C.c_void_p, C.c_int32, C.c_void_p, C.c_int32, C.c_int32,
        C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]),
    "jqk_unpack_codes": (C.c_int32, [
        C.POINTER(JqkHeadTables), C.c_int32, C.c_void_p, C.c_int32, C.c_void_p, C.c_int32, C.c_int32,
        C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]),
    "jqk_score_paged": (C.c_int32, [
        C.POINTER(JqkHeadTables), C.c_int32, C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_void_p,
        C.c_int32, C.c_void_p, C.c_int32, C.c_int32, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]),
    "jqk_decode_workspace_bytes": (C.c_size_t, [C.c_int32, C.c_int32, C.c_int32, C.c_int32]),
    "jqk_decode_default_split": (C.c_int32, [C.c_int32, C.c_int32, C.c_int32, C.c_int32]),
    "jqk_decode_split_for_lengths": (C.c_int32, [C.c_void_p, C.c_int32, C.c_int32, C.c_int32]),
    "jqk_decode_attend": (C.c_int32, [
        C.POINTER(JqkHeadTables), C.c_void_p, C.c_int32, C.c_int32, C.c_void_p, C.c_int32, C.c_int32,
        C.c_void_p, C.c_int32, C.c_int32, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_void_p,
        C.c_size_t, C.c_void_p, C.c_void_p]),
    "jqk_decode_attend_packed_values": (C.c_int32, [
        C.POINTER(JqkHeadTables), C.POINTER(JqkHeadTables), C.c_void_p, C.c_int32, C.c_int32, C.c_void_p, C.c_int32,
        C.c_int32, C.c_void_p, C.c_int32, C.c_int32, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_void_p,
        C.c_size_t, C.c_void_p, C.c_void_p]),
    "jqk_decode_append_attend": (C.c_int32, [
        C.POINTER(JqkHeadTables), C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_int64, C.c_int64, C.c_int64,
        C.c_int64, C.c_int32, C.c_int32, C.c_void_p, C.c_int32, C.c_int32, C.c_void_p, C.c_int32, C.c_int32,
        C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_void_p, C.c_size_t, C.c_void_p, C.c_void_p]),
    "jqk_decode_append_attend_packed_values": (C.c_int32, [
        C.POINTER(JqkHeadTables), C.POINTER(JqkHeadTables), C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_int32,
        C.c_int64, C.c_int64, C.c_int64, C.c_int64, C.c_int32, C.c_int32, C.c_void_p, C.c_int32, C.c_int32, C.c_void_p,
        C.c_int32, C.c_int32, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_void_p, C.c_size_t,
        C.c_void_p, C.c_void_p]),
    "jqk_decode_attend_static": (C.c_int32, [
        C.POINTER(JqkHeadTables), C.c_void_p, C.c_int32, C.c_int32, C.c_void_p, C.c_int32, C.c_int32,
        C.c_void_p, C.c_int32, C.c_int32, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_void_p,
        C.c_void_p]),
    "jqk_decode_attend_host": (C.c_int32, [
        C.POINTER(JqkHeadTables), C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_void_p, C.c_int32,
        C.c_int32, C.c_void_p, C.c_int32, C.c_int32, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32,
        C.c_void_p, C.c_size_t, C.c_void_p, C.c_void_p]),
    "jqk_moments_workspace_bytes": (C.c_size_t, [C.c_int64, C.c_int32, C.c_int32, C.c_int32]),
    "jqk_moments_accumulate": (C.c_int32, [
        C.c_void_p, C.c_void_p, C.c_int32, C.c_int64, C.c_int64, C.c_int64, C.c_int32, C.c_int32,
        C.c_int32, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_void_p,
        C.c_size_t, C.c_void_p]),
    "jqk_store_values_paged": (C.c_int32, [
        C.c_void_p, C.c_int32, C.c_int64, C.c_int64, C.c_int64, C.c_int32, C.c_int32, C.c_int32, C.c_void_p,
        C.c_void_p, C.c_int32, C.c_void_p, C.c_int32, C.c_int32, C.c_void_p, C.c_void_p, C.c_void_p]),
    "jqk_roundtrip_dense": (C.c_int32, [
        C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_void_p,
        C.c_int32, C.c_int64, C.c_int64, C.c_int64, C.c_void_p, C.c_void_p, C.c_void_p]),
    "jqk_selftest_bounded_wait": (C.c_int32, [C.c_int32, C.c_void_p, C.c_void_p]),
}

DTYPE_F32, DTYPE_BF16, DTYPE_F16 = 0, 1, 2
ABI_VERSION = 2              # JQK_VERSION of include/jointqk_b200.h
STATUS_BAD_PAGE, STATUS_WAIT_EXPIRED, STATUS_BAD_LENGTH = 1, 2, 4


def _load() -> C.CDLL:
    path = Path(_build.LIB_PATH)
    if _build.is_stale():
        try:
            _build.build()
        except Exception as exc:  # no compiler on this machine and no prebuilt library
            if not path.exists():
                raise ImportError(
                    f"jointqk_b200: CUDA library {path} is missing and could not be built ({exc}); "
                    "there is no non-CUDA implementation of this path") from exc
    lib = C.CDLL(str(path))
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError here means the library is out of date
        fn.restype = res
        fn.argtypes = args
    # a library built from other sources than this binding would read the tables struct wrongly
    if lib.jqk_version() != ABI_VERSION or lib.jqk_head_tables_bytes() != C.sizeof(JqkHeadTables):
        raise ImportError(
            f"jointqk_b200: {path} has interface version {lib.jqk_version()} and a tables struct of "
            f"{lib.jqk_head_tables_bytes()} bytes; this binding expects {ABI_VERSION} and {C.sizeof(JqkHeadTables)}.  "
            "Rebuild it: python -m jointqk_b200.build --force")
    return lib


lib = _load()


class JqkError(RuntimeError):
    pass


def check(rc: int) -> None:
    """Raise for a non-zero return: ValueError for rejected arguments, JqkError for CUDA errors."""
    if rc == 0:
        return
    msg = (lib.jqk_last_error() or b"").decode("utf-8", "replace")
    if rc < 0:
        raise ValueError(f"jointqk_b200: {msg} (code {rc})")
    raise JqkError(f"jointqk_b200: CUDA error {rc}: {msg}")


def torch_dtype_code(dtype) -> int:
    import torch

    if dtype == torch.float32:
        return DTYPE_F32
    if dtype == torch.bfloat16:
        return DTYPE_BF16
    if dtype == torch.float16:
        return DTYPE_F16
    raise TypeError(f"unsupported dtype {dtype}; expected float32, bfloat16 or float16")
