"""ctypes binding of ``librbf_b200.so`` (the C ABI declared in ``include/rbf_b200.h``).

The library is the only compute path of this package: if it is missing or fails to load, importing
callers get a ``RuntimeError`` - there is no PyTorch or CPU fallback.
"""

from __future__ import annotations

import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "librbf_b200.so")

ABI_VERSION = 3

STATUS_NAMES = {
    0: "ok",
    1: "bad argument",
    2: "bad layout",
    3: "workspace",
    4: "tensor map",
    5: "launch",
    6: "device",
}

# Every symbol include/rbf_b200.h declares, with its ctypes signature.
_c_i64p = ctypes.POINTER(ctypes.c_int64)
SIGNATURES = {
    "rbf_b200_abi_version": (ctypes.c_int, []),
    "rbf_b200_last_error": (ctypes.c_char_p, []),
    "rbf_b200_workspace_bytes": (ctypes.c_size_t, [ctypes.c_int] * 6),
    "rbf_b200_fwd": (
        ctypes.c_int,
        [ctypes.c_void_p] * 6 + [ctypes.c_size_t] + [ctypes.c_int] * 4 + [_c_i64p] * 4
        + [ctypes.c_int] * 3 + [ctypes.c_float, ctypes.c_void_p],
    ),
    "rbf_b200_bwd": (
        ctypes.c_int,
        [ctypes.c_void_p] * 10 + [ctypes.c_size_t] + [ctypes.c_int] * 4 + [_c_i64p] * 8
        + [ctypes.c_int] * 3 + [ctypes.c_float, ctypes.c_void_p],
    ),
    "rbf_b200_fwd_phases": (
        ctypes.c_int,
        [ctypes.c_void_p] * 6 + [ctypes.c_size_t] + [ctypes.c_int] * 4 + [_c_i64p] * 4
        + [ctypes.c_int] * 3 + [ctypes.c_float, ctypes.c_void_p, ctypes.c_int],
    ),
    "rbf_b200_bwd_phases": (
        ctypes.c_int,
        [ctypes.c_void_p] * 10 + [ctypes.c_size_t] + [ctypes.c_int] * 4 + [_c_i64p] * 8
        + [ctypes.c_int] * 3 + [ctypes.c_float, ctypes.c_void_p, ctypes.c_int],
    ),
    "rbf_b200_static_scratch_bytes": (ctypes.c_size_t, []),
    "rbf_b200_fwd_static": (
        ctypes.c_int,
        [ctypes.c_void_p] * 5 + [ctypes.c_int] * 4 + [_c_i64p] * 4 + [ctypes.c_int] * 3
        + [ctypes.c_float, ctypes.c_void_p],
    ),
    "rbf_b200_read_device_status": (
        ctypes.c_int,
        [ctypes.c_void_p, ctypes.c_void_p, ctypes.POINTER(ctypes.c_uint)],
    ),
    "rbf_b200_layer_norm_fwd": (
        ctypes.c_int,
        [ctypes.c_void_p] * 6 + [ctypes.c_int64, ctypes.c_int, ctypes.c_float, ctypes.c_int, ctypes.c_void_p],
    ),
    "rbf_b200_layer_norm_bwd_workspace_bytes": (ctypes.c_size_t, [ctypes.c_int64, ctypes.c_int]),
    "rbf_b200_layer_norm_bwd": (
        ctypes.c_int,
        [ctypes.c_void_p] * 9 + [ctypes.c_size_t, ctypes.c_int64, ctypes.c_int, ctypes.c_int, ctypes.c_void_p],
    ),
    "rbf_b200_add_layer_norm_fwd": (
        ctypes.c_int,
        [ctypes.c_void_p] * 8 + [ctypes.c_int64, ctypes.c_int, ctypes.c_float, ctypes.c_int, ctypes.c_void_p],
    ),
    "rbf_b200_layer_norm_bwd_add": (
        ctypes.c_int,
        [ctypes.c_void_p] * 10 + [ctypes.c_size_t, ctypes.c_int64, ctypes.c_int, ctypes.c_int, ctypes.c_void_p],
    ),
    "rbf_b200_column_sums_workspace_bytes": (ctypes.c_size_t, [ctypes.c_int64, ctypes.c_int]),
    "rbf_b200_column_sums": (
        ctypes.c_int,
        [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int64, ctypes.c_int, ctypes.c_int64,
         ctypes.c_int, ctypes.c_void_p],
    ),
    "rbf_b200_gelu_fwd": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64, ctypes.c_int, ctypes.c_void_p]),
    "rbf_b200_gelu_bwd": (
        ctypes.c_int,
        [ctypes.c_void_p] * 5 + [ctypes.c_size_t, ctypes.c_int64, ctypes.c_int, ctypes.c_int, ctypes.c_void_p],
    ),
    "rbf_b200_cross_entropy": (
        ctypes.c_int,
        [ctypes.c_void_p] * 5 + [ctypes.c_int, ctypes.c_int, ctypes.c_int64, ctypes.c_int64, ctypes.c_int64, ctypes.c_int,
                                 ctypes.c_void_p],
    ),
    "rbf_b200_scale_unless_one": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64, ctypes.c_int,
                                                 ctypes.c_void_p]),
    "rbf_b200_post_device_status": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]),
    "rbf_b200_qkv_prep": (
        ctypes.c_int,
        [ctypes.c_void_p] * 3 + [ctypes.c_int] + [ctypes.c_void_p] * 3 + [_c_i64p] * 2 + [ctypes.c_void_p, ctypes.c_size_t]
        + [ctypes.c_int] * 7 + [ctypes.c_float, ctypes.c_void_p],
    ),
    "rbf_b200_qkv_prep_bwd_workspace_bytes": (ctypes.c_size_t, [ctypes.c_int] * 5),
    "rbf_b200_qkv_prep_bwd": (
        ctypes.c_int,
        [ctypes.c_void_p] * 2 + [_c_i64p] * 2 + [ctypes.c_void_p] * 4 + [ctypes.c_size_t] + [ctypes.c_int] * 6
        + [ctypes.c_void_p],
    ),
    "rbf_b200_xsa_fwd": (ctypes.c_int, [ctypes.c_void_p] * 3 + [_c_i64p] * 3 + [ctypes.c_int] * 5 + [ctypes.c_void_p]),
    "rbf_b200_xsa_bwd": (ctypes.c_int, [ctypes.c_void_p] * 5 + [_c_i64p] * 5 + [ctypes.c_int] * 5 + [ctypes.c_void_p]),
    "rbf_b200_set_deterministic": (ctypes.c_int, [ctypes.c_int]),
    "rbf_b200_get_deterministic": (ctypes.c_int, []),
    "rbf_b200_selftest_wait_timeout": (
        ctypes.c_int,
        [ctypes.c_void_p, ctypes.c_size_t, ctypes.c_longlong, ctypes.c_void_p],
    ),
}

_lib = None


def load() -> ctypes.CDLL:
    """Loads the shared library once and attaches the signatures. Raises if it is not built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python -m rbf_attention_b200.build` "
            "(this package has no fallback path)"
        )
    lib = ctypes.CDLL(LIB_PATH)
    for name, (restype, argtypes) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError here means header and library disagree
        fn.restype = restype
        fn.argtypes = argtypes
    got = lib.rbf_b200_abi_version()
    if got != ABI_VERSION:
        raise RuntimeError(f"librbf_b200.so has ABI version {got}, this package expects {ABI_VERSION}")
    _lib = lib
    return lib


def strides3(t) -> ctypes.Array:
    """Element strides of dims (b, h, n) of a (B, H, N, D) tensor as an int64[3]."""
    s = t.stride()
    return (ctypes.c_int64 * 3)(s[0], s[1], s[2])


def check(rc: int, what: str) -> None:
    """Turns a non-zero status into the exception type a caller of the reference would see."""
    if rc == 0:
        return
    msg = load().rbf_b200_last_error().decode()
    text = f"{what}: {STATUS_NAMES.get(rc, rc)}: {msg}"
    if rc in (1, 2):
        raise ValueError(text)
    raise RuntimeError(text)
