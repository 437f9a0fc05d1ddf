"""The C-ABI library without a GPU: it loads, exports every symbol the header declares, and rejects bad
arguments before any CUDA work."""

import ctypes
import os
import re

import pytest

from rbf_attention_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "rbf_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(rbf_b200_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol(built_library):
    lib = ctypes.CDLL(built_library)
    names = _declared_symbols()
    assert "rbf_b200_fwd" in names and "rbf_b200_bwd" in names
    for name in names:
        assert hasattr(lib, name), f"{name} declared in include/rbf_b200.h but not exported"
    # and the ctypes table of the package covers the same set
    assert sorted(_lib.SIGNATURES) == names


def test_abi_version_and_workspace_size(built_library):
    lib = _lib.load()
    assert lib.rbf_b200_abi_version() == _lib.ABI_VERSION
    # forward: status block + key-norm bias slabs (32 bytes per padded row) (+ query norms, non-softmax variant)
    # backward: status block + key norms + row statistic (L re-pitched, or query norms) + delta; the single-kernel
    # backward adds two slab arrays and an fp32 (B, H, N, D) dQ accumulator
    rows = 2 * 3 * 256 * 4  # N = 200 pads to 256 rows
    slab = 2 * 3 * 256 * 32
    assert lib.rbf_b200_workspace_bytes(2, 3, 200, 64, 1, 0) == 256 + slab
    assert lib.rbf_b200_workspace_bytes(2, 3, 200, 64, 0, 0) == 256 + slab + rows
    assert lib.rbf_b200_workspace_bytes(2, 3, 200, 64, 1, 1) == 256 + 3 * rows + 2 * slab + 2 * 3 * 200 * 64 * 4
    assert lib.rbf_b200_workspace_bytes(2, 3, 200, 128, 1, 1) == 256 + 3 * rows + 2 * slab + 2 * 3 * 200 * 128 * 4
    assert lib.rbf_b200_workspace_bytes(2, 3, 200, 128, 0, 1) == 256 + 3 * rows + 2 * slab + 2 * 3 * 200 * 128 * 4
    assert lib.rbf_b200_workspace_bytes(2, 3, 200, 64, 0, 1) == 256 + 3 * rows + 2 * slab + 2 * 3 * 200 * 64 * 4
    assert lib.rbf_b200_workspace_bytes(0, 3, 200, 64, 1, 0) == 0


def _call_fwd(lib, *, q=0x1000, B=1, H=1, N=128, D=64, dtype=0, strides=(8192, 8192, 64), ws=0x10000, ws_bytes=1 << 20):
    s = (ctypes.c_int64 * 3)(*strides)
    return lib.rbf_b200_fwd(q, 0x2000, 0x3000, 0x4000, 0x5000, ws, ws_bytes, B, H, N, D, s, s, s, s, dtype, 1, 1,
                            0.125, None)


def test_bad_arguments_are_rejected_before_any_launch(built_library):
    lib = _lib.load()
    assert _call_fwd(lib, D=48) == 1 and b"head dim" in lib.rbf_b200_last_error()
    assert _call_fwd(lib, N=0) == 1
    assert _call_fwd(lib, dtype=7) == 1
    assert _call_fwd(lib, q=0) == 1 and b"q is NULL" in lib.rbf_b200_last_error()
    assert _call_fwd(lib, q=0x1004) == 2 and b"16-byte" in lib.rbf_b200_last_error()
    assert _call_fwd(lib, N=256, strides=(8192, 8192, 60)) == 2      # row stride not a multiple of 8 elements
    assert _call_fwd(lib, N=256, strides=(8192, 8192, 32)) == 2      # rows overlap
    assert _call_fwd(lib, ws=0) == 3
    assert _call_fwd(lib, ws_bytes=16) == 3 and b"needed" in lib.rbf_b200_last_error()
    with pytest.raises(ValueError):
        _lib.check(1, "x")
    with pytest.raises(RuntimeError):
        _lib.check(3, "x")


def test_deterministic_switch_and_selftest_arguments(built_library):
    lib = _lib.load()
    assert lib.rbf_b200_get_deterministic() == 0
    assert lib.rbf_b200_set_deterministic(1) == 0 and lib.rbf_b200_get_deterministic() == 1
    assert lib.rbf_b200_set_deterministic(0) == 1 and lib.rbf_b200_get_deterministic() == 0
    # the wait self-test validates before it launches
    assert lib.rbf_b200_selftest_wait_timeout(None, 256, 1000, None) == 3
    assert lib.rbf_b200_selftest_wait_timeout(0x10000, 64, 1000, None) == 3
    assert lib.rbf_b200_selftest_wait_timeout(0x10000, 256, 0, None) == 1
    assert lib.rbf_b200_selftest_wait_timeout(0x10000, 256, 3_000_000_000, None) == 1
    code = ctypes.c_uint(5)
    assert lib.rbf_b200_read_device_status(0x10000, None, None) == 1


def test_training_step_entries_validate_before_any_launch(built_library):
    """Cross entropy, LayerNorm, column sums and the status post reject bad arguments without touching a device."""
    lib = _lib.load()
    p = 0x10000
    assert lib.rbf_b200_cross_entropy(p, p, p, p, p, -1, 64, 64, 64, -100, 0, None) == 1
    assert lib.rbf_b200_cross_entropy(p, p, p, p, p, 4, 0, 64, 64, -100, 0, None) == 1
    assert lib.rbf_b200_cross_entropy(p, p, p, p, p, 4, 64, 64, 64, -100, 5, None) == 1 and b"dtype" in lib.rbf_b200_last_error()
    assert lib.rbf_b200_cross_entropy(p, p, p, p, p, 4, 64, 32, 64, -100, 0, None) == 1      # pitch < width
    assert lib.rbf_b200_cross_entropy(p, p, p, p, p, 0, 64, 64, 64, -100, 0, None) == 0      # nothing to do
    assert lib.rbf_b200_cross_entropy(None, p, p, p, p, 4, 64, 64, 64, -100, 0, None) == 1
    assert lib.rbf_b200_scale_unless_one(p, p, -1, 0, None) == 1
    assert lib.rbf_b200_scale_unless_one(p, p, 0, 0, None) == 0
    assert lib.rbf_b200_scale_unless_one(None, p, 8, 0, None) == 1
    assert lib.rbf_b200_layer_norm_fwd(p, p, p, p, p, p, 8, 500, 1e-5, 0, None) == 1 and b"cols" in lib.rbf_b200_last_error()
    assert lib.rbf_b200_layer_norm_fwd(p, p, p, p, p, p, 8, 512, 1e-5, 2, None) == 1
    assert lib.rbf_b200_layer_norm_fwd(p, p, p, p, p, p, 0, 512, 1e-5, 0, None) == 0
    assert lib.rbf_b200_layer_norm_fwd(p + 4, p, p, p, p, p, 8, 512, 1e-5, 0, None) == 2
    assert lib.rbf_b200_layer_norm_bwd(p, p, p, p, p, p, None, p, p, 1 << 20, 8, 512, 0, None) == 1
    # the forms that carry the residual connection: the residual and the sum go together; the sum is not y
    assert lib.rbf_b200_add_layer_norm_fwd(p, p, None, p, p, p, p, p, 8, 512, 1e-5, 0, None) == 1
    assert b"both" in lib.rbf_b200_last_error()
    assert lib.rbf_b200_add_layer_norm_fwd(p, None, p, p, p, p, p, p, 8, 512, 1e-5, 0, None) == 1
    assert lib.rbf_b200_add_layer_norm_fwd(p, p, p, p, p, p, p, p, 8, 512, 1e-5, 0, None) == 1
    assert lib.rbf_b200_add_layer_norm_fwd(p, p + 4, p, p, p, p + 32, p, p, 8, 512, 1e-5, 0, None) == 2
    assert lib.rbf_b200_add_layer_norm_fwd(p, p, p, p, p, p + 32, p, p, 0, 512, 1e-5, 0, None) == 0
    assert lib.rbf_b200_layer_norm_bwd_add(p, p, p + 2, p, p, p, p, p, p, p, 1 << 20, 8, 512, 0, None) == 2
    assert lib.rbf_b200_layer_norm_bwd_add(p, p, p, p, p, p, p, None, p, p, 1 << 20, 8, 512, 0, None) == 1
    assert lib.rbf_b200_column_sums(p, p, p, 1 << 20, 8, 12, 16, 0, None) == 1      # width not a multiple of 8
    assert lib.rbf_b200_column_sums(p, p, p, 1 << 20, 8, 16, 12, 0, None) == 2      # pitch
    assert lib.rbf_b200_column_sums(p + 2, p, p, 1 << 20, 8, 16, 16, 0, None) == 2  # alignment
    assert lib.rbf_b200_column_sums(p, None, p, 1 << 20, 8, 16, 16, 0, None) == 1
    assert lib.rbf_b200_post_device_status(None, p, None) == 1
    assert lib.rbf_b200_post_device_status(p, None, None) == 1


def test_gelu_entries_validate_before_any_launch(built_library):
    lib = _lib.load()
    p = 0x10000
    assert lib.rbf_b200_gelu_fwd(p, p, 12, 0, None) == 1            # not a multiple of 8
    assert lib.rbf_b200_gelu_fwd(p, p, 16, 2, None) == 1
    assert lib.rbf_b200_gelu_fwd(p, p + 2, 16, 0, None) == 2
    assert lib.rbf_b200_gelu_fwd(p, p, 0, 0, None) == 0
    assert lib.rbf_b200_gelu_bwd(p, p, p, None, None, 0, 8, 20, 0, None) == 1
    assert lib.rbf_b200_gelu_bwd(None, p, p, None, None, 0, 8, 16, 0, None) == 1
