"""The allocation-free forward entry point (rbf_b200_fwd_static) against the regular one.

Some callers of the library cannot allocate device memory at call time (an engine plug-in that must not allocate
after start-up, a latency-critical loop that cannot afford cudaMalloc's synchronisation, a bare FFI caller without
an allocator). They use the variant whose scratch is a fixed array inside the library. This file checks, through
the C ABI, that it gives the regular entry point's results on two calls in a row that share that array, and that
it refuses problems the array cannot hold. It sorts last so that a failure here cannot hide other tests.
"""

import ctypes
import math

import pytest
import torch

from rbf_attention_b200 import _lib

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


def _s3(t):
    return (ctypes.c_int64 * 3)(*t.stride()[:3])


def _regular(lib, q, k, v, causal, softmax):
    B, H, N, D = q.shape
    out = torch.empty_like(q)
    lse = torch.empty((B, H, N), dtype=torch.float32, device=q.device)
    nbytes = lib.rbf_b200_workspace_bytes(B, H, N, D, int(softmax), 0)
    ws = torch.empty(nbytes, dtype=torch.uint8, device=q.device)
    rc = lib.rbf_b200_fwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), lse.data_ptr(), ws.data_ptr(), nbytes,
                          B, H, N, D, _s3(q), _s3(k), _s3(v), _s3(out), 0, int(causal), int(softmax),
                          1.0 / math.sqrt(D), torch.cuda.current_stream().cuda_stream)
    assert rc == 0, lib.rbf_b200_last_error()
    return out, lse


def _static(lib, q, k, v, out, lse, causal, softmax):
    """Outputs are allocated by the caller beforehand; the call itself receives only pointers."""
    B, H, N, D = q.shape
    rc = lib.rbf_b200_fwd_static(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), lse.data_ptr(), B, H, N, D,
                                 _s3(q), _s3(k), _s3(v), _s3(out), 0, int(causal), int(softmax), 1.0 / math.sqrt(D),
                                 torch.cuda.current_stream().cuda_stream)
    return rc


def test_static_scratch_forward_matches_regular_forward_twice_in_a_row():
    lib = _lib.load()
    assert lib.rbf_b200_static_scratch_bytes() == 20 * 1024 * 1024
    g = torch.Generator().manual_seed(17)
    cases = [((2, 3, 700, 64), True, True), ((1, 4, 1028, 128), True, True), ((2, 2, 300, 64), False, False)]
    for shape, causal, softmax in cases:
        std = 1.0 if softmax else 0.5
        # two different problems back to back on one stream: the second must not see anything of the first
        pairs = []
        for _ in range(2):
            q, k, v = ((torch.randn(shape, generator=g) * std).to(DEV, torch.bfloat16) for _ in range(3))
            pairs.append((q, k, v, torch.empty_like(q), torch.empty(shape[:3], dtype=torch.float32, device=DEV)))
        for q, k, v, out, lse in pairs:
            assert _static(lib, q, k, v, out, lse, causal, softmax) == 0, lib.rbf_b200_last_error()
        # workspace = NULL names the built-in scratch of the current device: the status word both calls left there
        code = ctypes.c_uint(1)
        assert lib.rbf_b200_read_device_status(None, torch.cuda.current_stream().cuda_stream, ctypes.byref(code)) == 0
        assert code.value == 0
        torch.cuda.synchronize()
        for q, k, v, out, lse in pairs:
            ref_out, ref_lse = _regular(lib, q, k, v, causal, softmax)
            torch.cuda.synchronize()
            # same kernels on the same inputs: the tolerance of the parity tests (relative L2 6e-3) is met exactly
            assert torch.isfinite(out).all()
            err = (out.float() - ref_out.float()).norm() / ref_out.float().norm()
            assert err.item() <= 6e-3, err.item()
            assert torch.equal(out, ref_out)
            if softmax:
                assert torch.equal(lse, ref_lse)


def test_static_scratch_refuses_problems_beyond_its_size():
    lib = _lib.load()
    B, H, N, D = 16, 16, 4096, 64          # 16 * 16 * 4096 rows * 32 bytes = 32 MiB of slabs > 20 MiB
    q = torch.empty((1, 1, 128, D), dtype=torch.bfloat16, device=DEV)   # never dereferenced: the size check comes first
    s = (ctypes.c_int64 * 3)(H * N * D, N * D, D)
    rc = lib.rbf_b200_fwd_static(q.data_ptr(), q.data_ptr(), q.data_ptr(), q.data_ptr(), q.data_ptr(), B, H, N, D,
                                 s, s, s, s, 0, 1, 1, 0.125, None)
    assert rc == 3
    assert b"built-in scratch" in lib.rbf_b200_last_error()
