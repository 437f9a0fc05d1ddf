"""Operator boundary: the four ``rbf_attn_v5`` custom operators of the reference, with the same
schemas, fake kernels and autograd formulas, implemented by calls into ``librbf_b200.so``.

Reference counterparts (paths inside the reference project):
  rbf_attn_v5::scaled_fwd / scaled_bwd            rbf_attention.py:651-842
  rbf_attn_v5::non_softmax_fwd / non_softmax_bwd  rbf_attention.py:1355-1511
  run_triton_rbf / run_triton_non_softmax_rbf     rbf_attention.py:848-853
"""

from __future__ import annotations

import ctypes
import math
import os
import time

import torch

from . import _lib

_DTYPE_CODE = {torch.bfloat16: 0, torch.float16: 1}
_F32_CODE = 2          # forward only: fp32 tensors on TF32 operands, head dim 64


def _validate(name: str, t: torch.Tensor, like: torch.Tensor | None = None) -> None:
    if not isinstance(t, torch.Tensor):
        raise TypeError(f"{name} must be a tensor")
    if t.dim() != 4:
        raise ValueError(f"{name} must have shape (B, H, N, D), got {tuple(t.shape)}")
    if not t.is_cuda:
        raise RuntimeError(f"{name} must be a CUDA tensor: rbf_attention_b200 has no CPU path")
    if like is not None:
        if t.shape != like.shape:
            raise ValueError(f"{name} shape {tuple(t.shape)} differs from q shape {tuple(like.shape)}")
        if t.dtype != like.dtype:
            raise ValueError(f"{name} dtype {t.dtype} differs from q dtype {like.dtype}")
        if t.device != like.device:
            raise ValueError(f"{name} is on {t.device}, q is on {like.device}")


def _tma_ready(t: torch.Tensor) -> torch.Tensor:
    """Returns ``t`` if the TMA engine can address it in place (unit stride on D, 16-byte aligned base,
    strides of dims b, h, n multiples of 16 bytes), else a contiguous copy. The reference assumes
    ``stride(-1) == 1`` without checking (rbf_attention.py:111-138)."""
    B, H, N, D = t.shape
    per16 = 16 // t.element_size()
    ok = t.stride(3) == 1 and t.data_ptr() % 16 == 0
    for ext, s in zip((B, H, N), t.stride()[:3]):
        if ext > 1 and (s <= 0 or s % per16 != 0):
            ok = False
    if N > 1 and t.stride(2) < D:
        ok = False
    return t if ok else t.contiguous()


def _compute_dtype(q: torch.Tensor) -> torch.dtype:
    if q.dtype in _DTYPE_CODE:
        return q.dtype
    if q.dtype == torch.float32:
        # fp32 inputs: the forward at head dims up to 64 runs on TF32 operands (see _forward); everything else - the
        # backward, head dims above 64 - runs with fp16 tensor-core operands (11-bit significand, like the TF32 the
        # reference's Triton path uses for them, rbf_attention.py:183) and fp32 accumulation. There fp16's range
        # limit applies: |x| must stay below 65504, which attention activations do by orders of magnitude.
        return torch.float16
    raise ValueError(f"unsupported dtype {q.dtype} (bfloat16, float16 or float32)")


def _padded_head_dim(D: int) -> int:
    """Head dim the kernels run at: 64 or 128. Other head dims up to 128 run zero-padded to the next of the two, which
    is exact: zero columns add nothing to q.k, to |k|^2 or to |q|^2, and zero value columns give zero output columns
    (the reference pads to the next power of two inside its kernels, rbf_attention.py:661). The softmax scale keeps
    using the caller's D."""
    if D <= 64:
        return 64
    if D <= 128:
        return 128
    raise ValueError(f"head dim {D} is not supported (at most 128)")


def _pad_d(t: torch.Tensor, Dp: int) -> torch.Tensor:
    D = t.shape[-1]
    return t if D == Dp else torch.nn.functional.pad(t, (0, Dp - D))


def _device_index(device: torch.device) -> int:
    return device.index if device.index is not None else torch._C._cuda_getDevice()


def _stream_ptr(device: torch.device) -> int:
    """Raw handle of the current stream of ``device`` (the binding's own call: building a ``torch.cuda.Stream`` object
    for it costs 10 us, a tenth of what a whole operator call takes on the host)."""
    return torch._C._cuda_getCurrentRawStream(_device_index(device))


class _OnDevice:
    """``torch.cuda.device(device)`` that does nothing when ``device`` is already the current one."""

    __slots__ = ("index", "prev")

    def __init__(self, device: torch.device):
        self.index = _device_index(device)
        self.prev = -1

    def __enter__(self):
        cur = torch._C._cuda_getDevice()
        if cur != self.index:
            self.prev = cur
            torch._C._cuda_setDevice(self.index)
        return self

    def __exit__(self, *exc):
        if self.prev >= 0:
            torch._C._cuda_setDevice(self.prev)
        return False


def _workspace(B, H, N, D, softmax, backward, device) -> torch.Tensor:
    lib = _lib.load()
    nbytes = lib.rbf_b200_workspace_bytes(B, H, N, D, int(softmax), int(backward))
    # torch's caching allocator returns 512-byte aligned blocks, which satisfies the 256-byte rule
    return torch.empty(nbytes, dtype=torch.uint8, device=device)


class _StatusMonitor:
    """Surfaces device-side wait timeouts of the operator path without synchronising.

    Every kernel bounds its waits; one that runs out leaves a non-zero status word at the start of the call's
    workspace and the kernels return with incomplete results. After each launch a one-thread kernel on the launch
    stream stores the word into a ring of pinned host slots (a store through the mapped host address: a copy would
    queue on the copy engine behind the caller's own device-to-host transfers and hold the launch stream up for
    their duration); a slot holds -1 until its word has arrived, so no event is needed to see that it has. Later
    calls look at the slots that have been written and raise ``RuntimeError`` for a non-zero one. A timeout is therefore reported by a later operator call or by
    ``check_device_status()``, not by the call that suffered it. ``RBF_B200_SYNC_STATUS=1`` makes every call
    synchronise and check its own status (for debugging). Nothing is recorded while a CUDA graph is being captured.
    """

    SLOTS = 256
    _NOT_YET = -1          # slot value until the posting kernel has run (no status word is 0xffffffff: sites end at 250)

    def __init__(self, device):
        self.device = device
        self.host = torch.zeros(self.SLOTS, dtype=torch.int32).pin_memory()
        self.slots = self.host.numpy()          # same memory: reading a slot costs 0.1 us instead of 3
        self.base = self.host.data_ptr()
        self.what = [""] * self.SLOTS
        self.oldest = 0        # the pending entries are the slots oldest, oldest + 1, ..., next - 1 (mod SLOTS)
        self.next = 0
        self.pending = 0

    def _retire_oldest(self):
        i = self.oldest
        self.oldest = (i + 1) % self.SLOTS
        self.pending -= 1
        code = int(self.slots[i]) & 0xFFFFFFFF
        if code != 0:
            self.slots[i] = 0
            if self.what[i].startswith("range:"):
                raise RuntimeError(
                    f"{self.what[i][6:]}: float32 inputs exceed float16's range (|x| >= 65504) on a path that runs on "
                    "float16 tensor-core operands; its results contain inf / nan. Scale the inputs or use bfloat16"
                )
            raise RuntimeError(
                f"{self.what[i]}: a device-side wait ran out (site {code >> 24}, work unit {code & 0xFFFFFF}); "
                "the results of that call are incomplete"
            )

    def poll(self, wait=False):
        """Checks the entries whose status word has arrived, oldest first (all of them, after waiting for the device,
        when ``wait``)."""
        if wait and self.pending:
            torch.cuda.synchronize(self.device)
        while self.pending:
            if self.slots[self.oldest] == self._NOT_YET:
                if wait:
                    raise RuntimeError(f"{self.what[self.oldest]}: the status word did not arrive")
                break
            self._retire_oldest()

    def record_range_check(self, tensors, what):
        """fp32 tensors narrowed to fp16 operands: records (asynchronously, like the status word) whether the
        conversion overflowed, so that a later call raises instead of inf / nan passing silently."""
        flag = torch.zeros(4, dtype=torch.uint8, device=tensors[0].device)
        bad = tensors[0].new_zeros((), dtype=torch.bool)
        for t in tensors:
            bad = bad | torch.isinf(t).any()
        flag[0] = bad
        self.record(flag, "range:" + what)

    def record(self, ws, what):
        if torch.cuda.is_current_stream_capturing():
            return
        if self.pending == self.SLOTS:          # the ring is full: wait for its oldest entry, and for that one only
            self.poll()
            if self.pending == self.SLOTS:
                # (its kernel was enqueued SLOTS calls ago: the word arrives without any help from this thread. A
                # device-wide synchronisation here would also drain the caller's copy streams.)
                deadline = time.monotonic() + 10.0
                while self.slots[self.oldest] == self._NOT_YET:
                    if time.monotonic() > deadline:
                        torch.cuda.synchronize(self.device)
                        break
                    time.sleep(0)
                self._retire_oldest()
        i = self.next
        self.slots[i] = self._NOT_YET
        _lib.check(_lib.load().rbf_b200_post_device_status(ws.data_ptr(), self.base + 4 * i, _stream_ptr(ws.device)),
                   "rbf_b200_post_device_status")
        self.what[i] = what
        self.next = (i + 1) % self.SLOTS
        self.pending += 1
        if _SYNC_STATUS:
            self.poll(wait=True)


_SYNC_STATUS = os.environ.get("RBF_B200_SYNC_STATUS", "0") not in ("", "0")
_monitors: dict = {}


def _monitor(device) -> _StatusMonitor:
    key = device.index if device.index is not None else torch.cuda.current_device()
    m = _monitors.get(key)
    if m is None:
        m = _monitors[key] = _StatusMonitor(device)
    return m


def check_device_status(device=None) -> None:
    """Waits for every operator call made so far on ``device`` (default: the current one) and raises
    ``RuntimeError`` if one of them ended with a device-side wait that ran out."""
    if device is None:
        device = torch.device("cuda", torch.cuda.current_device())
    _monitor(torch.device(device)).poll(wait=True)


def _forward(q, k, v, is_causal: bool, softmax: bool):
    _validate("q", q)
    _validate("k", k, q)
    _validate("v", v, q)
    B, H, N, D0 = q.shape
    D = _padded_head_dim(D0)
    lib = _lib.load()
    # fp32 tensors at head dim <= 64: TF32 operands, as the reference's Triton path uses for them (fp32's exponent range)
    tf32 = q.dtype == torch.float32 and D == 64
    cdt = torch.float32 if tf32 else _compute_dtype(q)
    code = _F32_CODE if tf32 else _DTYPE_CODE[cdt]
    qc, kc, vc = (_tma_ready(_pad_d(t.to(cdt), D)) for t in (q, k, v))
    out = torch.empty((B, H, N, D), dtype=cdt, device=q.device)
    lse = torch.empty((B, H, N), dtype=torch.float32, device=q.device) if softmax else None
    ws = _workspace(B, H, N, D, softmax, False, q.device)
    mon = _monitor(q.device)
    mon.poll()
    with _OnDevice(q.device):
        rc = lib.rbf_b200_fwd(
            qc.data_ptr(), kc.data_ptr(), vc.data_ptr(), out.data_ptr(),
            lse.data_ptr() if softmax else None, ws.data_ptr(), ws.numel(),
            B, H, N, D, _lib.strides3(qc), _lib.strides3(kc), _lib.strides3(vc), _lib.strides3(out),
            code, int(bool(is_causal)), int(softmax), 1.0 / math.sqrt(D0), _stream_ptr(q.device),
        )
        _lib.check(rc, "rbf_b200_fwd")
        mon.record(ws, "rbf_b200_fwd")
        if q.dtype == torch.float32 and not tf32:
            mon.record_range_check((qc, kc, vc), "rbf_b200_fwd")
    if D != D0:
        out = out[..., :D0].contiguous()
    if cdt != q.dtype:
        out = out.to(q.dtype)
    return out, lse


def _backward(q, k, v, out, lse, dout, is_causal: bool, sm_scale: float, softmax: bool):
    _validate("q", q)
    _validate("k", k, q)
    _validate("v", v, q)
    _validate("dout", dout, q)
    B, H, N, D0 = q.shape
    D = _padded_head_dim(D0)
    lib = _lib.load()
    cdt = _compute_dtype(q)
    qc, kc, vc, doc = (_tma_ready(_pad_d(t.to(cdt), D)) for t in (q, k, v, dout))
    # the non-softmax variant takes the forward output when the caller has it: the single-kernel backward needs it
    have_out = out is not None
    oc = _tma_ready(_pad_d(out.to(cdt), D)) if have_out else None
    dq = torch.empty((B, H, N, D), dtype=cdt, device=q.device)
    dk = torch.empty_like(dq)
    dv = torch.empty_like(dq)
    ws = _workspace(B, H, N, D, softmax, True, q.device)
    z3 = (ctypes.c_int64 * 3)(0, 0, 0)
    mon = _monitor(q.device)
    mon.poll()
    # torch.use_deterministic_algorithms(True) selects the backward whose summation order is fixed
    lib.rbf_b200_set_deterministic(int(torch.are_deterministic_algorithms_enabled()))
    with _OnDevice(q.device):
        rc = lib.rbf_b200_bwd(
            qc.data_ptr(), kc.data_ptr(), vc.data_ptr(),
            oc.data_ptr() if have_out else None, lse.data_ptr() if softmax else None, doc.data_ptr(),
            dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), ws.data_ptr(), ws.numel(),
            B, H, N, D, _lib.strides3(qc), _lib.strides3(kc), _lib.strides3(vc),
            _lib.strides3(oc) if have_out else z3, _lib.strides3(doc),
            _lib.strides3(dq), _lib.strides3(dk), _lib.strides3(dv),
            _DTYPE_CODE[cdt], int(bool(is_causal)), int(softmax), float(sm_scale), _stream_ptr(q.device),
        )
        _lib.check(rc, "rbf_b200_bwd")
        mon.record(ws, "rbf_b200_bwd")
        if q.dtype == torch.float32:
            mon.record_range_check((qc, kc, vc, doc), "rbf_b200_bwd")
    if D != D0:
        dq, dk, dv = (t[..., :D0].contiguous() for t in (dq, dk, dv))
    if cdt != q.dtype:
        dq, dk, dv = dq.to(q.dtype), dk.to(q.dtype), dv.to(q.dtype)
    return dq, dk, dv


# ---------------------------------------------------------------------------------------------
# rbf_attn_v5::scaled_fwd / scaled_bwd  (rbf_attention.py:651-842)
# ---------------------------------------------------------------------------------------------
@torch.library.custom_op("rbf_attn_v5::scaled_fwd", mutates_args=())
def rbf_scaled_fwd(
    q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, is_causal: bool
) -> tuple[torch.Tensor, torch.Tensor]:
    out, lse = _forward(q, k, v, is_causal, softmax=True)
    return out, lse


@rbf_scaled_fwd.register_fake
def _(q, k, v, is_causal):
    B, H, N_CTX, D_HEAD = q.shape
    return (
        torch.empty_like(q, memory_format=torch.contiguous_format),
        torch.empty((B, H, N_CTX), device=q.device, dtype=torch.float32),
    )


@torch.library.custom_op("rbf_attn_v5::scaled_bwd", mutates_args=())
def rbf_scaled_bwd(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    out: torch.Tensor,
    L: torch.Tensor,
    dout: torch.Tensor,
    is_causal: bool,
    sm_scale: float,
) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    return _backward(q, k, v, out, L, dout, is_causal, sm_scale, softmax=True)


@rbf_scaled_bwd.register_fake
def _(q, k, v, out, L, dout, is_causal, sm_scale):
    return (
        torch.empty_like(q, memory_format=torch.contiguous_format),
        torch.empty_like(k, memory_format=torch.contiguous_format),
        torch.empty_like(v, memory_format=torch.contiguous_format),
    )


def _scaled_setup_context(ctx, inputs, output):
    q, k, v, is_causal = inputs
    out, L = output
    ctx.save_for_backward(q, k, v, out, L)
    ctx.is_causal = is_causal
    ctx.sm_scale = 1.0 / math.sqrt(q.shape[-1])


def _scaled_backward(ctx, dout, dL):
    # the gradient of L is ignored, as in the reference (rbf_attention.py:830)
    q, k, v, out, L = ctx.saved_tensors
    dq, dk, dv = torch.ops.rbf_attn_v5.scaled_bwd(q, k, v, out, L, dout, ctx.is_causal, ctx.sm_scale)
    return dq, dk, dv, None


torch.library.register_autograd(
    "rbf_attn_v5::scaled_fwd", _scaled_backward, setup_context=_scaled_setup_context
)


# ---------------------------------------------------------------------------------------------
# rbf_attn_v5::non_softmax_fwd / non_softmax_bwd  (rbf_attention.py:1355-1511)
# ---------------------------------------------------------------------------------------------
@torch.library.custom_op("rbf_attn_v5::non_softmax_fwd", mutates_args=())
def rbf_non_softmax_fwd(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, is_causal: bool) -> torch.Tensor:
    return _forward(q, k, v, is_causal, softmax=False)[0]


@rbf_non_softmax_fwd.register_fake
def _(q, k, v, is_causal):
    return torch.empty_like(q, memory_format=torch.contiguous_format)


@torch.library.custom_op("rbf_attn_v5::non_softmax_bwd", mutates_args=())
def rbf_non_softmax_bwd(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    dout: torch.Tensor,
    is_causal: bool,
    sm_scale: float,
) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    # The reference's operator does not receive the forward output. The single-kernel backward needs it
    # (rowsum_j dS_ij = dO_i . O_i), and recomputing it costs less than the two-kernel backward it saves.
    out = _forward(q, k, v, is_causal, softmax=False)[0]
    return _backward(q, k, v, out, None, dout, is_causal, sm_scale, softmax=False)


@rbf_non_softmax_bwd.register_fake
def _(q, k, v, dout, is_causal, sm_scale):
    return (
        torch.empty_like(q, memory_format=torch.contiguous_format),
        torch.empty_like(k, memory_format=torch.contiguous_format),
        torch.empty_like(v, memory_format=torch.contiguous_format),
    )


# Same backward with the forward output passed in (no counterpart in the reference): what autograd calls, since the
# output is at hand there.
@torch.library.custom_op("rbf_attn_v5::non_softmax_bwd_with_out", mutates_args=())
def rbf_non_softmax_bwd_with_out(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    out: torch.Tensor,
    dout: torch.Tensor,
    is_causal: bool,
    sm_scale: float,
) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    return _backward(q, k, v, out, None, dout, is_causal, sm_scale, softmax=False)


@rbf_non_softmax_bwd_with_out.register_fake
def _(q, k, v, out, dout, is_causal, sm_scale):
    return (
        torch.empty_like(q, memory_format=torch.contiguous_format),
        torch.empty_like(k, memory_format=torch.contiguous_format),
        torch.empty_like(v, memory_format=torch.contiguous_format),
    )


def _non_softmax_setup_context(ctx, inputs, output):
    q, k, v, is_causal = inputs
    ctx.save_for_backward(q, k, v, output)
    ctx.is_causal = is_causal
    ctx.sm_scale = 1.0 / math.sqrt(q.shape[-1])


def _non_softmax_backward(ctx, dout):
    q, k, v, out = ctx.saved_tensors
    dq, dk, dv = torch.ops.rbf_attn_v5.non_softmax_bwd_with_out(q, k, v, out, dout, ctx.is_causal, ctx.sm_scale)
    return dq, dk, dv, None


torch.library.register_autograd(
    "rbf_attn_v5::non_softmax_fwd", _non_softmax_backward, setup_context=_non_softmax_setup_context
)


# ---------------------------------------------------------------------------------------------
# The attention block's RBF branch as one operator: fused q/k preparation (SuSiE positions, register-position rows,
# key norms) + attention, reading and writing the projection layouts in place. Replaces, for the "rbf_triton" and
# "rbf_non_softmax" attention types with SuSiE positions, the torch ops of rbf_attention.py:1659-1688 and :1761
# (split, broadcast adds, concatenation, transpose copy) and their autograd.
# ---------------------------------------------------------------------------------------------
def _bhsd_view(t: torch.Tensor) -> torch.Tensor:
    """(B, S, H, D) memory seen as (B, H, S, D), no copy."""
    return t.permute(0, 2, 1, 3)


@torch.library.custom_op("rbf_attn_b200::susie_block_fwd", mutates_args=())
def susie_block_fwd(
    qkv: torch.Tensor,
    pos_weight: torch.Tensor,
    reg_pos_emb: torch.Tensor | None,
    table: torch.Tensor,
    num_heads: int,
    softmax: bool,
) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """qkv (B, S, 3 H D), pos_weight (H, D/2), reg_pos_emb (H, R, D) or None, table (>= S - R, D) ->
    (out (B, S, H D), L (B, H, S) fp32 [empty when softmax is False], qk (2, B, S, H, D) = the prepared q', k')."""
    if not qkv.is_cuda:
        raise RuntimeError("qkv must be a CUDA tensor: rbf_attention_b200 has no CPU path")
    if qkv.dtype not in _DTYPE_CODE:
        raise ValueError(f"unsupported dtype {qkv.dtype} (bfloat16 or float16)")
    B, S, E3 = qkv.shape
    E = E3 // 3
    H = num_heads
    D = E // H
    R = 0 if reg_pos_emb is None else reg_pos_emb.shape[-2]
    if D not in (64, 128):
        raise ValueError(f"head dim {D} is not supported (64 or 128)")
    lib = _lib.load()
    dev = qkv.device
    qkv = qkv.contiguous()
    params_fp32 = pos_weight.dtype == torch.float32
    if not params_fp32 and pos_weight.dtype != qkv.dtype:
        raise ValueError("pos_weight must be float32 or have the dtype of qkv")
    pw = pos_weight.contiguous()
    rp = None if R == 0 else reg_pos_emb.to(pw.dtype).contiguous()
    table = table.to(device=dev, dtype=torch.float32).contiguous()
    if table.shape[0] < S - R:
        raise ValueError(f"the position table holds {table.shape[0]} rows, {S - R} text positions are needed")
    qk = torch.empty((2, B, S, H, D), dtype=qkv.dtype, device=dev)
    out = torch.empty((B, S, H, D), dtype=qkv.dtype, device=dev)
    lse = torch.empty((B, H, S) if softmax else (0,), dtype=torch.float32, device=dev)
    q, k = _bhsd_view(qk[0]), _bhsd_view(qk[1])
    v = _bhsd_view(qkv.view(B, S, 3, H, D)[:, :, 2])
    o = _bhsd_view(out)
    ws = _workspace(B, H, S, D, softmax, False, dev)
    scale = 1.0 / math.sqrt(D)
    mon = _monitor(dev)
    mon.poll()
    with _OnDevice(dev):
        stream = _stream_ptr(dev)
        rc = lib.rbf_b200_qkv_prep(
            qkv.data_ptr(), pw.data_ptr(), None if rp is None else rp.data_ptr(), int(params_fp32), table.data_ptr(),
            q.data_ptr(), k.data_ptr(), _lib.strides3(q), _lib.strides3(k), ws.data_ptr(), ws.numel(),
            B, S, H, D, R, _DTYPE_CODE[qkv.dtype], int(softmax), scale, stream)
        _lib.check(rc, "rbf_b200_qkv_prep")
        rc = lib.rbf_b200_fwd_phases(
            q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr() if softmax else None,
            ws.data_ptr(), ws.numel(), B, H, S, D, _lib.strides3(q), _lib.strides3(k), _lib.strides3(v),
            _lib.strides3(o), _DTYPE_CODE[qkv.dtype], 1, int(softmax), scale, stream, 2)
        _lib.check(rc, "rbf_b200_fwd")
        mon.record(ws, "rbf_b200_fwd (attention block)")
    return out.view(B, S, E), lse, qk


@susie_block_fwd.register_fake
def _(qkv, pos_weight, reg_pos_emb, table, num_heads, softmax):
    B, S, E3 = qkv.shape
    E = E3 // 3
    D = E // num_heads
    return (
        qkv.new_empty((B, S, E)),
        qkv.new_empty((B, num_heads, S) if softmax else (0,), dtype=torch.float32),
        qkv.new_empty((2, B, S, num_heads, D)),
    )


@torch.library.custom_op("rbf_attn_b200::susie_block_bwd", mutates_args=())
def susie_block_bwd(
    qkv: torch.Tensor,
    qk: torch.Tensor,
    out: torch.Tensor,
    lse: torch.Tensor,
    dout: torch.Tensor,
    table: torch.Tensor,
    num_registers: int,
    softmax: bool,
) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """-> (dqkv (B, S, 3 H D), d_pos_weight (H, D/2) fp32, d_reg_pos_emb (H, R, D) fp32)."""
    _, B, S, H, D = qk.shape
    E = H * D
    R = num_registers
    lib = _lib.load()
    dev = qkv.device
    dt = _DTYPE_CODE[qkv.dtype]
    qkv = qkv.contiguous()
    dout = dout.to(qkv.dtype).contiguous()
    table = table.to(device=dev, dtype=torch.float32).contiguous()
    q, k = _bhsd_view(qk[0]), _bhsd_view(qk[1])
    v = _bhsd_view(qkv.view(B, S, 3, H, D)[:, :, 2])
    o = _bhsd_view(out.view(B, S, H, D))
    do = _bhsd_view(dout.view(B, S, H, D))
    dqkv = torch.empty((B, S, 3, H, D), dtype=qkv.dtype, device=dev)
    dq, dk, dv = (_bhsd_view(dqkv[:, :, i]) for i in range(3))
    d_pw = torch.empty((H, D // 2), dtype=torch.float32, device=dev)
    d_rp = torch.empty((H, R, D), dtype=torch.float32, device=dev)
    ws = _workspace(B, H, S, D, softmax, True, dev)
    nb2 = lib.rbf_b200_qkv_prep_bwd_workspace_bytes(B, S, H, D, R)
    ws2 = torch.empty(nb2, dtype=torch.uint8, device=dev)
    mon = _monitor(dev)
    mon.poll()
    lib.rbf_b200_set_deterministic(int(torch.are_deterministic_algorithms_enabled()))
    with _OnDevice(dev):
        stream = _stream_ptr(dev)
        rc = lib.rbf_b200_bwd(
            q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr() if softmax else None,
            do.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), ws.data_ptr(), ws.numel(), B, H, S, D,
            _lib.strides3(q), _lib.strides3(k), _lib.strides3(v), _lib.strides3(o), _lib.strides3(do),
            _lib.strides3(dq), _lib.strides3(dk), _lib.strides3(dv), dt, 1, int(softmax), 1.0 / math.sqrt(D), stream)
        _lib.check(rc, "rbf_b200_bwd")
        mon.record(ws, "rbf_b200_bwd (attention block)")
        rc = lib.rbf_b200_qkv_prep_bwd(
            dq.data_ptr(), dk.data_ptr(), _lib.strides3(dq), _lib.strides3(dk), table.data_ptr(), d_pw.data_ptr(),
            d_rp.data_ptr() if R > 0 else None, ws2.data_ptr(), nb2, B, S, H, D, R, dt, stream)
        _lib.check(rc, "rbf_b200_qkv_prep_bwd")
    return dqkv.view(B, S, 3 * E), d_pw, d_rp


@susie_block_bwd.register_fake
def _(qkv, qk, out, lse, dout, table, num_registers, softmax):
    _, B, S, H, D = qk.shape
    return (
        qkv.new_empty((B, S, 3 * H * D)),
        qkv.new_empty((H, D // 2), dtype=torch.float32),
        qkv.new_empty((H, num_registers, D), dtype=torch.float32),
    )


def _susie_block_setup_context(ctx, inputs, output):
    qkv, pos_weight, reg_pos_emb, table, num_heads, softmax = inputs
    out, lse, qk = output
    ctx.save_for_backward(qkv, qk, out, lse, table)
    ctx.softmax = softmax
    ctx.num_registers = 0 if reg_pos_emb is None else reg_pos_emb.shape[-2]
    ctx.pw_dtype = pos_weight.dtype
    ctx.rp_dtype = None if reg_pos_emb is None else reg_pos_emb.dtype
    ctx.set_materialize_grads(False)


def _susie_block_backward(ctx, dout, dlse, dqk):
    # only `out` carries a gradient: L and the saved q', k' are by-products (the reference ignores dL too)
    qkv, qk, out, lse, table = ctx.saved_tensors
    if dout is None:
        return None, None, None, None, None, None
    dqkv, d_pw, d_rp = torch.ops.rbf_attn_b200.susie_block_bwd(
        qkv, qk, out, lse, dout, table, ctx.num_registers, ctx.softmax)
    d_rp = None if ctx.rp_dtype is None else d_rp.to(ctx.rp_dtype)
    return dqkv, d_pw.to(ctx.pw_dtype), d_rp, None, None, None


torch.library.register_autograd(
    "rbf_attn_b200::susie_block_fwd", _susie_block_backward, setup_context=_susie_block_setup_context
)


def susie_block_attention(qkv, pos_weight, reg_pos_emb, table, num_heads, softmax=True):
    """Attention of one block from the fused projection output: (B, S, 3 H D) -> (B, S, H D), causal, with the SuSiE
    position term and the register-position rows added to q and k inside the operator."""
    return torch.ops.rbf_attn_b200.susie_block_fwd(qkv, pos_weight, reg_pos_emb, table, num_heads, softmax)[0]


# ---------------------------------------------------------------------------------------------
# Exclusive self attention (the block's apply_xsa option, rbf_attention.py:1757-1759) as one fused pass each way
# ---------------------------------------------------------------------------------------------
@torch.library.custom_op("rbf_attn_b200::xsa_fwd", mutates_args=())
def xsa_fwd(o: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
    """out = o - (o . vh) vh with vh = v / max(|v|, 1e-12), row by row; o, v (B, H, N, D)."""
    _validate("o", o)
    _validate("v", v, o)
    if o.dtype not in _DTYPE_CODE:
        raise ValueError(f"unsupported dtype {o.dtype} (bfloat16 or float16)")
    B, H, N, D = o.shape
    lib = _lib.load()
    oc, vc = _tma_ready(o), _tma_ready(v)
    out = torch.empty((B, H, N, D), dtype=o.dtype, device=o.device)
    with _OnDevice(o.device):
        rc = lib.rbf_b200_xsa_fwd(oc.data_ptr(), vc.data_ptr(), out.data_ptr(), _lib.strides3(oc), _lib.strides3(vc),
                                  _lib.strides3(out), B, H, N, D, _DTYPE_CODE[o.dtype], _stream_ptr(o.device))
    _lib.check(rc, "rbf_b200_xsa_fwd")
    return out


@xsa_fwd.register_fake
def _(o, v):
    return torch.empty_like(o, memory_format=torch.contiguous_format)


@torch.library.custom_op("rbf_attn_b200::xsa_bwd", mutates_args=())
def xsa_bwd(g: torch.Tensor, o: torch.Tensor, v: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    B, H, N, D = o.shape
    lib = _lib.load()
    gc, oc, vc = _tma_ready(g.to(o.dtype)), _tma_ready(o), _tma_ready(v)
    d_o = torch.empty((B, H, N, D), dtype=o.dtype, device=o.device)
    d_v = torch.empty_like(d_o)
    with _OnDevice(o.device):
        rc = lib.rbf_b200_xsa_bwd(gc.data_ptr(), oc.data_ptr(), vc.data_ptr(), d_o.data_ptr(), d_v.data_ptr(),
                                  _lib.strides3(gc), _lib.strides3(oc), _lib.strides3(vc), _lib.strides3(d_o),
                                  _lib.strides3(d_v), B, H, N, D, _DTYPE_CODE[o.dtype], _stream_ptr(o.device))
    _lib.check(rc, "rbf_b200_xsa_bwd")
    return d_o, d_v


@xsa_bwd.register_fake
def _(g, o, v):
    return (torch.empty_like(o, memory_format=torch.contiguous_format),
            torch.empty_like(o, memory_format=torch.contiguous_format))


def _xsa_setup_context(ctx, inputs, output):
    o, v = inputs
    ctx.save_for_backward(o, v)


def _xsa_backward(ctx, g):
    o, v = ctx.saved_tensors
    return torch.ops.rbf_attn_b200.xsa_bwd(g, o, v)


torch.library.register_autograd("rbf_attn_b200::xsa_fwd", _xsa_backward, setup_context=_xsa_setup_context)


def exclusive_self_attention(o, v):
    """Removes from every attention output row its component along the value row of the same position."""
    return torch.ops.rbf_attn_b200.xsa_fwd(o, v)


# ---------------------------------------------------------------------------------------------
# Linear layers whose bias gradient is the library's column sum (nn.Linear in train_rbf_transformer.py:143, 216 and
# rbf_attention.py:1625-1626)
# ---------------------------------------------------------------------------------------------
@torch.library.custom_op("rbf_attn_b200::column_sums", mutates_args=())
def column_sums(x: torch.Tensor) -> torch.Tensor:
    """fp32 sums over the rows of a 16-bit CUDA matrix (rows, cols), cols a multiple of 8."""
    if x.dim() != 2 or not x.is_cuda or x.dtype not in _DTYPE_CODE or x.shape[1] % 8 != 0:
        raise ValueError("column_sums: a 16-bit CUDA matrix whose width is a multiple of 8")
    ok = x.stride(1) == 1 and x.stride(0) >= x.shape[1] and x.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0
    xc = x if ok else x.contiguous()
    rows, cols = xc.shape
    lib = _lib.load()
    out = torch.empty(cols, dtype=torch.float32, device=x.device)
    with _OnDevice(x.device):
        nbytes = lib.rbf_b200_column_sums_workspace_bytes(rows, cols)
        ws = torch.empty(max(nbytes, 16), dtype=torch.uint8, device=x.device)
        rc = lib.rbf_b200_column_sums(xc.data_ptr(), out.data_ptr(), ws.data_ptr(), ws.numel(), rows, cols,
                                      xc.stride(0) if rows > 1 else cols, _DTYPE_CODE[x.dtype], _stream_ptr(x.device))
    _lib.check(rc, "rbf_b200_column_sums")
    return out


@column_sums.register_fake
def _(x):
    return x.new_empty(x.shape[1], dtype=torch.float32)


class _LinearBiasSum(torch.autograd.Function):
    """``F.linear`` whose backward takes the bias gradient from ``column_sums`` (the two GEMMs are PyTorch's)."""

    @staticmethod
    def forward(ctx, x, weight, bias):
        ctx.save_for_backward(x, weight)
        return torch.nn.functional.linear(x, weight, bias)

    @staticmethod
    def backward(ctx, g):
        x, weight = ctx.saved_tensors
        g2 = g.reshape(-1, g.shape[-1])
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            dx = g.matmul(weight)
        if ctx.needs_input_grad[1]:
            dw = g2.t().mm(x.reshape(-1, x.shape[-1]))
        if ctx.needs_input_grad[2]:
            db = torch.ops.rbf_attn_b200.column_sums(g2).to(g.dtype)
        return dx, dw, db


@torch.library.custom_op("rbf_attn_b200::gelu_fwd", mutates_args=())
def gelu_fwd(h: torch.Tensor) -> torch.Tensor:
    """Exact (erf) GELU of a 16-bit CUDA tensor whose element count is a multiple of 8."""
    if not h.is_cuda or h.dtype not in _DTYPE_CODE or h.numel() % 8 != 0:
        raise ValueError("gelu_fwd: a 16-bit CUDA tensor with a multiple of 8 elements")
    hc = h.contiguous()
    out = torch.empty_like(hc)
    with _OnDevice(h.device):
        rc = _lib.load().rbf_b200_gelu_fwd(hc.data_ptr(), out.data_ptr(), hc.numel(), _DTYPE_CODE[h.dtype],
                                           _stream_ptr(h.device))
    _lib.check(rc, "rbf_b200_gelu_fwd")
    return out


@gelu_fwd.register_fake
def _(h):
    return torch.empty_like(h, memory_format=torch.contiguous_format)


@torch.library.custom_op("rbf_attn_b200::gelu_bwd", mutates_args=())
def gelu_bwd(h: torch.Tensor, dy: torch.Tensor, with_bias: bool) -> tuple[torch.Tensor, torch.Tensor]:
    """dh = dy * gelu'(h) for (..., cols) tensors and, with ``with_bias``, its fp32 sum over all leading dims."""
    cols = h.shape[-1]
    hc, gc = h.contiguous(), dy.to(h.dtype).contiguous()
    rows = hc.numel() // cols
    lib = _lib.load()
    dh = torch.empty_like(hc)
    dbias = torch.empty(cols if with_bias else 0, dtype=torch.float32, device=h.device)
    with _OnDevice(h.device):
        nbytes = lib.rbf_b200_column_sums_workspace_bytes(rows, cols) if with_bias else 0
        ws = torch.empty(max(nbytes, 16), dtype=torch.uint8, device=h.device)
        rc = lib.rbf_b200_gelu_bwd(hc.data_ptr(), gc.data_ptr(), dh.data_ptr(), dbias.data_ptr() if with_bias else None,
                                   ws.data_ptr(), ws.numel(), rows, cols, _DTYPE_CODE[h.dtype], _stream_ptr(h.device))
    _lib.check(rc, "rbf_b200_gelu_bwd")
    return dh, dbias


@gelu_bwd.register_fake
def _(h, dy, with_bias):
    return (torch.empty_like(h, memory_format=torch.contiguous_format),
            h.new_empty(h.shape[-1] if with_bias else 0, dtype=torch.float32))


class _LinearGelu(torch.autograd.Function):
    """``gelu(F.linear(x, weight, bias))``: the GEMMs are PyTorch's, the activation and its backward - which also
    yields the bias gradient - are the library's."""

    @staticmethod
    def forward(ctx, x, weight, bias):
        h = torch.nn.functional.linear(x, weight, bias)
        ctx.save_for_backward(x, weight, h)
        return torch.ops.rbf_attn_b200.gelu_fwd(h)

    @staticmethod
    def backward(ctx, g):
        x, weight, h = ctx.saved_tensors
        dh, dbias = torch.ops.rbf_attn_b200.gelu_bwd(h, g, ctx.needs_input_grad[2])
        dh2 = dh.reshape(-1, dh.shape[-1])
        dx = dh.matmul(weight) if ctx.needs_input_grad[0] else None
        dw = dh2.t().mm(x.reshape(-1, x.shape[-1])) if ctx.needs_input_grad[1] else None
        db = dbias.to(g.dtype) if ctx.needs_input_grad[2] else None
        return dx, dw, db


def linear_gelu(module: torch.nn.Linear, x: torch.Tensor) -> torch.Tensor:
    """``F.gelu(module(x))`` (exact form) on the library's kernels for 16-bit CUDA activations; anything else through
    PyTorch."""
    if (x.is_cuda and x.dtype in _DTYPE_CODE and module.bias is not None and module.weight.dtype == x.dtype
            and module.out_features % 8 == 0):
        return _LinearGelu.apply(x, module.weight, module.bias)
    return torch.nn.functional.gelu(module(x))


def linear(module: torch.nn.Linear, x: torch.Tensor) -> torch.Tensor:
    """``module(x)``; for 16-bit CUDA activations and a bias, the bias gradient comes from the library's column-sum
    kernel instead of PyTorch's generic reduction."""
    if (x.is_cuda and x.dtype in _DTYPE_CODE and module.bias is not None and module.weight.dtype == x.dtype
            and module.out_features % 8 == 0 and torch.is_grad_enabled() and module.bias.requires_grad):
        return _LinearBiasSum.apply(x, module.weight, module.bias)
    return module(x)


# ---------------------------------------------------------------------------------------------
# LayerNorm of the language model's blocks (nn.LayerNorm, train_rbf_transformer.py:139-150, 215, 241)
# ---------------------------------------------------------------------------------------------
def layer_norm_supported(x: torch.Tensor, weight, bias) -> bool:
    """16-bit CUDA activations with an affine LayerNorm over 256, 512, 768 or 1024 columns."""
    return (x.is_cuda and x.dtype in _DTYPE_CODE and weight is not None and bias is not None
            and weight.dtype == x.dtype and bias.dtype == x.dtype
            and x.shape[-1] % 256 == 0 and 0 < x.shape[-1] <= 1024)


@torch.library.custom_op("rbf_attn_b200::layer_norm_fwd", mutates_args=())
def layer_norm_fwd(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor,
                   eps: float) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """y = (x - mean) * rstd * weight + bias over the last dim; returns (y, mean, rstd), the statistics in fp32."""
    if not layer_norm_supported(x, weight, bias):
        raise ValueError("layer_norm_fwd: 16-bit CUDA tensors with 256, 512, 768 or 1024 columns")
    cols = x.shape[-1]
    xc = x.contiguous()
    rows = xc.numel() // cols
    y = torch.empty_like(xc)
    mean = torch.empty(rows, dtype=torch.float32, device=x.device)
    rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
    wc, bc = weight.contiguous(), bias.contiguous()
    with _OnDevice(x.device):
        rc = _lib.load().rbf_b200_layer_norm_fwd(xc.data_ptr(), wc.data_ptr(), bc.data_ptr(), y.data_ptr(),
                                                 mean.data_ptr(), rstd.data_ptr(), rows, cols, float(eps),
                                                 _DTYPE_CODE[x.dtype], _stream_ptr(x.device))
    _lib.check(rc, "rbf_b200_layer_norm_fwd")
    return y, mean, rstd


@layer_norm_fwd.register_fake
def _(x, weight, bias, eps):
    rows = x.numel() // x.shape[-1]
    return (torch.empty_like(x, memory_format=torch.contiguous_format), x.new_empty(rows, dtype=torch.float32),
            x.new_empty(rows, dtype=torch.float32))


@torch.library.custom_op("rbf_attn_b200::layer_norm_bwd", mutates_args=())
def layer_norm_bwd(x: torch.Tensor, dy: torch.Tensor, weight: torch.Tensor, mean: torch.Tensor,
                   rstd: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    cols = x.shape[-1]
    xc, dyc, wc = x.contiguous(), dy.to(x.dtype).contiguous(), weight.contiguous()
    rows = xc.numel() // cols
    lib = _lib.load()
    dx = torch.empty_like(xc)
    dgamma = torch.empty(cols, dtype=torch.float32, device=x.device)
    dbeta = torch.empty(cols, dtype=torch.float32, device=x.device)
    with _OnDevice(x.device):
        nbytes = lib.rbf_b200_layer_norm_bwd_workspace_bytes(rows, cols)
        ws = torch.empty(max(nbytes, 16), dtype=torch.uint8, device=x.device)
        rc = lib.rbf_b200_layer_norm_bwd(xc.data_ptr(), dyc.data_ptr(), wc.data_ptr(), mean.data_ptr(), rstd.data_ptr(),
                                         dx.data_ptr(), dgamma.data_ptr(), dbeta.data_ptr(), ws.data_ptr(), ws.numel(),
                                         rows, cols, _DTYPE_CODE[x.dtype], _stream_ptr(x.device))
    _lib.check(rc, "rbf_b200_layer_norm_bwd")
    return dx, dgamma.to(weight.dtype), dbeta.to(weight.dtype)


@layer_norm_bwd.register_fake
def _(x, dy, weight, mean, rstd):
    return (torch.empty_like(x, memory_format=torch.contiguous_format), torch.empty_like(weight),
            torch.empty_like(weight))


def _ln_setup_context(ctx, inputs, output):
    x, weight, _bias, _eps = inputs
    ctx.save_for_backward(x, weight, output[1], output[2])
    ctx.set_materialize_grads(False)


def _ln_backward(ctx, g_y, _g_mean, _g_rstd):
    if g_y is None:
        return None, None, None, None
    x, weight, mean, rstd = ctx.saved_tensors
    dx, dgamma, dbeta = torch.ops.rbf_attn_b200.layer_norm_bwd(x, g_y, weight, mean, rstd)
    return dx, dgamma, dbeta, None


torch.library.register_autograd("rbf_attn_b200::layer_norm_fwd", _ln_backward, setup_context=_ln_setup_context)


def layer_norm(x, weight, bias, eps: float = 1e-5):
    """``F.layer_norm(x, (x.shape[-1],), weight, bias, eps)`` on the library's kernels (see layer_norm_supported)."""
    return torch.ops.rbf_attn_b200.layer_norm_fwd(x, weight, bias, eps)[0]


@torch.library.custom_op("rbf_attn_b200::add_layer_norm_fwd", mutates_args=())
def add_layer_norm_fwd(x: torch.Tensor, residual: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor,
                       eps: float) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    """s = x + residual (rounded to the dtype, as the separate addition leaves it) and y = LayerNorm(s) from one pass;
    returns (s, y, mean, rstd)."""
    if not layer_norm_supported(x, weight, bias):
        raise ValueError("add_layer_norm_fwd: 16-bit CUDA tensors with 256, 512, 768 or 1024 columns")
    if residual.shape != x.shape or residual.dtype != x.dtype or residual.device != x.device:
        raise ValueError(f"residual must have the shape, dtype and device of x: {tuple(residual.shape)} {residual.dtype} "
                         f"against {tuple(x.shape)} {x.dtype}")
    cols = x.shape[-1]
    xc, rc_ = x.contiguous(), residual.contiguous()
    rows = xc.numel() // cols
    s, y = torch.empty_like(xc), torch.empty_like(xc)
    mean = torch.empty(rows, dtype=torch.float32, device=x.device)
    rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
    wc, bc = weight.contiguous(), bias.contiguous()
    with _OnDevice(x.device):
        rc = _lib.load().rbf_b200_add_layer_norm_fwd(xc.data_ptr(), rc_.data_ptr(), s.data_ptr(), wc.data_ptr(),
                                                     bc.data_ptr(), y.data_ptr(), mean.data_ptr(), rstd.data_ptr(), rows,
                                                     cols, float(eps), _DTYPE_CODE[x.dtype], _stream_ptr(x.device))
    _lib.check(rc, "rbf_b200_add_layer_norm_fwd")
    return s, y, mean, rstd


@add_layer_norm_fwd.register_fake
def _(x, residual, weight, bias, eps):
    rows = x.numel() // x.shape[-1]
    return (torch.empty_like(x, memory_format=torch.contiguous_format),
            torch.empty_like(x, memory_format=torch.contiguous_format), x.new_empty(rows, dtype=torch.float32),
            x.new_empty(rows, dtype=torch.float32))


@torch.library.custom_op("rbf_attn_b200::layer_norm_bwd_add", mutates_args=())
def layer_norm_bwd_add(x: torch.Tensor, dy: torch.Tensor, dres: torch.Tensor, weight: torch.Tensor, mean: torch.Tensor,
                       rstd: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """The LayerNorm backward with ``dres`` (the gradient reaching x along the skip path) added to dx before the
    rounding: (dx, dgamma, dbeta)."""
    cols = x.shape[-1]
    xc, dyc, wc = x.contiguous(), dy.to(x.dtype).contiguous(), weight.contiguous()
    drc = dres.to(x.dtype).contiguous()
    if drc.shape != xc.shape:
        raise ValueError(f"dres must have the shape of x: {tuple(dres.shape)} against {tuple(x.shape)}")
    rows = xc.numel() // cols
    lib = _lib.load()
    dx = torch.empty_like(xc)
    dgamma = torch.empty(cols, dtype=torch.float32, device=x.device)
    dbeta = torch.empty(cols, dtype=torch.float32, device=x.device)
    with _OnDevice(x.device):
        nbytes = lib.rbf_b200_layer_norm_bwd_workspace_bytes(rows, cols)
        ws = torch.empty(max(nbytes, 16), dtype=torch.uint8, device=x.device)
        rc = lib.rbf_b200_layer_norm_bwd_add(xc.data_ptr(), dyc.data_ptr(), drc.data_ptr(), wc.data_ptr(), mean.data_ptr(),
                                             rstd.data_ptr(), dx.data_ptr(), dgamma.data_ptr(), dbeta.data_ptr(),
                                             ws.data_ptr(), ws.numel(), rows, cols, _DTYPE_CODE[x.dtype],
                                             _stream_ptr(x.device))
    _lib.check(rc, "rbf_b200_layer_norm_bwd_add")
    return dx, dgamma.to(weight.dtype), dbeta.to(weight.dtype)


@layer_norm_bwd_add.register_fake
def _(x, dy, dres, weight, mean, rstd):
    return (torch.empty_like(x, memory_format=torch.contiguous_format), torch.empty_like(weight),
            torch.empty_like(weight))


def _add_ln_setup_context(ctx, inputs, output):
    _x, _residual, weight, _bias, _eps = inputs
    ctx.save_for_backward(output[0], weight, output[2], output[3])
    ctx.set_materialize_grads(False)


def _add_ln_backward(ctx, g_s, g_y, _g_mean, _g_rstd):
    # the sum has one gradient, shared by x and residual: the LayerNorm's plus whatever reached s from elsewhere
    if g_y is None:
        return g_s, g_s, None, None, None
    s, weight, mean, rstd = ctx.saved_tensors
    if g_s is None:
        dx, dgamma, dbeta = torch.ops.rbf_attn_b200.layer_norm_bwd(s, g_y, weight, mean, rstd)
    else:
        dx, dgamma, dbeta = torch.ops.rbf_attn_b200.layer_norm_bwd_add(s, g_y, g_s, weight, mean, rstd)
    return dx, dx, dgamma, dbeta, None


torch.library.register_autograd("rbf_attn_b200::add_layer_norm_fwd", _add_ln_backward,
                                setup_context=_add_ln_setup_context)


def add_layer_norm(x, residual, weight, bias, eps: float = 1e-5):
    """``s = x + residual; y = F.layer_norm(s, (s.shape[-1],), weight, bias, eps)`` in one pass over the activations
    (and one in the backward, which takes the skip path's gradient with it): returns (s, y)."""
    s, y, _mean, _rstd = torch.ops.rbf_attn_b200.add_layer_norm_fwd(x, residual, weight, bias, eps)
    return s, y


# ---------------------------------------------------------------------------------------------
# Cross entropy of the language-model step (torch.nn.CrossEntropyLoss(ignore_index=-100),
# train_rbf_transformer.py:282): loss and d(loss)/d(logits) from one kernel
# ---------------------------------------------------------------------------------------------
_CE_DTYPE = {torch.bfloat16: 0, torch.float16: 1, torch.float32: 2}


@torch.library.custom_op("rbf_attn_b200::cross_entropy_fwd", mutates_args=())
def cross_entropy_fwd(logits: torch.Tensor, targets: torch.Tensor, ignore_index: int) -> tuple[torch.Tensor, torch.Tensor]:
    """Mean cross entropy over the rows whose target is not ``ignore_index`` (fp32 scalar) and its gradient with
    respect to ``logits`` (same shape and dtype), from one pass: logits (rows, cols) with unit column stride,
    targets (rows,) int64."""
    if logits.dim() != 2 or targets.dim() != 1 or targets.shape[0] != logits.shape[0]:
        raise ValueError(f"logits must be (rows, cols) and targets (rows,), got {tuple(logits.shape)}, {tuple(targets.shape)}")
    if not logits.is_cuda or targets.device != logits.device:
        raise RuntimeError("logits and targets must be CUDA tensors on one device: rbf_attention_b200 has no CPU path")
    if logits.dtype not in _CE_DTYPE:
        raise ValueError(f"unsupported dtype {logits.dtype} (bfloat16, float16 or float32)")
    if targets.dtype != torch.int64:
        raise ValueError(f"targets must be int64, got {targets.dtype}")
    rows, cols = logits.shape
    x = logits if logits.stride(1) == 1 and (rows <= 1 or logits.stride(0) >= cols) else logits.contiguous()
    t = targets.contiguous()
    counted = ((t != ignore_index) & (t >= 0) & (t < cols)).sum()
    grad_scale = 1.0 / counted.to(torch.float32)          # no counted row: inf * 0 = nan, as torch's mean of nothing
    loss_rows = torch.empty(rows, dtype=torch.float32, device=x.device)
    dlogits = torch.empty((rows, cols), dtype=x.dtype, device=x.device)
    with _OnDevice(x.device):
        rc = _lib.load().rbf_b200_cross_entropy(
            x.data_ptr(), t.data_ptr(), grad_scale.data_ptr(), loss_rows.data_ptr(), dlogits.data_ptr(), rows, cols,
            x.stride(0) if rows > 1 else cols, cols, int(ignore_index), _CE_DTYPE[x.dtype], _stream_ptr(x.device))
    _lib.check(rc, "rbf_b200_cross_entropy")
    return loss_rows.sum() * grad_scale, dlogits


@cross_entropy_fwd.register_fake
def _(logits, targets, ignore_index):
    return logits.new_empty((), dtype=torch.float32), torch.empty_like(logits, memory_format=torch.contiguous_format)


@torch.library.custom_op("rbf_attn_b200::scale_unless_one_", mutates_args=("x",))
def scale_unless_one_(x: torch.Tensor, factor: torch.Tensor) -> None:
    """x *= factor (a one-element tensor) unless factor == 1, decided on the device."""
    if not x.is_contiguous():
        raise ValueError("x must be contiguous")
    f = factor.reshape(1).to(device=x.device, dtype=torch.float32)
    with _OnDevice(x.device):
        rc = _lib.load().rbf_b200_scale_unless_one(x.data_ptr(), f.data_ptr(), x.numel(), _CE_DTYPE[x.dtype],
                                                   _stream_ptr(x.device))
    _lib.check(rc, "rbf_b200_scale_unless_one")


def _ce_setup_context(ctx, inputs, output):
    ctx.save_for_backward(output[1])
    ctx.set_materialize_grads(False)        # no zero tensor of the logits' size for the unused second output


def _ce_backward(ctx, g_loss, _g_dlogits):
    # the gradient was formed by the forward; it is scaled in place (a no-op for the usual g_loss = 1), so a graph
    # retained for a second backward pass with g_loss != 1 would see it scaled twice
    if g_loss is None:
        return None, None, None
    (dlogits,) = ctx.saved_tensors
    torch.ops.rbf_attn_b200.scale_unless_one_(dlogits, g_loss)
    return dlogits, None, None


torch.library.register_autograd("rbf_attn_b200::cross_entropy_fwd", _ce_backward, setup_context=_ce_setup_context)


def cross_entropy(logits, targets, ignore_index: int = -100):
    """``F.cross_entropy(logits, targets, ignore_index=ignore_index)`` (mean reduction) for 2-D CUDA logits, with the
    gradient produced by the forward kernel."""
    return torch.ops.rbf_attn_b200.cross_entropy_fwd(logits, targets, ignore_index)[0]


# ---------------------------------------------------------------------------------------------
# Wrappers with the reference's names (rbf_attention.py:848-853)
# ---------------------------------------------------------------------------------------------
def run_triton_rbf(q, k, v, is_causal=True):
    """Softmax RBF attention. The name is the reference's; nothing here uses Triton."""
    return torch.ops.rbf_attn_v5.scaled_fwd(q, k, v, is_causal)[0]


def run_triton_non_softmax_rbf(q, k, v, is_causal=True):
    """Non-softmax RBF attention ``exp(-g|q-k|^2) V``. The name is the reference's."""
    return torch.ops.rbf_attn_v5.non_softmax_fwd(q, k, v, is_causal)
