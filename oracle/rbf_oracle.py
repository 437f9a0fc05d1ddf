"""CPU oracle for RBF attention: TEST INFRASTRUCTURE ONLY.

This file restates, on the CPU, the materialised-matrix math that the reference project uses as
its own ground truth for the fused RBF attention path. Only the test-suite, the smoke check and
the benchmark's CPU-baseline leg may import it; the product (``rbf_attention_b200``) never does.

Parity status: PINNED. ``tests/golden/make_golden.py`` imports the reference's own PyTorch
implementation (``compute_rbf_logits``, the ``rbf_slow`` / ``rbf_non_softmax_slow`` branches of
``CustomCausalAttention`` and ``rbf_math_forward``) and stores its outputs and autograd gradients
as fixtures; ``tests/test_oracle.py`` checks every function below against those fixtures and
against the algebraic identity that ``rbf_math_test.py`` proves (distance form == dot-product form
with a key-norm bias). The reference has no test of its own for the non-softmax variant, so that
variant is pinned by fixtures generated from ``rbf_attention.py:1747-1753`` only.

Reference lines restated here (paths are inside the reference project):
  * logits                 rbf_attention.py:1547-1553  (``compute_rbf_logits``)
  * causal mask            rbf_attention.py:1556-1565  (strict upper triangle masked)
  * softmax variant        rbf_attention.py:1738-1744  (``rbf_slow`` branch)
  * non-softmax variant    rbf_attention.py:1747-1753  (``rbf_non_softmax_slow`` branch)
  * base-2 log-sum-exp L   rbf_attention.py:149-150, 217-219
  * backward formulas      rbf_attention.py:275, 418-447, 612-626 (softmax);
                           rbf_attention.py:1133-1154, 1316-1336 (non-softmax)
"""

from __future__ import annotations

import math
import time

import numpy as np

LOG2E = 1.4426950408889634


# --------------------------------------------------------------------------------------------
# numpy float64 restatement with hand-derived gradients (no autograd involved)
# --------------------------------------------------------------------------------------------
def rbf_logits(q: np.ndarray, k: np.ndarray) -> np.ndarray:
    """-(|q|^2 + |k|^2 - 2 q.k) / sqrt(D)   (rbf_attention.py:1547-1553)."""
    q = q.astype(np.float64)
    k = k.astype(np.float64)
    d = q.shape[-1]
    q_sq = (q * q).sum(-1, keepdims=True)
    k_sq = (k * k).sum(-1)[..., None, :]
    dot = q @ np.swapaxes(k, -1, -2)
    return -(q_sq + k_sq - 2.0 * dot) / math.sqrt(d)


def _causal_keep(n: int) -> np.ndarray:
    """True where key index <= query index (rbf_attention.py:187, 1556-1565)."""
    return np.tril(np.ones((n, n), dtype=bool))


def forward(q, k, v, causal: bool = True, softmax: bool = True):
    """Returns (out, L). ``L`` is the base-2 log-sum-exp of the key-norm-biased logits
    ``(2 g q.k - g |k|^2) * log2(e)`` (rbf_attention.py:217-219); ``None`` for the non-softmax variant.
    """
    q64, k64, v64 = (np.asarray(t, dtype=np.float64) for t in (q, k, v))
    n, d = q64.shape[-2], q64.shape[-1]
    gamma = 1.0 / math.sqrt(d)
    logits = rbf_logits(q64, k64)
    if causal:
        logits = np.where(_causal_keep(n), logits, -np.inf)
    if softmax:
        m = logits.max(-1, keepdims=True)
        e = np.exp(logits - m)
        den = e.sum(-1, keepdims=True)
        p = e / den
        # the fused path drops the per-row -g|q|^2 term (softmax is invariant to it): add it back
        q_sq = (q64 * q64).sum(-1)
        L = (m[..., 0] + np.log(den[..., 0]) + gamma * q_sq) * LOG2E
    else:
        p = np.exp(logits)
        L = None
    return p @ v64, L


def backward(q, k, v, dout, causal: bool = True, softmax: bool = True):
    """Hand-derived gradients (dq, dk, dv) in float64.

    softmax:      dV = P^T dO; dP = dO V^T; dS = P*(dP - rowsum(O*dO));
                  dQ = 2g dS K; dK = 2g (dS^T Q - colsum(dS)*K)          (rbf_attention.py:418-447, 612-626)
    non-softmax:  dS = P*dP; dQ = 2g (dS K - rowsum(dS)*Q); dK as above  (rbf_attention.py:1133-1154, 1316-1336)
    """
    q64, k64, v64, do64 = (np.asarray(t, dtype=np.float64) for t in (q, k, v, dout))
    n, d = q64.shape[-2], q64.shape[-1]
    gamma = 1.0 / math.sqrt(d)
    logits = rbf_logits(q64, k64)
    if causal:
        logits = np.where(_causal_keep(n), logits, -np.inf)
    if softmax:
        m = logits.max(-1, keepdims=True)
        e = np.exp(logits - m)
        p = e / e.sum(-1, keepdims=True)
    else:
        p = np.exp(logits)
    out = p @ v64
    dv = np.swapaxes(p, -1, -2) @ do64
    dp = do64 @ np.swapaxes(v64, -1, -2)
    if softmax:
        delta = (out * do64).sum(-1, keepdims=True)
        ds = p * (dp - delta)
        dq = 2.0 * gamma * (ds @ k64)
    else:
        ds = p * dp
        dq = 2.0 * gamma * (ds @ k64 - ds.sum(-1, keepdims=True) * q64)
    dk = 2.0 * gamma * (np.swapaxes(ds, -1, -2) @ q64 - ds.sum(-2)[..., None] * k64)
    return dq, dk, dv


# --------------------------------------------------------------------------------------------
# PyTorch restatement (what the reference itself runs on the CPU); used for cross-checks at sizes
# where float64 numpy is slow, and as the timed CPU baseline.
# --------------------------------------------------------------------------------------------
def torch_logits(q, k):
    """compute_rbf_logits, rbf_attention.py:1547-1553 (fp32 math, cast back to the input dtype)."""
    q_f32, k_f32 = q.float(), k.float()
    q_sq = q_f32.pow(2).sum(dim=-1, keepdim=True)
    k_sq = k_f32.pow(2).sum(dim=-1).unsqueeze(-2)
    dist_sq = q_sq + k_sq - 2.0 * (q_f32 @ k_f32.transpose(-2, -1))
    return (-dist_sq / (q.size(-1) ** 0.5)).to(q.dtype)


def torch_forward(q, k, v, causal: bool = True, softmax: bool = True):
    """rbf_slow (rbf_attention.py:1738-1744) / rbf_non_softmax_slow (:1747-1753) on any dtype."""
    import torch

    logits = torch_logits(q, k)
    if causal:
        n = q.shape[-2]
        mask = torch.ones(n, n, dtype=torch.bool, device=q.device).triu_(1)
        logits = logits.masked_fill(mask, float("-inf"))
    w = torch.softmax(logits, dim=-1) if softmax else torch.exp(logits)
    return w @ v


def torch_forward_backward(q, k, v, dout, causal: bool = True, softmax: bool = True, dtype=None):
    """Forward + autograd backward in ``dtype`` (default: the inputs' dtype). Returns (out, dq, dk, dv)."""
    import torch

    dtype = dtype or q.dtype
    qq, kk, vv = (t.detach().to(dtype).clone().requires_grad_(True) for t in (q, k, v))
    out = torch_forward(qq, kk, vv, causal, softmax)
    out.backward(dout.to(dtype))
    return out.detach(), qq.grad, kk.grad, vv.grad


def torch_lse2(q, k, causal: bool = True):
    """Base-2 LSE of the biased logits, as the fused forward saves it (rbf_attention.py:217-219)."""
    import torch

    d = q.shape[-1]
    c = LOG2E / math.sqrt(d)
    qf, kf = q.double(), k.double()
    s = 2.0 * c * (qf @ kf.transpose(-1, -2)) - c * kf.pow(2).sum(-1).unsqueeze(-2)
    if causal:
        n = q.shape[-2]
        s = s.masked_fill(torch.ones(n, n, dtype=torch.bool).triu_(1), float("-inf"))
    return (torch.logsumexp(s * math.log(2.0), dim=-1) / math.log(2.0)).float()


# --------------------------------------------------------------------------------------------
# Seeded synthetic inputs for the benchmark configurations
# --------------------------------------------------------------------------------------------
def make_inputs(B, H, N, D, *, seed=0, dtype=None, key_norm_sigma=0.0, std=1.0, device="cpu"):
    """Q, K, V, dO ~ N(0, std^2). With ``key_norm_sigma`` > 0 every key row is multiplied by one
    LogNormal(0, sigma) draw so that a few keys have outlier norms. Values are rounded to ``dtype``
    (so that oracle and kernel see identical numbers) and returned in that dtype."""
    import torch

    dtype = dtype or torch.float32
    g = torch.Generator(device="cpu").manual_seed(seed)
    q = torch.randn(B, H, N, D, generator=g) * std
    k = torch.randn(B, H, N, D, generator=g) * std
    v = torch.randn(B, H, N, D, generator=g) * std
    do = torch.randn(B, H, N, D, generator=g)
    if key_norm_sigma > 0:
        s = torch.exp(torch.randn(B, H, N, 1, generator=g) * key_norm_sigma)
        k = k * s
    return tuple(t.to(dtype).to(device) for t in (q, k, v, do))


def time_cpu_forward_backward(B, H, N, D, causal=True, softmax=True, repeats=3, threads=None, seed=0):
    """Times the reference's CPU path (fp32 PyTorch, materialised N x N matrix, autograd backward).
    Returns (seconds per fwd+bwd, threads used)."""
    import os

    import torch

    threads = threads or os.cpu_count() or 1
    torch.set_num_threads(threads)
    q, k, v, do = make_inputs(B, H, N, D, seed=seed)
    torch_forward_backward(q, k, v, do, causal, softmax)  # warm-up
    best = float("inf")
    for _ in range(repeats):
        t0 = time.perf_counter()
        torch_forward_backward(q, k, v, do, causal, softmax)
        best = min(best, time.perf_counter() - t0)
    return best, threads


def error_report(got, ref):
    """max-abs, max-abs relative to max|ref|, and relative L2 error of ``got`` against ``ref``."""
    import torch

    g, r = got.double().cpu(), ref.double().cpu()
    diff = (g - r).abs()
    return {
        "max_abs": diff.max().item(),
        "rel_max": (diff.max() / r.abs().max().clamp_min(1e-30)).item(),
        "rel_l2": ((g - r).norm() / r.norm().clamp_min(1e-30)).item(),
    }
