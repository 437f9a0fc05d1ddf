"""The CPU oracle against the fixtures generated from the reference's own PyTorch code, and against the
algebraic identity the reference's rbf_math_test.py demonstrates. No GPU involved."""

import math
import os

import numpy as np
import pytest
import torch

from oracle import rbf_oracle as oracle


def _load(golden_dir, name):
    return np.load(os.path.join(golden_dir, name))


@pytest.mark.parametrize("causal", [True, False])
@pytest.mark.parametrize("softmax", [True, False])
def test_numpy_oracle_matches_reference_small(golden_dir, causal, softmax):
    g = _load(golden_dir, "attn_small.npz")
    scale = 1.0 if softmax else 0.5
    q, k, v, do = g["q"] * scale, g["k"] * scale, g["v"] * scale, g["do"]
    tag = f"{'c' if causal else 'f'}{'s' if softmax else 'n'}"
    out, _ = oracle.forward(q, k, v, causal, softmax)
    dq, dk, dv = oracle.backward(q, k, v, do, causal, softmax)
    # the fixtures are the reference's fp32 results; the oracle is float64
    np.testing.assert_allclose(out, g[f"o_{tag}"], atol=2e-5, rtol=1e-4)
    np.testing.assert_allclose(dq, g[f"dq_{tag}"], atol=5e-5, rtol=1e-4)
    np.testing.assert_allclose(dk, g[f"dk_{tag}"], atol=5e-5, rtol=1e-4)
    np.testing.assert_allclose(dv, g[f"dv_{tag}"], atol=5e-5, rtol=1e-4)


@pytest.mark.parametrize("causal", [True, False])
@pytest.mark.parametrize("softmax", [True, False])
def test_torch_oracle_matches_reference_small(golden_dir, causal, softmax):
    g = _load(golden_dir, "attn_small.npz")
    scale = 1.0 if softmax else 0.5
    q, k, v, do = (torch.tensor(g[n]) for n in ("q", "k", "v", "do"))
    q, k, v = q * scale, k * scale, v * scale
    tag = f"{'c' if causal else 'f'}{'s' if softmax else 'n'}"
    out, dq, dk, dv = oracle.torch_forward_backward(q, k, v, do, causal, softmax)
    for got, name in ((out, "o"), (dq, "dq"), (dk, "dk"), (dv, "dv")):
        np.testing.assert_allclose(got.numpy(), g[f"{name}_{tag}"], atol=1e-5, rtol=1e-5)


def test_oracle_matches_reference_parity_script_case(golden_dir):
    """test_equivalence.py:36-68: B2 H4 N128 D64, seed 42, causal, through the reference's fp32 SDPA trick."""
    g = _load(golden_dir, "attn_equiv.npz")
    torch.manual_seed(42)
    q, k, v, do = (torch.randn(2, 4, 128, 64) for _ in range(4))
    out, dq, dk, dv = oracle.torch_forward_backward(q, k, v, do, True, True)
    for got, name in ((out, "o"), (dq, "dq"), (dk, "dk"), (dv, "dv")):
        np.testing.assert_allclose(got[:, :, ::8].numpy(), g[name], atol=2e-5, rtol=1e-4)
    sums = [t.double().sum().item() for t in (out, dq, dk, dv)]
    np.testing.assert_allclose(sums, g["sums"], atol=5e-3)


def test_oracle_matches_reference_config1(golden_dir):
    """Benchmark configuration 1: fp32 B2 H4 N256 D64 causal, seed 0."""
    g = _load(golden_dir, "attn_config1.npz")
    q, k, v, do = oracle.make_inputs(2, 4, 256, 64, seed=0)
    out, dq, dk, dv = oracle.torch_forward_backward(q, k, v, do, True, True)
    for got, name in ((out, "o"), (dq, "dq"), (dk, "dk"), (dv, "dv")):
        np.testing.assert_allclose(got[:, :, ::16].numpy(), g[name], atol=1e-5, rtol=1e-5)
    # float64 hand-derived gradients on the same inputs
    dq64, dk64, dv64 = oracle.backward(q.numpy(), k.numpy(), v.numpy(), do.numpy(), True, True)
    np.testing.assert_allclose(dq64[:, :, ::16], g["dq"], atol=1e-4, rtol=1e-4)
    np.testing.assert_allclose(dk64[:, :, ::16], g["dk"], atol=1e-4, rtol=1e-4)
    np.testing.assert_allclose(dv64[:, :, ::16], g["dv"], atol=1e-4, rtol=1e-4)


def test_distance_form_equals_biased_dot_product_form():
    """rbf_math_test.py:16-66: softmax(-|q-k|^2 g) == softmax(2 g q.k - g |k|^2), float64."""
    rng = np.random.default_rng(42)
    q, k, v = (rng.standard_normal((2, 4, 128, 64)) for _ in range(3))
    gamma = 1.0 / math.sqrt(64)
    biased = 2 * gamma * q @ np.swapaxes(k, -1, -2) - gamma * (k * k).sum(-1)[..., None, :]
    keep = np.tril(np.ones((128, 128), dtype=bool))
    biased = np.where(keep, biased, -np.inf)
    e = np.exp(biased - biased.max(-1, keepdims=True))
    out_biased = (e / e.sum(-1, keepdims=True)) @ v
    out, L = oracle.forward(q, k, v, True, True)
    np.testing.assert_allclose(out, out_biased, atol=1e-12)
    # L is the base-2 LSE of the biased logits
    lse2 = (np.log(np.exp(biased - biased.max(-1, keepdims=True)).sum(-1)) + biased.max(-1)) * oracle.LOG2E
    np.testing.assert_allclose(L, lse2, atol=1e-10)
    np.testing.assert_allclose(oracle.torch_lse2(torch.tensor(q), torch.tensor(k), True).numpy(), lse2, atol=1e-4)


def test_hand_gradients_match_autograd_float64():
    g = torch.Generator().manual_seed(3)
    q, k, v, do = (torch.randn(1, 2, 33, 64, generator=g, dtype=torch.float64) * 0.7 for _ in range(4))
    for causal in (True, False):
        for softmax in (True, False):
            _, dq, dk, dv = oracle.torch_forward_backward(q, k, v, do, causal, softmax)
            hq, hk, hv = oracle.backward(q.numpy(), k.numpy(), v.numpy(), do.numpy(), causal, softmax)
            # the reference's logits are always evaluated in fp32 (rbf_attention.py:1548), hence 2e-6
            np.testing.assert_allclose(hq, dq.numpy(), atol=2e-6)
            np.testing.assert_allclose(hk, dk.numpy(), atol=2e-6)
            np.testing.assert_allclose(hv, dv.numpy(), atol=2e-6)


def test_make_inputs_is_seeded_and_outlier_norms():
    a = oracle.make_inputs(1, 2, 64, 64, seed=5, key_norm_sigma=0.5)
    b = oracle.make_inputs(1, 2, 64, 64, seed=5, key_norm_sigma=0.5)
    for x, y in zip(a, b):
        assert torch.equal(x, y)
    plain = oracle.make_inputs(1, 2, 4096, 64, seed=5)[1].norm(dim=-1)
    heavy = oracle.make_inputs(1, 2, 4096, 64, seed=5, key_norm_sigma=0.5)[1].norm(dim=-1)
    assert heavy.max() > 2.0 * plain.max() * 0.8
