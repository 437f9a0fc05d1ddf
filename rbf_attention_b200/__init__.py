"""B200-native fused RBF attention (forward + backward), a drop-in for the reference project's
``rbf_attn_v5`` operators and the attention block that calls them."""

from .ops import run_triton_non_softmax_rbf, run_triton_rbf  # noqa: F401

__all__ = ["run_triton_rbf", "run_triton_non_softmax_rbf"]
