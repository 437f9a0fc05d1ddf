"""Causal language model around the RBF attention block, with the reference's module and parameter names
(``train_rbf_transformer.py:113-244``: ``token_emb``, ``register_tokens``, ``blocks.<i>.{attn, ln1, ff, ln2}``,
``ln_f``, ``to_logits``), so that reference checkpoints load and the data-parallel training step of the benchmark
runs the same architecture: pre-LayerNorm blocks, 4x GELU MLP, zero-initialised register tokens prepended to the
sequence and sliced off before the final norm, untied output projection."""

from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

from .attention import CustomCausalAttention


def vocab_projection(linear: nn.Linear, x: torch.Tensor, keep_padding: bool = False) -> torch.Tensor:
    """``linear(x)`` for an output width (the vocabulary) whose rows are not 16-byte aligned in 16-bit types. With the
    reference's vocabulary of 50257 the logits' row pitch is odd, and the GEMM library falls back to kernels of an old
    architecture for all three products of this layer (measured on B200: 77 of the 116 ms of a training step). The
    product is evaluated at the width rounded up to a multiple of 64 - the weight is zero-padded on the fly, 51 MB -
    and the caller gets the first ``out_features`` columns as a view; parameters and state dict are unchanged.
    With ``keep_padding`` the padded width is returned as it is, the extra columns holding -inf (probability zero,
    gradient zero): a loss evaluated on it equals the loss on the sliced logits and saves the copies a strided view of
    6.6 GB of logits costs on its way through log-softmax and back."""
    V = linear.out_features
    pad = (-V) % 64
    if pad == 0 or not x.is_cuda or x.dtype == torch.float32:
        return linear(x)
    weight = F.pad(linear.weight, (0, 0, 0, pad))
    if keep_padding:
        bias = torch.zeros(V, dtype=x.dtype, device=x.device) if linear.bias is None else linear.bias
        return F.linear(x, weight, F.pad(bias, (0, pad), value=float("-inf")))
    bias = None if linear.bias is None else F.pad(linear.bias, (0, pad))
    return F.linear(x, weight, bias)[..., :V]


def apply_layer_norm(ln: nn.LayerNorm, x: torch.Tensor) -> torch.Tensor:
    """``ln(x)``: 16-bit CUDA activations of a supported width go through the library's one-pass kernels
    (``ops.layer_norm``, a warp per row; PyTorch's kernels reach a sixth of the memory bandwidth at 512 columns),
    anything else through PyTorch."""
    if x.is_cuda and len(ln.normalized_shape) == 1 and ln.elementwise_affine:
        from . import ops

        if ops.layer_norm_supported(x, ln.weight, ln.bias):
            return ops.layer_norm(x, ln.weight, ln.bias, ln.eps)
    return ln(x)


def apply_add_layer_norm(ln: nn.LayerNorm, x: torch.Tensor, delta):
    """``x = x + delta; return x, ln(x)`` (``delta`` None: ``x, ln(x)``): the residual addition rides on the
    LayerNorm that follows it, forward and backward, where the library's kernels apply."""
    if delta is None:
        return x, apply_layer_norm(ln, x)
    if x.is_cuda and len(ln.normalized_shape) == 1 and ln.elementwise_affine and delta.shape == x.shape \
            and delta.dtype == x.dtype:
        from . import ops

        if ops.layer_norm_supported(x, ln.weight, ln.bias):
            return ops.add_layer_norm(x, delta, ln.weight, ln.bias, ln.eps)
    x = x + delta
    return x, ln(x)


def cross_entropy(logits: torch.Tensor, targets: torch.Tensor, ignore_index: int = -100) -> torch.Tensor:
    """The training loss of the reference (``torch.nn.CrossEntropyLoss(ignore_index=-100)`` on flattened logits,
    train_rbf_transformer.py:282, 340-345). CUDA logits go through the library's single-kernel loss + gradient
    (``ops.cross_entropy``: one read and one write of the logits instead of four passes and an fp32 copy); anything
    else (the CPU oracle runs of the tests) is PyTorch's."""
    logits = logits.reshape(-1, logits.shape[-1])
    targets = targets.reshape(-1)
    if logits.is_cuda:
        from . import ops

        return ops.cross_entropy(logits, targets, ignore_index)
    return F.cross_entropy(logits, targets, ignore_index=ignore_index)


class TransformerBlock(nn.Module):
    def __init__(self, emb_dim, num_heads, max_seq_len, use_rope, attention_type, use_qk_norm=False, use_xsa=False,
                 num_registers=0):
        super().__init__()
        self.attention_type = attention_type
        self.use_qk_norm = use_qk_norm
        self.use_xsa = use_xsa
        self.attn = CustomCausalAttention(num_heads, emb_dim, max_seq_len, use_rope, attention_type, use_qk_norm,
                                          use_xsa, num_registers)
        self.ln1 = nn.LayerNorm(emb_dim)
        self.ff = nn.Sequential(nn.Linear(emb_dim, 4 * emb_dim), nn.GELU(), nn.Linear(4 * emb_dim, emb_dim))
        self.ln2 = nn.LayerNorm(emb_dim)

    def forward(self, x):
        x, mlp_out, attn_weights = self.forward_deferred(x)
        return x + mlp_out, attn_weights

    def forward_deferred(self, x, pending=None):
        """The block on ``x + pending`` with its own last residual addition left to the caller: returns
        (x, mlp_out, attention weights) with the block's output being ``x + mlp_out``. A stack of blocks hands
        ``mlp_out`` to the next block as ``pending``, so that every residual addition is made by the LayerNorm pass
        that follows it."""
        x, normed = apply_add_layer_norm(self.ln1, x, pending)
        attn_out, attn_weights = self.attn(normed)
        x, normed = apply_add_layer_norm(self.ln2, x, attn_out)
        return x, self._mlp(normed), attn_weights

    def _mlp(self, x):
        """``self.ff(x)`` (Linear, GELU, Linear) with the activation, its backward and the bias gradients of both
        projections from the library."""
        if x.is_cuda:
            from . import ops

            exact_gelu = isinstance(self.ff[1], nn.GELU) and self.ff[1].approximate == "none"
            hidden = ops.linear_gelu(self.ff[0], x) if exact_gelu else self.ff[1](ops.linear(self.ff[0], x))
            return ops.linear(self.ff[2], hidden)
        return self.ff(x)


class CausalLM(nn.Module):
    def __init__(self, vocab_size, d_model=256, num_layers=4, num_heads=4, max_seq_len=1024, pos_emb_type="none",
                 use_qk_norm=False, num_registers=0, attention_type="standard"):
        super().__init__()
        if use_qk_norm and attention_type.startswith("rbf"):
            raise AssertionError("QK-Norm requires standard attention")
        if pos_emb_type not in ("none", "rope", "learned"):
            raise ValueError(f"Unsupported pos_emb_type: {pos_emb_type}")
        self.num_registers = num_registers
        self.use_qk_norm = use_qk_norm
        self.pos_emb_type = pos_emb_type
        if num_registers > 0:
            if attention_type.startswith("rbf"):
                # zero registers start at distance |q|^2 from every query (the reference's choice for RBF)
                init = torch.zeros(num_registers, d_model)
            elif attention_type.startswith("standard"):
                init = torch.randn(num_registers, d_model) * d_model**-0.5
            else:
                raise ValueError(f"Unsupported attention type: {attention_type}")
            self.register_tokens = nn.Parameter(init)
        self.token_emb = nn.Embedding(vocab_size, d_model)
        if pos_emb_type == "learned":
            self.pos_emb = nn.Embedding(max_seq_len, d_model)
        self.use_rope = pos_emb_type == "rope"
        self.blocks = nn.ModuleList(
            TransformerBlock(d_model, num_heads, max_seq_len, self.use_rope, attention_type, use_qk_norm=use_qk_norm,
                             use_xsa=False, num_registers=num_registers)
            for _ in range(num_layers)
        )
        self.ln_f = nn.LayerNorm(d_model)
        self.to_logits = nn.Linear(d_model, vocab_size)

    def forward(self, idx, padded_logits: bool = False):
        """Returns (logits, attention weights per block). ``padded_logits`` (not in the reference): the logits keep the
        vocabulary rounded up to a multiple of 64 with -inf in the extra columns, see ``vocab_projection``."""
        bsz, seq = idx.shape
        x = self.token_emb(idx)
        if self.pos_emb_type == "learned":
            x = x + self.pos_emb(torch.arange(seq, device=idx.device))
        if self.num_registers > 0:
            x = torch.cat([self.register_tokens.unsqueeze(0).expand(bsz, -1, -1).to(x.dtype), x], dim=1)
        weights = []
        pending = None                      # the last block's MLP output, added by the next LayerNorm pass
        for block in self.blocks:
            x, pending, w = block.forward_deferred(x, pending)
            weights.append(w)
        _, normed = apply_add_layer_norm(self.ln_f, x, pending)     # row-wise: the register rows are dropped after it
        if self.num_registers > 0:
            # contiguous: F.linear takes a strided 3-D input through matmul + a separate bias pass over the logits
            normed = normed[:, self.num_registers:, :].contiguous()
        return vocab_projection(self.to_logits, normed, keep_padding=padded_logits), weights


def zipf_token_ids(batch, seq_len, vocab_size, exponent=1.1, seed=0):
    """(batch, seq_len) int64 token ids with P(id = k) proportional to (k + 1)^-exponent, seeded, on the CPU."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    probs = torch.arange(1, vocab_size + 1, dtype=torch.float64).pow(-exponent)
    return torch.multinomial(probs / probs.sum(), batch * seq_len, replacement=True, generator=g).view(batch, seq_len)
