"""Generates tests/golden/*.npz by running the reference project's own PyTorch code on the CPU.

Run where the reference checkout is available:
    python tests/golden/make_golden.py /path/to/reference
The reference module imports matplotlib (not installed here) for its plotting helpers only, so a stub
module is registered before the import. Nothing else of the reference is altered.

Fixtures (all fp32 unless noted):
  attn_small.npz     full tensors, softmax + non-softmax, causal + non-causal, B1 H2 N80 D64 (ragged N)
  attn_equiv.npz     the reference's own parity-script case (test_equivalence.py:36-68: B2 H4 N128 D64,
                     seed 42, causal) through its fp32 augmented-dimension SDPA (`rbf_math_forward`);
                     rows subsampled by 8 to keep the file small
  attn_config1.npz   benchmark configuration 1 (B2 H4 N256 D64 causal, seed 0) through the `rbf_slow` math;
                     rows subsampled by 16, plus per-tensor sums
  block_small.npz    CustomCausalAttention(rbf_slow / rbf_non_softmax_slow) with SuSiE positions and 4 register
                     tokens: parameters, input, output and parameter gradients
  lm_small.npz       train_rbf_transformer.CausalLM (2 layers, d 64, 2 heads, 2 register tokens, rbf_slow): token ids,
                     logits, loss and all parameter gradients
"""

import math
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def import_reference(path):
    stub = types.ModuleType("matplotlib")
    stub.pyplot = types.ModuleType("matplotlib.pyplot")
    sys.modules.setdefault("matplotlib", stub)
    sys.modules.setdefault("matplotlib.pyplot", stub.pyplot)
    sys.path.insert(0, path)
    import rbf_attention as ref  # noqa: E402

    return ref


def slow_attention(ref, q, k, v, causal, softmax):
    """The rbf_slow / rbf_non_softmax_slow branches (rbf_attention.py:1738-1753) on raw (B,H,N,D) tensors."""
    logits = ref.compute_rbf_logits(q, k)
    if causal:
        mask = torch.ones(q.shape[-2], q.shape[-2], dtype=torch.bool).triu_(1)
        logits = logits.masked_fill(mask, float("-inf"))
    w = torch.softmax(logits, dim=-1) if softmax else torch.exp(logits)
    return w @ v


def grads(fn, q, k, v, do):
    qq, kk, vv = (t.clone().requires_grad_(True) for t in (q, k, v))
    out = fn(qq, kk, vv)
    out.backward(do)
    return out.detach(), qq.grad, kk.grad, vv.grad


def main(ref_path):
    ref = import_reference(ref_path)
    torch.manual_seed(0)

    # ---- attn_small: full tensors ------------------------------------------------------------
    g = torch.Generator().manual_seed(1234)
    B, H, N, D = 1, 2, 80, 64
    q, k, v, do = (torch.randn(B, H, N, D, generator=g) for _ in range(4))
    q_ns, k_ns, v_ns = q * 0.5, k * 0.5, v * 0.5
    data = {"q": q, "k": k, "v": v, "do": do}
    for causal in (True, False):
        for softmax in (True, False):
            qq, kk, vv = (q, k, v) if softmax else (q_ns, k_ns, v_ns)
            o, dq, dk, dv = grads(lambda a, b, c: slow_attention(ref, a, b, c, causal, softmax), qq, kk, vv, do)
            tag = f"{'c' if causal else 'f'}{'s' if softmax else 'n'}"
            data.update({f"o_{tag}": o, f"dq_{tag}": dq, f"dk_{tag}": dk, f"dv_{tag}": dv})
    np.savez_compressed(os.path.join(HERE, "attn_small.npz"), **{n: t.numpy() for n, t in data.items()})

    # ---- attn_equiv: the reference's parity-script case -----------------------------------------
    sys.path.insert(0, ref_path)
    import test_equivalence as te  # noqa: E402

    torch.manual_seed(42)
    B, H, N, D = 2, 4, 128, 64
    q = torch.randn(B, H, N, D)
    k = torch.randn(B, H, N, D)
    v = torch.randn(B, H, N, D)
    do = torch.randn(B, H, N, D)
    o, dq, dk, dv = grads(lambda a, b, c: te.rbf_math_forward(a, b, c, is_causal=True), q, k, v, do)
    sub = slice(None, None, 8)
    np.savez_compressed(
        os.path.join(HERE, "attn_equiv.npz"),
        o=o[:, :, sub].numpy(), dq=dq[:, :, sub].numpy(), dk=dk[:, :, sub].numpy(), dv=dv[:, :, sub].numpy(),
        sums=np.array([t.double().sum().item() for t in (o, dq, dk, dv)]),
    )

    # ---- attn_config1: benchmark configuration 1 -------------------------------------------------
    g = torch.Generator().manual_seed(0)
    B, H, N, D = 2, 4, 256, 64
    q, k, v, do = (torch.randn(B, H, N, D, generator=g) for _ in range(4))
    o, dq, dk, dv = grads(lambda a, b, c: slow_attention(ref, a, b, c, True, True), q, k, v, do)
    sub = slice(None, None, 16)
    np.savez_compressed(
        os.path.join(HERE, "attn_config1.npz"),
        o=o[:, :, sub].numpy(), dq=dq[:, :, sub].numpy(), dk=dk[:, :, sub].numpy(), dv=dv[:, :, sub].numpy(),
        sums=np.array([t.double().sum().item() for t in (o, dq, dk, dv)]),
    )

    # ---- block_small: the attention block with SuSiE positions and register tokens ---------------
    out = {}
    for kind in ("rbf_slow", "rbf_non_softmax_slow"):
        torch.manual_seed(7)
        blk = ref.CustomCausalAttention(num_heads=2, emb_dims=128, max_seq_len=64, use_rope=True,
                                        attention_type=kind, num_registers=4)
        x = torch.randn(2, 24, 128) * (0.5 if "non_softmax" in kind else 1.0)
        x.requires_grad_(True)
        y, _ = blk(x)
        gy = torch.randn(y.shape, generator=torch.Generator().manual_seed(8))
        y.backward(gy)
        tag = "s" if kind == "rbf_slow" else "n"
        out[f"x_{tag}"] = x.detach().numpy()
        out[f"y_{tag}"] = y.detach().numpy()
        out[f"gy_{tag}"] = gy.numpy()
        out[f"gx_{tag}"] = x.grad.numpy()
        for name, prm in blk.named_parameters():
            out[f"param_{tag}.{name}"] = prm.detach().numpy()
            out[f"grad_{tag}.{name}"] = prm.grad.numpy()
    np.savez_compressed(os.path.join(HERE, "block_small.npz"), **out)

    # ---- lm_small: the language model (register tokens, SuSiE positions) through the rbf_slow branch ------
    import train_rbf_transformer as trt  # noqa: E402

    torch.manual_seed(11)
    lm = trt.CausalLM(vocab_size=97, d_model=64, num_layers=2, num_heads=2, max_seq_len=32, pos_emb_type="rope",
                      num_registers=2, attention_type="rbf_slow")
    with torch.no_grad():
        lm.register_tokens.normal_(0.0, 0.02)     # the reference initialises them to zero; make them matter
    idx = torch.randint(0, 97, (3, 12), generator=torch.Generator().manual_seed(12))
    logits, _ = lm(idx)
    loss = torch.nn.functional.cross_entropy(logits[:, :-1].reshape(-1, 97), idx[:, 1:].reshape(-1))
    loss.backward()
    out = {"idx": idx.numpy(), "logits": logits.detach().numpy(), "loss": np.array(loss.item())}
    for name, prm in lm.named_parameters():
        out[f"param.{name}"] = prm.detach().numpy()
        out[f"grad.{name}"] = prm.grad.numpy()
    np.savez_compressed(os.path.join(HERE, "lm_small.npz"), **out)
    print("wrote fixtures to", HERE)


if __name__ == "__main__":
    if len(sys.argv) < 2:
        sys.exit("usage: python tests/golden/make_golden.py /path/to/reference")
    main(sys.argv[1])
