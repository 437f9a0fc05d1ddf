"""Host-side logic that needs no GPU: operator schemas and fake kernels, the attention block's parameters and
comparator branches against the reference fixtures, the drop-in module name, input validation, and the
batch x head partition (including a two-rank gloo run)."""

import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import rbf_attention_b200  # noqa: F401  (registers the operators)
from rbf_attention_b200 import attention, ops, sharding

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_operator_schemas_match_the_reference():
    ns = torch.ops.rbf_attn_v5
    assert str(ns.scaled_fwd.default._schema) == (
        "rbf_attn_v5::scaled_fwd(Tensor q, Tensor k, Tensor v, bool is_causal) -> (Tensor, Tensor)")
    assert str(ns.scaled_bwd.default._schema) == (
        "rbf_attn_v5::scaled_bwd(Tensor q, Tensor k, Tensor v, Tensor out, Tensor L, Tensor dout, "
        "bool is_causal, float sm_scale) -> (Tensor, Tensor, Tensor)")
    assert str(ns.non_softmax_fwd.default._schema) == (
        "rbf_attn_v5::non_softmax_fwd(Tensor q, Tensor k, Tensor v, bool is_causal) -> Tensor")
    assert str(ns.non_softmax_bwd.default._schema) == (
        "rbf_attn_v5::non_softmax_bwd(Tensor q, Tensor k, Tensor v, Tensor dout, bool is_causal, "
        "float sm_scale) -> (Tensor, Tensor, Tensor)")


def test_fake_kernels_give_reference_shapes():
    q = torch.empty(2, 4, 100, 64, device="meta", dtype=torch.bfloat16).transpose(1, 2).transpose(1, 2)
    out, L = torch.ops.rbf_attn_v5.scaled_fwd(q, q, q, True)
    assert out.shape == q.shape and out.dtype == q.dtype and out.is_contiguous()
    assert L.shape == (2, 4, 100) and L.dtype == torch.float32
    dq, dk, dv = torch.ops.rbf_attn_v5.scaled_bwd(q, q, q, out, L, out, True, 0.125)
    assert dq.shape == dk.shape == dv.shape == q.shape
    o2 = torch.ops.rbf_attn_v5.non_softmax_fwd(q, q, q, True)
    assert o2.shape == q.shape
    assert len(torch.ops.rbf_attn_v5.non_softmax_bwd(q, q, q, o2, True, 0.125)) == 3


def test_cpu_tensors_are_refused_loudly():
    q = torch.randn(1, 1, 16, 64)
    with pytest.raises(RuntimeError, match="no CPU path"):
        ops.run_triton_rbf(q, q, q)
    with pytest.raises(RuntimeError, match="no CPU path"):
        ops.run_triton_non_softmax_rbf(q, q, q)


def test_dropin_module_name_is_the_implementation():
    import rbf_attention

    assert rbf_attention is attention
    for name in ("CustomCausalAttention", "run_triton_rbf", "run_triton_non_softmax_rbf", "rbf_flex_attention",
                 "compute_rbf_logits", "get_unrotated_sinusoids"):
        assert hasattr(rbf_attention, name)


@pytest.mark.parametrize("tag,kind", [("s", "rbf_slow"), ("n", "rbf_non_softmax_slow")])
def test_block_comparator_branches_match_reference_fixture(golden_dir, tag, kind):
    g = np.load(os.path.join(golden_dir, "block_small.npz"))
    blk = attention.CustomCausalAttention(2, 128, max_seq_len=64, use_rope=True, attention_type=kind, num_registers=4)
    state = {k[len(f"param_{tag}."):]: torch.tensor(g[k]) for k in g.files if k.startswith(f"param_{tag}.")}
    assert set(state) == {"qkv_proj.weight", "qkv_proj.bias", "proj.weight", "proj.bias", "pos_weight", "reg_pos_emb"}
    blk.load_state_dict(state)          # same keys and shapes as the reference's state dict
    x = torch.tensor(g[f"x_{tag}"]).requires_grad_(True)
    y, w = blk(x)
    y.backward(torch.tensor(g[f"gy_{tag}"]))
    assert w is not None and w.shape == (2, 2, 24, 24)
    np.testing.assert_allclose(y.detach().numpy(), g[f"y_{tag}"], atol=1e-6)
    np.testing.assert_allclose(x.grad.numpy(), g[f"gx_{tag}"], atol=1e-6)
    for name, prm in blk.named_parameters():
        np.testing.assert_allclose(prm.grad.numpy(), g[f"grad_{tag}.{name}"], atol=1e-5, err_msg=name)


def test_block_buffers_are_not_persistent_and_rbf_types_use_susie():
    blk = attention.CustomCausalAttention(8, 512, max_seq_len=128, attention_type="rbf_triton", num_registers=4)
    assert blk.positional_encoding_type == "susie"
    assert "susie_cache" not in blk.state_dict()
    assert blk.pos_weight.shape == (1, 8, 1, 32) and blk.reg_pos_emb.shape == (1, 8, 4, 64)
    std = attention.CustomCausalAttention(8, 512, max_seq_len=128, attention_type="standard")
    assert std.positional_encoding_type == "rope" and "cos" not in std.state_dict()


def test_shard_batch_heads_covers_every_pair_exactly_once():
    for B, H, world in [(8, 16, 1), (8, 16, 2), (8, 16, 4), (8, 16, 8), (2, 32, 8), (4, 16, 8), (2, 32, 4), (3, 8, 4)]:
        seen = np.zeros((B, H), dtype=int)
        for rank in range(world):
            sb, sh = sharding.shard_batch_heads(B, H, rank, world)
            seen[sb, sh] += 1
        assert (seen == 1).all(), (B, H, world)
        b_loc, h_loc = sharding.local_shape(B, H, world)
        assert b_loc * h_loc * world == B * H
    with pytest.raises(ValueError):
        sharding.shard_batch_heads(3, 5, 0, 2)
    with pytest.raises(ValueError):
        sharding.shard_batch_heads(8, 16, 8, 8)


def test_attention_flops_convention():
    assert sharding.attention_flops(8, 16, 4096, 64, True) == pytest.approx(9.62e11, rel=2e-3)
    assert sharding.attention_flops(2, 32, 16384, 128, False) == pytest.approx(3.079e13, rel=2e-3)
    assert sharding.attention_flops(4, 16, 8192, 64, True, backward=False) == pytest.approx(4 * 64 * 8192**2 * 64 / 2)


_GLOO_WORKER = r"""
import os, sys
sys.path.insert(0, sys.argv[1])
import torch, torch.distributed as dist
from rbf_attention_b200 import sharding
from oracle import rbf_oracle as oracle
dist.init_process_group("gloo", init_method="tcp://127.0.0.1:" + sys.argv[2], rank=int(sys.argv[3]), world_size=2)
rank = dist.get_rank()
B, H, N, D = 2, 4, 48, 64
q, k, v, do = oracle.make_inputs(B, H, N, D, seed=11)
sb, sh = sharding.shard_batch_heads(B, H, rank, 2)
local = oracle.torch_forward(q[sb, sh], k[sb, sh], v[sb, sh], True, True).contiguous()
parts = [torch.empty_like(local) for _ in range(2)]
dist.all_gather(parts, local)          # only to check the partition; the data path itself has no collective
full = oracle.torch_forward(q, k, v, True, True)
for r, part in enumerate(parts):
    rb, rh = sharding.shard_batch_heads(B, H, r, 2)
    assert torch.allclose(full[rb, rh], part, atol=1e-6), r
t = torch.tensor([float(local.numel())])
dist.all_reduce(t)
assert t.item() == full.numel()
dist.barrier()
dist.destroy_process_group()
print("ok", rank)
"""


def test_two_rank_partition_with_gloo(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(_GLOO_WORKER)
    port = str(29500 + os.getpid() % 2000)
    procs = [subprocess.Popen([sys.executable, str(script), ROOT, port, str(r)], stdout=subprocess.PIPE,
                              stderr=subprocess.STDOUT, text=True) for r in range(2)]
    outs = [p.communicate(timeout=180)[0] for p in procs]
    for r, (p, o) in enumerate(zip(procs, outs)):
        assert p.returncode == 0 and f"ok {r}" in o, o


_DP_WORKER = r"""
import os, sys
sys.path.insert(0, sys.argv[1])
import torch, torch.distributed as dist
import torch.nn.functional as F
from rbf_attention_b200 import lm
rank, world = int(sys.argv[3]), 2
dist.init_process_group("gloo", init_method="tcp://127.0.0.1:" + sys.argv[2], rank=rank, world_size=world)
VOCAB = 211
def make():
    torch.manual_seed(0)
    m = lm.CausalLM(VOCAB, d_model=64, num_layers=2, num_heads=2, max_seq_len=32, pos_emb_type="rope",
                    num_registers=2, attention_type="rbf_slow")
    with torch.no_grad():
        m.register_tokens.normal_(0.0, 0.3)
    return m
def loss_of(model, ids):
    logits, _ = model(ids[:, :-1])
    return F.cross_entropy(logits.reshape(-1, VOCAB), ids[:, 1:].reshape(-1))
ids_all = lm.zipf_token_ids(4, 33, VOCAB, seed=1)          # the global batch; every rank takes two sequences
mine = ids_all[2 * rank: 2 * rank + 2]
model = make()
ddp = torch.nn.parallel.DistributedDataParallel(model)
opt = torch.optim.AdamW(model.parameters(), lr=1e-3)
loss_of(ddp, mine).backward()                              # gradients are averaged over the ranks by the all-reduce
grads = [p.grad.clone() for p in model.parameters()]
# (1) both ranks hold the same gradients
for g in grads:
    other = [torch.empty_like(g) for _ in range(world)]
    dist.all_gather(other, g)
    assert torch.equal(other[0], other[1])
# (2) they equal the single-process gradients on the concatenated batch (mean over 4 sequences of equal length)
single = make()
loss_of(single, ids_all).backward()
for (name, p), g in zip(single.named_parameters(), grads):
    assert torch.allclose(p.grad, g, atol=2e-6, rtol=1e-4), (name, (p.grad - g).abs().max().item())
# (3) after the optimizer step the replicas are still identical
opt.step()
for p in model.parameters():
    other = [torch.empty_like(p.data) for _ in range(world)]
    dist.all_gather(other, p.data)
    assert torch.equal(other[0], other[1])
dist.barrier()
dist.destroy_process_group()
print("ok", rank)
"""


def test_two_rank_data_parallel_training_step_with_gloo(tmp_path):
    """The data-parallel step of the end-to-end configuration on two CPU ranks (materialised-matrix attention, which
    needs no GPU): gradient all-reduce through DistributedDataParallel, AdamW step (train_rbf_transformer.py:258-349
    trains one replica; the all-reduce is what the multi-GPU benchmark adds)."""
    script = tmp_path / "dp_worker.py"
    script.write_text(_DP_WORKER)
    port = str(31500 + os.getpid() % 2000)
    procs = [subprocess.Popen([sys.executable, str(script), ROOT, port, str(r)], stdout=subprocess.PIPE,
                              stderr=subprocess.STDOUT, text=True) for r in range(2)]
    outs = [p.communicate(timeout=300)[0] for p in procs]
    for r, (p, o) in enumerate(zip(procs, outs)):
        assert p.returncode == 0 and f"ok {r}" in o, o


def test_language_model_matches_reference_fixture(golden_dir):
    """train_rbf_transformer.CausalLM (rbf_slow, 2 register tokens, SuSiE positions): same state-dict keys, logits,
    loss and parameter gradients."""
    from rbf_attention_b200 import lm

    g = np.load(os.path.join(golden_dir, "lm_small.npz"))
    model = lm.CausalLM(vocab_size=97, d_model=64, num_layers=2, num_heads=2, max_seq_len=32, pos_emb_type="rope",
                        num_registers=2, attention_type="rbf_slow")
    state = {k[len("param."):]: torch.tensor(g[k]) for k in g.files if k.startswith("param.")}
    assert set(state) == set(dict(model.named_parameters()))
    model.load_state_dict(state)
    idx = torch.tensor(g["idx"])
    logits, weights = model(idx)
    assert len(weights) == 2 and weights[0].shape == (3, 2, 14, 14)
    loss = torch.nn.functional.cross_entropy(logits[:, :-1].reshape(-1, 97), idx[:, 1:].reshape(-1))
    loss.backward()
    np.testing.assert_allclose(logits.detach().numpy(), g["logits"], atol=1e-5)
    np.testing.assert_allclose(loss.item(), g["loss"], atol=1e-6)
    for name, prm in model.named_parameters():
        np.testing.assert_allclose(prm.grad.numpy(), g[f"grad.{name}"], atol=2e-5, err_msg=name)


def test_zipf_token_ids_are_seeded_and_heavy_headed():
    from rbf_attention_b200 import lm

    a = lm.zipf_token_ids(4, 257, 50257, seed=3)
    b = lm.zipf_token_ids(4, 257, 50257, seed=3)
    assert torch.equal(a, b) and a.shape == (4, 257) and a.max() < 50257 and a.min() >= 0
    assert (a < 10).float().mean() > 0.2        # a Zipf(1.1) head: the ten most frequent ids carry > 20 % of the mass
