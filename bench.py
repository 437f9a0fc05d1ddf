"""Benchmark of the fused RBF attention forward+backward on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--workload config2|config3|config3_full|config4|config5_lm]

A step is one forward + backward pass of the attention operator over one batch of seeded synthetic
inputs. ``value`` is algorithmic TFLOP/s (4 B H N^2 D forward + 10 B H N^2 D backward, halved when causal)
with inputs resident in HBM; ``e2e`` is the same metric through the public PyTorch operator with HOST
(pinned) inputs and outputs, copies inside the timed region. With N > 1 every rank runs the same per-GPU
workload on its own seed (independent batch x head pairs, no collective in the data path) and ``value``
is the sum over ranks divided by the slowest rank's time. One JSON line is printed by rank 0.

``--workload config5_lm`` runs the data-parallel language-model training step instead (tokens/s; NCCL gradient
all-reduce through DistributedDataParallel when N > 1).

``--impl reference`` times the reference project's own CPU path (materialised-matrix PyTorch math with
autograd, restated in oracle/rbf_oracle.py) on the host cores, one (batch, head) pair of the workload per step.
"""

from __future__ import annotations

import argparse
import ctypes
import json
import math
import os
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOADS = {
    # BASELINE configuration 2: outlier key norms (one LogNormal(0, 0.5) factor per key row)
    "config2": dict(B=8, H=16, N=4096, D=64, causal=True, softmax=True, std=1.0, key_norm_sigma=0.5),
    "config3": dict(B=2, H=32, N=16384, D=128, causal=True, softmax=True, std=1.0, key_norm_sigma=0.0),
    "config3_full": dict(B=2, H=32, N=16384, D=128, causal=False, softmax=True, std=1.0, key_norm_sigma=0.0),
    "config4": dict(B=4, H=16, N=8192, D=64, causal=True, softmax=False, std=0.5, key_norm_sigma=0.0),
}
METRIC = "rbf_attn_fwd_bwd_tflops"
UNIT = "TFLOP/s"


def flops(w, forward=True, backward=True):
    per = (4.0 if forward else 0.0) + (10.0 if backward else 0.0)
    f = per * w["B"] * w["H"] * float(w["N"]) ** 2 * w["D"]
    return f * 0.5 if w["causal"] else f


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as fh:
            d = json.load(fh)
        return float(d["bf16_tflops"]), "measured (MEASURED_PEAKS.json bf16_tflops, burst)"
    return 1590.0, "fallback (1.59 PFLOP/s, earlier measurement on this pool)"


# ---------------------------------------------------------------------------------------------
# clocks during the timed region (NVML, read-only)
# ---------------------------------------------------------------------------------------------
class ClockSampler:
    REASONS = {0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown",
               0x80: "hw_power_brake_slowdown"}

    def __init__(self, index: int, period_s: float = 0.02):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml

            pynvml.nvmlInit()
            self._nv = pynvml
            self._h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM)
            self._period = period_s
        except Exception:
            self._nv = None

    def _run(self):
        nv = self._nv
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM))
                mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self._h)
                for bit, name in self.REASONS.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(self._period)

    def __enter__(self):
        if self._nv is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": 0}
        s = sorted(self.samples)
        return {"sm_mhz": s[len(s) // 2], "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(s)}


# ---------------------------------------------------------------------------------------------
# the reference's CPU path (oracle port), used by --impl reference and the cpu_baseline leg
# ---------------------------------------------------------------------------------------------
def cpu_pairs_per_second(w, budget_s=12.0, max_pairs=4):
    """Times forward+backward of single (batch, head) pairs of workload ``w`` with the fp32 PyTorch CPU math on
    all host threads. Returns (TFLOP/s, threads, pairs timed, seconds per pair)."""
    import torch

    from oracle import rbf_oracle as oracle

    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    q, k, v, do = oracle.make_inputs(1, 1, w["N"], w["D"], seed=0, std=w["std"], key_norm_sigma=w["key_norm_sigma"])
    times = []
    t_start = time.perf_counter()
    while len(times) < max_pairs and (not times or time.perf_counter() - t_start + times[-1] < budget_s):
        t0 = time.perf_counter()
        oracle.torch_forward_backward(q, k, v, do, w["causal"], w["softmax"])
        times.append(time.perf_counter() - t0)
    best = min(times)
    pair = dict(w, B=1, H=1)
    return flops(pair) / best / 1e12, threads, len(times), best


def run_reference(args, w, rank, world):
    if rank != 0:
        return
    import torch

    from oracle import rbf_oracle as oracle

    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    q, k, v, do = oracle.make_inputs(1, 1, w["N"], w["D"], seed=0, std=w["std"], key_norm_sigma=w["key_norm_sigma"])
    for _ in range(max(1, min(args.warmup, 2))):
        oracle.torch_forward_backward(q, k, v, do, w["causal"], w["softmax"])
    steps = max(1, args.steps)
    t0 = time.perf_counter()
    for _ in range(steps):
        oracle.torch_forward_backward(q, k, v, do, w["causal"], w["softmax"])
    dt = time.perf_counter() - t0
    pair = dict(w, B=1, H=1)
    value = flops(pair) * steps / dt / 1e12
    sample = (f"1 of {w['B'] * w['H']} (batch, head) pairs per step at full N={w['N']}, D={w['D']}, fp32, "
              f"materialised N x N matrix, autograd backward")
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": steps,
        "warmup": args.warmup, "ms_per_step": dt / steps * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": args.workload, **{k_: w[k_] for k_ in ("B", "H", "N", "D", "causal", "softmax")},
                   "timed_on": "host CPU"},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------------------------
# our arm
# ---------------------------------------------------------------------------------------------
class DeviceRunner:
    """Pre-allocated device buffers and raw C-ABI calls (no allocation inside the timed region)."""

    def __init__(self, w, device, seed):
        import torch

        from rbf_attention_b200 import _lib, synthetic

        self.torch, self.w, self.lib = torch, w, _lib.load()
        self._libmod = _lib
        B, H, N, D = w["B"], w["H"], w["N"], w["D"]
        host = synthetic.make_inputs(B, H, N, D, seed=seed, dtype=torch.bfloat16, std=w["std"],
                                     key_norm_sigma=w["key_norm_sigma"])
        self.host = [t.pin_memory() for t in host]
        self.q, self.k, self.v, self.do = (t.to(device) for t in host)
        self.out = torch.empty_like(self.q)
        self.lse = torch.empty((B, H, N), dtype=torch.float32, device=device)
        self.dq, self.dk, self.dv = (torch.empty_like(self.q) for _ in range(3))
        nb = max(self.lib.rbf_b200_workspace_bytes(B, H, N, D, int(w["softmax"]), 1),
                 self.lib.rbf_b200_workspace_bytes(B, H, N, D, int(w["softmax"]), 0))
        self.ws = torch.empty(nb, dtype=torch.uint8, device=device)
        self.s = _lib.strides3(self.q)
        self.scale = 1.0 / math.sqrt(D)
        self.stream = torch.cuda.current_stream(device).cuda_stream

    def fwd(self, phases=7):
        w = self.w
        rc = self.lib.rbf_b200_fwd_phases(
            self.q.data_ptr(), self.k.data_ptr(), self.v.data_ptr(), self.out.data_ptr(), self.lse.data_ptr(),
            self.ws.data_ptr(), self.ws.numel(), w["B"], w["H"], w["N"], w["D"], self.s, self.s, self.s, self.s, 0,
            int(w["causal"]), int(w["softmax"]), self.scale, self.stream, phases)
        self._libmod.check(rc, "rbf_b200_fwd")

    def bwd(self, phases=7):
        w = self.w
        rc = self.lib.rbf_b200_bwd_phases(
            self.q.data_ptr(), self.k.data_ptr(), self.v.data_ptr(), self.out.data_ptr(), self.lse.data_ptr(),
            self.do.data_ptr(), self.dq.data_ptr(), self.dk.data_ptr(), self.dv.data_ptr(), self.ws.data_ptr(),
            self.ws.numel(), w["B"], w["H"], w["N"], w["D"], self.s, self.s, self.s, self.s, self.s, self.s, self.s,
            self.s, 0, int(w["causal"]), int(w["softmax"]), self.scale, self.stream, phases)
        self._libmod.check(rc, "rbf_b200_bwd")

    def step(self):
        self.fwd()
        self.bwd()

    def check_status(self):
        code = ctypes.c_uint(0)
        rc = self.lib.rbf_b200_read_device_status(self.ws.data_ptr(), self.stream, ctypes.byref(code))
        self._libmod.check(rc, "device status")


def time_loop(torch, fn, steps):
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / steps


def run_ours(args, w, rank, world, local_rank):
    import torch
    import torch.distributed as dist

    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device: the product has no CPU path")
    device = torch.device("cuda", local_rank)
    torch.cuda.set_device(device)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)

    runner = DeviceRunner(w, device, seed=1000 + rank)
    for _ in range(max(args.warmup, 3)):
        runner.step()
    runner.check_status()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-resident throughput: exactly K steps, max over ranks --------------------------
    barrier()
    with ClockSampler(local_rank) as clocks:
        ms = time_loop(torch, runner.step, args.steps)
        # per-kernel times for the roofline line (same buffers, same stream)
        fused = True                             # single-kernel backward (plus the dQ conversion kernel)
        phase_ms = {"fwd": time_loop(torch, lambda: runner.fwd(2), args.steps)}
        if fused:
            phase_ms["bwd_fused"] = time_loop(torch, lambda: runner.bwd(2), args.steps)
        else:
            phase_ms["bwd_dkdv"] = time_loop(torch, lambda: runner.bwd(2), args.steps)
            phase_ms["bwd_dq"] = time_loop(torch, lambda: runner.bwd(4), args.steps)
        phase_ms["prepass"] = time_loop(torch, lambda: (runner.fwd(1), runner.bwd(1)), args.steps)
    barrier()
    runner.check_status()
    t = torch.tensor([ms], device=device, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_max = t.item()
    total_flops = flops(w) * world
    value = total_flops / (ms_max * 1e-3) / 1e12

    # ---- end to end through the public operator with host buffers -----------------------------
    from rbf_attention_b200 import ops

    fn = ops.run_triton_rbf if w["softmax"] else ops.run_triton_non_softmax_rbf
    hq, hk, hv, hdo = runner.host
    outs_host = [torch.empty_like(hq).pin_memory() for _ in range(4)]

    # Three streams, double-buffered device inputs: the host->device copy of step s+1, the kernels of step s and the
    # device->host copy of step s-1 overlap (PCIe is full duplex). Every step still moves all of its inputs and all
    # of its results across the bus inside the timed region.
    s_in, s_out = torch.cuda.Stream(device), torch.cuda.Stream(device)
    s_main = torch.cuda.current_stream(device)
    dev_in = [[torch.empty_like(runner.q) for _ in range(4)] for _ in range(2)]
    in_ready = [torch.cuda.Event() for _ in range(2)]
    in_free = [torch.cuda.Event() for _ in range(2)]
    out_done = [torch.cuda.Event() for _ in range(2)]
    keep = [None, None]
    counter = [0]

    def e2e_step():
        i = counter[0] & 1
        counter[0] += 1
        with torch.cuda.stream(s_in):
            s_in.wait_event(in_free[i])            # kernels of the step that last used this buffer set are done
            for dst, src in zip(dev_in[i], (hq, hk, hv, hdo)):
                dst.copy_(src, non_blocking=True)
            in_ready[i].record(s_in)
        s_main.wait_event(in_ready[i])
        q, k, v = (t_.detach().requires_grad_(True) for t_ in dev_in[i][:3])
        out = fn(q, k, v, w["causal"])
        out.backward(dev_in[i][3])
        in_free[i].record(s_main)
        results = (out.detach(), q.grad, k.grad, v.grad)
        keep[i] = results                           # keep the tensors alive until their copy has run
        with torch.cuda.stream(s_out):
            s_out.wait_event(in_free[i])
            s_out.wait_event(out_done[i ^ 1])       # one device->host copy at a time into the pinned result buffers
            for dst, src in zip(outs_host, results):
                dst.copy_(src, non_blocking=True)
                src.record_stream(s_out)
            out_done[i].record(s_out)
        s_main.wait_event(out_done[i ^ 1])          # the timed stream ends only after the previous step's read-back

    def e2e_flush():
        s_main.wait_event(out_done[(counter[0] - 1) & 1])

    for ev in in_free + out_done:
        ev.record(s_main)
    e2e_steps = max(2, min(args.steps, 10))
    for _ in range(2):
        e2e_step()
    e2e_flush()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record()
    for _ in range(e2e_steps):
        e2e_step()
    e2e_flush()
    e1.record()
    torch.cuda.synchronize()
    e2e_ms = e0.elapsed_time(e1) / e2e_steps
    t = torch.tensor([e2e_ms], device=device, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    e2e_value = total_flops / (t.item() * 1e-3) / 1e12
    tensor_bytes = hq.numel() * hq.element_size()

    if rank == 0:
        peak, peak_src = measured_peaks()
        # dominant kernel: algorithmic GEMMs per launch - forward 2 (S, PV); dK/dV kernel 4 (S, dP, dV, dK);
        # dQ kernel 1 (dQ; its S and dP are recomputation and are not counted)
        # single-kernel backward: all 5
        gemms = {"fwd": 2, "bwd_fused": 5} if fused else {"fwd": 2, "bwd_dkdv": 4, "bwd_dq": 1}
        # dram__bytes_read.sum + dram__bytes_write.sum of one launch, from the ncu capture of a quarter of the batch
        # (profiles/ncu_full_fwd_bwd_fused_config2_quarter.md), times four: traffic grows in proportion to B
        ncu_traffic = {("config2", "bwd_fused"): 4 * (109.726720e6 + 30.068992e6),
                       ("config2", "fwd"): 4 * (54.800640e6 + 2.691584e6)}
        dom = max(gemms, key=lambda n: phase_ms[n])
        unit_flops = 2.0 * w["B"] * w["H"] * float(w["N"]) ** 2 * w["D"] * (0.5 if w["causal"] else 1.0)
        achieved = gemms[dom] * unit_flops / (phase_ms[dom] * 1e-3) / 1e12
        cpu_tf, cores, pairs, pair_s = cpu_pairs_per_second(w)
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_max, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": args.workload, **{k_: w[k_] for k_ in ("B", "H", "N", "D", "causal", "softmax")},
                       "per_gpu_batch_heads": w["B"] * w["H"], "parallelism": f"bh-shard x{world}, no collective",
                       "l2": "inputs+outputs per step (>= 0.5 GB) exceed the 126 MB L2",
                       "tolerance": "bf16 operands, fp32 accumulate; rel-L2 <= 6e-3 vs fp32 oracle (tests/)"},
            "frac_of_peak": value / world / peak,
            "phase_ms": phase_ms,
            "roofline": {"bound": "tensor", "kernel": dom, "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
                         "frac": achieved / peak, "traffic": ncu_traffic.get((args.workload, dom)),
                         "traffic_unit": "bytes per launch (ncu, quarter batch x 4)", "peak_source": peak_src,
                         "algorithmic_gemms_per_launch": gemms[dom]},
            "cpu_baseline": {"value": cpu_tf, "unit": UNIT, "cores": cores, "kind": "port",
                             "sample": f"{pairs} x one (batch, head) pair at full N (fp32 PyTorch CPU math, "
                                       f"{pair_s:.2f} s per pair), scaled by FLOPs"},
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": 4 * tensor_bytes,
                    "d2h_bytes_per_step": 4 * tensor_bytes, "ms_per_step": t.item(), "steps": e2e_steps},
            # per step: forward = pre-pass + main; backward = pre-pass + (single kernel + dQ convert | dK/dV + dQ)
            "gpu_launches": 5 * args.steps,
            "clocks": clocks.summary(),
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def run_profile_case(args, w):
    """Warm-up steps, then ``--steps`` forward+backward passes on cuda:0 and nothing else."""
    import torch

    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    runner = DeviceRunner(w, device, seed=1000)
    for _ in range(args.warmup):
        runner.step()
    ms = time_loop(torch, runner.step, args.steps)
    runner.check_status()
    print(f"profile case {w}: {ms:.3f} ms per step", flush=True)


# ---------------------------------------------------------------------------------------------
# configuration 5: data-parallel language-model training step (tokens/s)
# ---------------------------------------------------------------------------------------------
LM = dict(vocab=50257, d_model=512, layers=8, heads=8, seq=1024, batch=64, registers=4)
LM_METRIC, LM_UNIT = "lm_train_tokens_per_s", "tokens/s"


def lm_model(attention_type, dtype, device):
    import torch

    from rbf_attention_b200 import lm

    torch.manual_seed(0)
    model = lm.CausalLM(LM["vocab"], LM["d_model"], LM["layers"], LM["heads"], max_seq_len=LM["seq"],
                        pos_emb_type="rope", num_registers=LM["registers"], attention_type=attention_type)
    return model.to(device=device, dtype=dtype)


def lm_cpu_tokens_per_second(steps=1, batch=1, seq=256):
    """The reference's CPU path for this model: fp32, materialised attention (rbf_slow), AdamW step, on all host
    threads, on a bounded sample (batch x seq tokens per step). Returns (tokens/s, threads, description)."""
    import torch

    from rbf_attention_b200 import lm

    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    model = lm_model("rbf_slow", torch.float32, "cpu")
    opt = torch.optim.AdamW(model.parameters(), lr=1e-4)
    ids = lm.zipf_token_ids(batch, seq + 1, LM["vocab"], seed=0)

    def step():
        logits, _ = model(ids[:, :-1])
        loss = torch.nn.functional.cross_entropy(logits.reshape(-1, LM["vocab"]), ids[:, 1:].reshape(-1))
        loss.backward()
        opt.step()
        opt.zero_grad(set_to_none=True)

    step()
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    dt = time.perf_counter() - t0
    return batch * seq * steps / dt, threads, f"{batch} sequence(s) of {seq} tokens per step, fp32, rbf_slow attention, AdamW"


def run_lm(args, rank, world, local_rank):
    import torch
    import torch.distributed as dist

    from rbf_attention_b200 import lm

    cfg = {"workload": "config5_lm", "model": f"CausalLM {LM['layers']}x{LM['d_model']}, {LM['heads']} heads x 64, "
           f"MLP 4x, {LM['registers']} register tokens, SuSiE, vocab {LM['vocab']}", "global_batch": LM["batch"] * world,
           "seq_len": LM["seq"], "parallelism": f"dp{world}", "optimizer": "AdamW (fused), bf16 weights"}
    if args.impl == "reference":
        if rank != 0:
            return
        tps, threads, sample = lm_cpu_tokens_per_second(steps=max(1, min(args.steps, 3)))
        print(json.dumps({
            "impl": "reference", "metric": LM_METRIC, "value": tps, "unit": LM_UNIT, "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": None, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": cfg,
            "cpu_baseline": {"value": tps, "unit": LM_UNIT, "cores": threads, "kind": "port", "sample": sample},
            "e2e": {"value": tps, "unit": LM_UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}), flush=True)
        return

    device = torch.device("cuda", local_rank)
    torch.cuda.set_device(device)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    model = lm_model("rbf_triton", torch.bfloat16, device)
    net = torch.nn.parallel.DistributedDataParallel(model, device_ids=[local_rank], gradient_as_bucket_view=True) \
        if world > 1 else model
    opt = torch.optim.AdamW(model.parameters(), lr=1e-4, fused=True)
    ids_host = lm.zipf_token_ids(LM["batch"], LM["seq"] + 1, LM["vocab"], seed=100 + rank).pin_memory()
    ids_dev = ids_host.to(device)
    loss_host = torch.zeros((), dtype=torch.float32).pin_memory()

    def step(ids):
        logits, _ = net(ids[:, :-1])
        loss = torch.nn.functional.cross_entropy(logits.view(-1, LM["vocab"]), ids[:, 1:].reshape(-1))
        loss.backward()
        opt.step()
        opt.zero_grad(set_to_none=True)
        return loss

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        step(ids_dev)
    barrier()
    with ClockSampler(local_rank) as clocks:
        ms = time_loop(torch, lambda: step(ids_dev), args.steps)
    barrier()

    def e2e_step():
        ids = ids_host.to(device, non_blocking=True)
        loss_host.copy_(step(ids).detach(), non_blocking=True)

    e2e_steps = max(2, min(args.steps, 10))
    e2e_step()
    barrier()
    e2e_ms = time_loop(torch, e2e_step, e2e_steps)
    t = torch.tensor([ms, e2e_ms], device=device, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    tokens = LM["batch"] * LM["seq"] * world
    if rank == 0:
        peak, peak_src = measured_peaks()
        n_params = sum(p.numel() for p in model.parameters())
        dense = 6.0 * (n_params - LM["vocab"] * LM["d_model"]) * LM["batch"] * LM["seq"]     # embedding lookup is free
        n_attn = LM["seq"] + LM["registers"]
        attn = LM["layers"] * 14.0 * LM["batch"] * LM["heads"] * n_attn * n_attn * 64 * 0.5
        achieved = (dense + attn) / (t[0].item() * 1e-3) / 1e12
        cpu_tps, cores, sample = lm_cpu_tokens_per_second()
        print(json.dumps({
            "metric": LM_METRIC, "value": tokens / (t[0].item() * 1e-3), "unit": LM_UNIT, "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": t[0].item(), "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "config": cfg,
            "roofline": {"bound": "tensor", "kernel": "whole step (cuBLAS GEMMs dominate; attention is ~9 % of the FLOPs)",
                         "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak, "traffic": None,
                         "peak_source": peak_src},
            "cpu_baseline": {"value": cpu_tps, "unit": LM_UNIT, "cores": cores, "kind": "port", "sample": sample},
            "e2e": {"value": tokens / (t[1].item() * 1e-3), "unit": LM_UNIT,
                    "h2d_bytes_per_step": ids_host.numel() * 8, "d2h_bytes_per_step": 4, "ms_per_step": t[1].item()},
            "gpu_launches": LM["layers"] * 5 * args.steps, "clocks": clocks.summary()}), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="config2", choices=sorted(WORKLOADS) + ["config5_lm"])
    ap.add_argument("--profile-case", action="store_true",
                    help="small case for profilers: a quarter of the workload's batch, kernels only, no JSON line")
    args = ap.parse_args()
    if args.workload == "config5_lm":
        return run_lm(args, int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1")),
                      int(os.environ.get("LOCAL_RANK", "0")))
    w = dict(WORKLOADS[args.workload])
    if args.profile_case:
        w["B"] = max(1, w["B"] // 4)
        return run_profile_case(args, w)
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, w, rank, world)
    else:
        run_ours(args, w, rank, world, local_rank)


if __name__ == "__main__":
    main()
