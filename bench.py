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
all-reduce through DistributedDataParallel when N > 1; ``--compile`` wraps the model in ``torch.compile`` as the
reference's training script does).

The default line also carries, under ``"also"``, the other benchmark configurations timed with the same event loop
(configuration 3 causal and full, configuration 4, the reference's own micro-benchmark shape; at N = 1) and the
language-model step (at every N), and under ``"gpu_baselines"`` the reference's Triton operators and its SDPA
formulation timed on the same GPU when the reference project is staged under ``baseline/_ref/reference``.

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


def config_of(name, w, world):
    """The ``config`` object of the JSON line; both arms build it here so that they describe the same workload."""
    return {"workload": name, **{k_: w[k_] for k_ in ("B", "H", "N", "D", "causal", "softmax")},
            "parallelism": f"bh-shard x{world}, no collective"}


# DRAM bytes (read, write) of ONE launch of the named kernel from ncu captures of a reduced batch, and the factor that
# scales the capture to the full batch (traffic grows in proportion to B). Configuration 2: dram__bytes_read.sum and
# dram__bytes_write.sum of a --set full capture; configurations 3 and 4: dram__bytes.sum.per_second x
# gpu__time_duration.sum of a sections capture (read + write together).
NCU_DRAM_BYTES = {
    ("config2", "bwd_fused"): (109.639680e6, 29.786880e6, 4),
    ("config2", "fwd"): (54.870528e6, 3.142912e6, 4),
    ("config3", "bwd_fused"): (0.256082e12 * 5.218400e-3, 0.0, 2),
    ("config3", "fwd"): (1.167834e12 * 2.020160e-3, 0.0, 2),
    ("config4", "bwd_fused"): (311.094650e9 * 451.008e-6, 0.0, 4),
    ("config4", "fwd"): (327.947988e9 * 182.112e-6, 0.0, 4),
}


def ncu_traffic(workload, kernel):
    rec = NCU_DRAM_BYTES.get((workload, kernel))
    return None if rec is None else (rec[0] + rec[1]) * rec[2]


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as fh:
            d = json.load(fh)
        return float(d["bf16_tflops"]), "measured (MEASURED_PEAKS.json bf16_tflops, burst)"
    return 1590.0, "fallback (1.59 PFLOP/s, earlier measurement on this pool)"


def sustained_peak():
    """The dense bf16 rate a seconds-long GEMM loop holds under the power cap: the fairer denominator for the
    configurations whose steps take tens of milliseconds and run power-capped themselves."""
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as fh:
            d = json.load(fh)
        if "bf16_tflops_sustained" in d:
            return float(d["bf16_tflops_sustained"]), "measured (MEASURED_PEAKS.json bf16_tflops_sustained)"
    return 1400.0, "fallback (about 1.4 PFLOP/s sustained, earlier measurement on this pool)"


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
        "config": config_of(args.workload, w, args.gpus), "timed_on": "host CPU",
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------------------------
# our arm
# ---------------------------------------------------------------------------------------------
class DeviceRunner:
    """Pre-allocated device buffers and raw C-ABI calls (no allocation inside the timed region). ``host=True`` draws
    the inputs on the CPU (seeded) and keeps pinned copies for the end-to-end leg; ``host=False`` draws them on the
    device from a seeded generator (the other configurations, which have no end-to-end leg)."""

    def __init__(self, w, device, seed, host=True, dtype=None):
        import torch

        from rbf_attention_b200 import _lib, synthetic

        self.torch, self.w, self.lib = torch, w, _lib.load()
        self._libmod = _lib
        dtype = dtype or torch.bfloat16
        self.dtype_code = 0 if dtype == torch.bfloat16 else 1
        B, H, N, D = w["B"], w["H"], w["N"], w["D"]
        if host:
            tensors = synthetic.make_inputs(B, H, N, D, seed=seed, dtype=dtype, std=w["std"],
                                            key_norm_sigma=w["key_norm_sigma"])
            self.host = [t.pin_memory() for t in tensors]
            self.q, self.k, self.v, self.do = (t.to(device) for t in tensors)
        else:
            g = torch.Generator(device=device).manual_seed(seed)
            self.host = None
            self.q, self.k, self.v = ((torch.randn(B, H, N, D, device=device, generator=g) * w["std"]).to(dtype)
                                      for _ in range(3))
            self.do = torch.randn(B, H, N, D, device=device, generator=g).to(dtype)
            if w["key_norm_sigma"] > 0:
                f = torch.exp(torch.randn(B, H, N, 1, device=device, generator=g) * w["key_norm_sigma"])
                self.k = (self.k.float() * f).to(dtype)
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
            self.ws.data_ptr(), self.ws.numel(), w["B"], w["H"], w["N"], w["D"], self.s, self.s, self.s, self.s,
            self.dtype_code, int(w["causal"]), int(w["softmax"]), self.scale, self.stream, phases)
        self._libmod.check(rc, "rbf_b200_fwd")

    def bwd(self, phases=7):
        w = self.w
        rc = self.lib.rbf_b200_bwd_phases(
            self.q.data_ptr(), self.k.data_ptr(), self.v.data_ptr(), self.out.data_ptr(), self.lse.data_ptr(),
            self.do.data_ptr(), self.dq.data_ptr(), self.dk.data_ptr(), self.dv.data_ptr(), self.ws.data_ptr(),
            self.ws.numel(), w["B"], w["H"], w["N"], w["D"], self.s, self.s, self.s, self.s, self.s, self.s, self.s,
            self.s, self.dtype_code, int(w["causal"]), int(w["softmax"]), self.scale, self.stream, phases)
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


# Kernel launches of one step: forward = (pre-pass) + main; backward = pre-pass + single kernel + dQ conversion.
LAUNCHES_PER_STEP = 5
# Algorithmic GEMMs per launch of the two main kernels: forward S and PV; the single-kernel backward all five.
GEMMS = {"fwd": 2, "bwd_fused": 5}


def timed_workload(torch, runner, w, steps, warmup, local_rank):
    """Warm-up, then the whole step with CUDA events (the headline), then - directly afterwards, in the same clock
    and power state - the same number of steps once more with events between the kernels of each step, which gives the
    average duration of every phase over steps like the timed ones (a loop over one phase alone, run after a long
    sequence of others, lands in a different power state: on a 1 kW part the clocks drop after about 100 ms of load and
    the same kernel then measures up to 14 % slower). Returns (ms per step, phase times, clocks)."""
    for _ in range(max(warmup, 3)):
        runner.step()
    runner.check_status()
    with ClockSampler(local_rank) as clocks:
        ms = time_loop(torch, runner.step, steps)
        marks = [[torch.cuda.Event(enable_timing=True) for _ in range(5)] for _ in range(steps)]
        for ev in marks:
            ev[0].record()
            runner.fwd(1)
            ev[1].record()
            runner.fwd(2)
            ev[2].record()
            runner.bwd(1)
            ev[3].record()
            runner.bwd(6)
            ev[4].record()
        torch.cuda.synchronize()
    seg = [sum(ev[i].elapsed_time(ev[i + 1]) for ev in marks) / steps for i in range(4)]
    phase_ms = {"fwd": seg[1], "bwd_fused": seg[3], "prepass": seg[0] + seg[2]}
    runner.check_status()
    return ms, phase_ms, clocks.summary()


def roofline_of(workload, w, phase_ms, peak, peak_src):
    dom = max(GEMMS, key=lambda n: phase_ms[n])
    unit_flops = 2.0 * w["B"] * w["H"] * float(w["N"]) ** 2 * w["D"] * (0.5 if w["causal"] else 1.0)
    achieved = GEMMS[dom] * unit_flops / (phase_ms[dom] * 1e-3) / 1e12
    return {"bound": "tensor", "kernel": dom, "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
            "frac": achieved / peak, "traffic": ncu_traffic(workload, dom),
            "traffic_unit": "bytes per launch (ncu capture of a reduced batch, scaled to the full batch)",
            "peak_source": peak_src, "algorithmic_gemms_per_launch": GEMMS[dom]}


def also_attention(torch, device, local_rank, peak, peak_src, steps):
    """The other attention configurations, device-resident, each with its own clock record."""
    out = {}
    for name in ("config3", "config3_full", "config4"):
        w = dict(WORKLOADS[name])
        try:
            runner = DeviceRunner(w, device, seed=2000, host=False)
            ms, phase_ms, clocks = timed_workload(torch, runner, w, steps, 3, local_rank)
            value = flops(w) / (ms * 1e-3) / 1e12
            sus, sus_src = sustained_peak()
            out[name] = {"value": value, "unit": UNIT, "ms_per_step": ms, "steps": steps, "phase_ms": phase_ms,
                         "frac_of_peak": value / peak, "frac_of_sustained_peak": value / sus,
                         "sustained_peak": sus, "sustained_peak_source": sus_src,
                         "roofline": roofline_of(name, w, phase_ms, peak, peak_src),
                         "clocks": clocks, "config": config_of(name, w, 1)}
            del runner
        except Exception as exc:   # the headline must survive a failure here
            out[name] = {"error": repr(exc)[:300]}
        torch.cuda.empty_cache()
    # The reference's own micro-benchmark shape (its rbf_attention.py: B4 H8 D64 fp16 causal, N = 1024 ... 8192),
    # forward and backward milliseconds like its plots: backward = (forward + backward) - forward.
    shape = {}
    for n in (1024, 2048, 4096, 8192):
        w = dict(B=4, H=8, N=n, D=64, causal=True, softmax=True, std=1.0, key_norm_sigma=0.0)
        try:
            runner = DeviceRunner(w, device, seed=3000 + n, host=False, dtype=torch.float16)
            for _ in range(5):
                runner.step()
            fwd = time_loop(torch, runner.fwd, 20)
            both = time_loop(torch, runner.step, 20)
            runner.check_status()
            shape[str(n)] = {"fwd_ms": fwd, "bwd_ms": both - fwd, "tflops": flops(w) / (both * 1e-3) / 1e12}
            del runner
        except Exception as exc:
            shape[str(n)] = {"error": repr(exc)[:300]}
    out["reference_benchmark_shape"] = {"dtype": "fp16", "B": 4, "H": 8, "D": 64, "causal": True, "by_N": shape}
    torch.cuda.empty_cache()
    return out


def also_layer(torch, device):
    """The reference's layer benchmark (its rbf_attention.py run_layer_benchmarks: CustomCausalAttention with 8 heads
    x 64, fp16, batch 4, "RBF Triton + SuSiE" with and without XSA; forward under no_grad, backward = forward+backward
    - forward) on the block operator, and on the operator-by-operator path for comparison; plus the streaming
    kernels of the block (q/k preparation, its parameter gradients, XSA) alone against the HBM roofline."""
    import ctypes as ct

    from rbf_attention_b200 import _lib, attention

    out = {"dtype": "fp16", "batch": 4, "heads": 8, "head_dim": 64, "by_N": {}}
    fused_flag = attention.CustomCausalAttention._fused_block
    try:
        for n in (1024, 2048, 4096, 8192):
            x = torch.randn(4, n, 512, device=device, dtype=torch.float16, requires_grad=True)
            dout = torch.randn_like(x)
            rec = {}
            for label, xsa, fused in (("block_operator", False, True), ("operator_by_operator", False, False),
                                      ("block_with_xsa", True, True)):
                torch.manual_seed(0)
                layer = attention.CustomCausalAttention(8, 512, max_seq_len=8192, use_rope=True, attention_type="rbf_triton",
                                                        apply_xsa=xsa).to(device, torch.float16)
                attention.CustomCausalAttention._fused_block = fused_flag if fused else (lambda self, qkv: False)

                def fwd_bwd():
                    x.grad = None
                    y, _ = layer(x)
                    y.backward(dout)

                for _ in range(3):
                    fwd_bwd()
                with torch.no_grad():
                    fwd = time_loop(torch, lambda: layer(x)[0], 20)
                both = time_loop(torch, fwd_bwd, 20)
                rec[label] = {"fwd_ms": fwd, "bwd_ms": both - fwd}
                if label == "block_operator":
                    # the same forward + backward replayed from a CUDA graph: what the layer costs on the device once
                    # the host's launch rate (about 85 launches per iteration) is out of the way
                    try:
                        side = torch.cuda.Stream(device)
                        side.wait_stream(torch.cuda.current_stream(device))
                        with torch.cuda.stream(side):
                            for _ in range(3):
                                fwd_bwd()
                        torch.cuda.current_stream(device).wait_stream(side)
                        graph = torch.cuda.CUDAGraph()
                        x.grad = None
                        with torch.cuda.graph(graph):
                            y, _ = layer(x)
                            y.backward(dout)
                        for _ in range(3):
                            graph.replay()
                        rec["block_operator_cuda_graph"] = {"fwd_plus_bwd_ms": time_loop(torch, graph.replay, 20)}
                        del graph
                    except Exception as exc:      # capture is an extra: the eager numbers above stand without it
                        rec["block_operator_cuda_graph"] = {"error": repr(exc)[:200]}
            out["by_N"][str(n)] = rec
    except Exception as exc:
        out["error"] = repr(exc)[:300]
    finally:
        attention.CustomCausalAttention._fused_block = fused_flag
    # the block's streaming kernels at the language model's shape (B64 S1028 H8 D64, bf16): achieved HBM bandwidth
    try:
        lib = _lib.load()
        B, S, H, D, R = 64, 1028, 8, 64, 4
        E = H * D
        qkv = torch.randn(B, S, 3 * E, device=device, dtype=torch.bfloat16)
        pw = torch.rand(H, D // 2, device=device) + 0.2
        rp = torch.randn(H, R, D, device=device) * 0.1
        table = attention.get_unrotated_sinusoids(S, D, device).contiguous()
        qk = torch.empty(2, B, S, H, D, device=device, dtype=torch.bfloat16)
        q, k = qk[0].permute(0, 2, 1, 3), qk[1].permute(0, 2, 1, 3)
        nb = lib.rbf_b200_workspace_bytes(B, H, S, D, 1, 0)
        ws = torch.empty(nb, dtype=torch.uint8, device=device)
        nb2 = lib.rbf_b200_qkv_prep_bwd_workspace_bytes(B, S, H, D, R)
        ws2 = torch.empty(nb2, dtype=torch.uint8, device=device)
        d_pw = torch.empty(H, D // 2, device=device)
        d_rp = torch.empty(H, R, D, device=device)
        o2 = torch.empty(B, H, S, D, device=device, dtype=torch.bfloat16)
        stream = torch.cuda.current_stream(device).cuda_stream
        s3 = _lib.strides3
        n_pad = (S + 127) // 128 * 128
        tensor = B * S * E * 2

        def prep():
            _lib.check(lib.rbf_b200_qkv_prep(qkv.data_ptr(), pw.data_ptr(), rp.data_ptr(), 1, table.data_ptr(), q.data_ptr(),
                                             k.data_ptr(), s3(q), s3(k), ws.data_ptr(), nb, B, S, H, D, R, 0, 1, 0.125, stream), "prep")

        def prep_bwd():
            _lib.check(lib.rbf_b200_qkv_prep_bwd(q.data_ptr(), k.data_ptr(), s3(q), s3(k), table.data_ptr(), d_pw.data_ptr(),
                                                 d_rp.data_ptr(), ws2.data_ptr(), nb2, B, S, H, D, R, 0, stream), "prep_bwd")

        def xsa():
            _lib.check(lib.rbf_b200_xsa_fwd(q.data_ptr(), k.data_ptr(), o2.data_ptr(), s3(q), s3(k), s3(o2), B, H, S, D, 0, stream), "xsa")

        def xsa_bwd():
            _lib.check(lib.rbf_b200_xsa_bwd(o2.data_ptr(), q.data_ptr(), k.data_ptr(), qk[0].permute(0, 2, 1, 3).data_ptr(),
                                            o2.data_ptr(), s3(o2), s3(q), s3(k), s3(q), s3(o2), B, H, S, D, 0, stream), "xsa_bwd")

        hbm = None
        path = os.path.join(ROOT, "MEASURED_PEAKS.json")
        if os.path.exists(path):
            with open(path) as fh:
                hbm = float(json.load(fh).get("hbm_gbs", 0.0)) or None
        kernels = {}
        for name, fn, nbytes in (("qkv_prep", prep, 4 * tensor + B * H * n_pad * 32),        # read q, k; write q', k', slabs
                                 ("qkv_prep_bwd", prep_bwd, 2 * tensor),                     # read dq', dk'
                                 ("xsa_fwd", xsa, 3 * tensor), ("xsa_bwd", xsa_bwd, 5 * tensor)):
            for _ in range(3):
                fn()
            ms = time_loop(torch, fn, 20)
            gbs = nbytes / (ms * 1e-3) / 1e9
            kernels[name] = {"ms": ms, "algorithmic_bytes": nbytes, "achieved_gbs": gbs,
                             "frac_of_hbm_peak": None if hbm is None else gbs / hbm}
        out["streaming_kernels"] = {"shape": "B64 S1028 H8 D64 bf16 (one layer of configuration 5)", "hbm_peak_gbs": hbm,
                                    "kernels": kernels}
    except Exception as exc:
        out["streaming_kernels"] = {"error": repr(exc)[:300]}
    torch.cuda.empty_cache()
    return out


def gpu_baselines(torch, w, runner, steps=10):
    """The reference project's own GPU implementations on this GPU and workload, for comparison only: its Triton
    operators (JIT-compiled and autotuned here by the installed Triton) and its SDPA formulation on an augmented
    head dim. Needs the reference staged under baseline/_ref/reference; the first call pays JIT and autotuning."""
    ref_dir = os.path.join(ROOT, "baseline", "_ref", "reference")
    if not os.path.exists(os.path.join(ref_dir, "rbf_attention.py")):
        return {"unavailable": "the reference project is not staged under baseline/_ref/reference"}
    import importlib.util
    import types

    for name in ("matplotlib", "matplotlib.pyplot"):       # the reference imports it for its plots; not installed
        sys.modules.setdefault(name, types.ModuleType(name))
    try:
        spec = importlib.util.spec_from_file_location("rbf_attention_reference", os.path.join(ref_dir, "rbf_attention.py"))
        ref = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(ref)
    except Exception as exc:
        return {"unavailable": f"import of the reference failed: {exc!r}"[:300]}
    q, k, v = (t.detach().clone().requires_grad_(True) for t in (runner.q, runner.k, runner.v))
    arms = {"triton_reference": (ref.run_triton_rbf if w["softmax"] else ref.run_triton_non_softmax_rbf)}
    if w["softmax"]:
        arms["sdpa_augmented"] = ref.rbf_math_forward
    out = {}
    for name, fn in arms.items():
        def step():
            o = fn(q, k, v, w["causal"])
            o.backward(runner.do)
            q.grad = k.grad = v.grad = None

        try:
            t0 = time.perf_counter()
            step()
            torch.cuda.synchronize()
            first = time.perf_counter() - t0
            for _ in range(3):
                step()
            with torch.no_grad():
                fwd = time_loop(torch, lambda: fn(q, k, v, w["causal"]), steps)
            ms = time_loop(torch, step, steps)
            out[name] = {"value": flops(w) / (ms * 1e-3) / 1e12, "unit": UNIT, "ms_per_step": ms, "fwd_ms": fwd,
                         "first_call_s": first}
        except Exception as exc:
            out[name] = {"unavailable": repr(exc)[:300]}
    return out


def e2e_leg(torch, dist, runner, w, device, world, steps):
    """End to end through the public operator with host buffers. Three streams, double-buffered device inputs: the
    host->device copy of step s+1, the kernels of step s and the device->host copy of step s-1 overlap (PCIe is full
    duplex). Every step moves all of its inputs and all of its results across the bus inside the timed region.
    Returns (ms per step, ms per step of the same loop with the kernels left out = the copy floor, ms of one step's
    transfers in the slower single direction with the bus otherwise idle)."""
    from rbf_attention_b200 import ops

    fn = ops.run_triton_rbf if w["softmax"] else ops.run_triton_non_softmax_rbf
    hq, hk, hv, hdo = runner.host
    outs_host = [torch.empty_like(hq).pin_memory() for _ in range(4)]
    s_in, s_out = torch.cuda.Stream(device), torch.cuda.Stream(device)
    s_main = torch.cuda.current_stream(device)
    dev_in = [[torch.empty_like(runner.q) for _ in range(4)] for _ in range(2)]
    dev_out = [torch.empty_like(runner.q) for _ in range(4)]          # stand-in results of the copy-only loop
    in_ready = [torch.cuda.Event() for _ in range(2)]
    in_free = [torch.cuda.Event() for _ in range(2)]
    out_done = [torch.cuda.Event() for _ in range(2)]
    keep = [None, None]
    counter = [0]

    in_flight = []                                   # one event per step whose read-back has been enqueued

    def step(compute=True):
        # The host stays at most three steps ahead of the device (a stream of real batches could not be enqueued
        # earlier either): with the whole run enqueued at once, the caching allocator never sees a finished
        # read-back when it is asked for the next step's tensors and grows by a step's worth of memory per step.
        if len(in_flight) >= 3:
            in_flight.pop(0).synchronize()
        i = counter[0] & 1
        counter[0] += 1
        with torch.cuda.stream(s_in):
            s_in.wait_event(in_free[i])            # kernels of the step that last used this buffer set are done
            for dst, src in zip(dev_in[i], (hq, hk, hv, hdo)):
                dst.copy_(src, non_blocking=True)
            in_ready[i].record(s_in)
        s_main.wait_event(in_ready[i])
        if compute:
            q, k, v = (t_.detach().requires_grad_(True) for t_ in dev_in[i][:3])
            out = fn(q, k, v, w["causal"])
            out.backward(dev_in[i][3])
            results = (out.detach(), q.grad, k.grad, v.grad)
        else:
            results = tuple(dev_out)
        in_free[i].record(s_main)
        keep[i] = results                           # keep the tensors alive until their copy has run
        with torch.cuda.stream(s_out):
            s_out.wait_event(in_free[i])
            s_out.wait_event(out_done[i ^ 1])       # one device->host copy at a time into the pinned result buffers
            for dst, src in zip(outs_host, results):
                dst.copy_(src, non_blocking=True)
                src.record_stream(s_out)
            out_done[i].record(s_out)
            done = torch.cuda.Event()
            done.record(s_out)
            in_flight.append(done)
        s_main.wait_event(out_done[i ^ 1])          # the timed stream ends only after the previous step's read-back

    def flush():
        s_main.wait_event(out_done[(counter[0] - 1) & 1])

    def timed(compute):
        for ev in in_free + out_done:
            ev.record(s_main)
        for _ in range(2):
            step(compute)
        flush()
        if world > 1:
            dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        for _ in range(steps):
            step(compute)
        flush()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / steps

    def one_way(to_device):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        for _ in range(4):
            for d, h in zip(dev_in[0], (hq, hk, hv, hdo)):
                (d if to_device else h).copy_(h if to_device else d, non_blocking=True)
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / 4

    return timed(True), timed(False), max(one_way(True), one_way(False))


def run_ours(args, w, rank, world, local_rank):
    import torch
    import torch.distributed as dist

    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device: the product has no CPU path")
    device = torch.device("cuda", local_rank)
    torch.cuda.set_device(device)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(values):
        t = torch.tensor(values, device=device, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.tolist()

    peak, peak_src = measured_peaks()
    runner = DeviceRunner(w, device, seed=1000 + rank)
    for _ in range(max(args.warmup, 3)):
        runner.step()
    runner.check_status()

    # ---- device-resident throughput: exactly K steps, max over ranks --------------------------
    barrier()
    ms, phase_ms, clocks = timed_workload(torch, runner, w, args.steps, 0, local_rank)
    barrier()
    (ms_max,) = max_over_ranks([ms])
    total_flops = flops(w) * world
    value = total_flops / (ms_max * 1e-3) / 1e12

    # ---- end to end through the public operator with host buffers -----------------------------
    e2e_steps = max(2, min(args.steps, 200))   # first transfer in and last transfer out are not overlapped: (K + 1) / K
    e2e_ms, floor_ms, one_way_ms = max_over_ranks(list(e2e_leg(torch, dist, runner, w, device, world, e2e_steps)))
    tensor_bytes = runner.q.numel() * runner.q.element_size()

    # ---- the other configurations ---------------------------------------------------------------
    also = {}
    baselines = None
    if args.also and args.workload == "config2":
        if world == 1:
            baselines = gpu_baselines(torch, w, runner)
        del runner
        torch.cuda.empty_cache()
        if world == 1:
            also.update(also_attention(torch, device, local_rank, peak, peak_src, max(10, min(args.steps, 20))))
            also["reference_layer_benchmark"] = also_layer(torch, device)
        barrier()
        try:
            also["config5_lm"] = lm_step_record(torch, dist, rank, world, local_rank, steps=8, warmup=3, compile_model=False)
        except Exception as exc:
            also["config5_lm"] = {"error": repr(exc)[:300]}

    if rank == 0:
        cpu_tf, cores, pairs, pair_s = cpu_pairs_per_second(w)
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_max, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": config_of(args.workload, w, world),
            "per_gpu_batch_heads": w["B"] * w["H"],
            "l2": "inputs+outputs per step (>= 0.5 GB) exceed the 126 MB L2",
            "tolerance": "bf16 operands, fp32 accumulate; rel-L2 <= 6e-3 vs fp32 oracle (tests/)",
            "frac_of_peak": value / world / peak,
            "phase_ms": phase_ms,
            "roofline": roofline_of(args.workload, w, phase_ms, peak, peak_src),
            "cpu_baseline": {"value": cpu_tf, "unit": UNIT, "cores": cores, "kind": "port",
                             "sample": f"{pairs} x one (batch, head) pair at full N (fp32 PyTorch CPU math, "
                                       f"{pair_s:.2f} s per pair), scaled by FLOPs"},
            "e2e": {"value": total_flops / (e2e_ms * 1e-3) / 1e12, "unit": UNIT,
                    "h2d_bytes_per_step": 4 * tensor_bytes, "d2h_bytes_per_step": 4 * tensor_bytes,
                    "ms_per_step": e2e_ms, "steps": e2e_steps,
                    # the same three-stream loop with the kernels left out: what the host link alone costs per step
                    "copy_floor_ms": floor_ms,
                    # one step's transfers in the slower direction with the bus otherwise idle (the hard lower bound)
                    "copy_one_direction_ms": one_way_ms},
            "gpu_launches": LAUNCHES_PER_STEP * args.steps,
            "clocks": clocks,
        }
        if also:
            line["also"] = also
        if baselines is not None:
            line["gpu_baselines"] = baselines
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def run_profile_case(args, w):
    """Warm-up steps, then ``--steps`` forward+backward passes on cuda:0 and nothing else."""
    import torch

    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    runner = DeviceRunner(w, device, seed=1000, host=False)
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


def lm_config(world, compile_model):
    return {"workload": "config5_lm", "model": f"CausalLM {LM['layers']}x{LM['d_model']}, {LM['heads']} heads x 64, "
            f"MLP 4x, {LM['registers']} register tokens, SuSiE, vocab {LM['vocab']}", "global_batch": LM["batch"] * world,
            "seq_len": LM["seq"], "parallelism": f"dp{world}", "optimizer": "AdamW (fused), bf16 weights",
            "torch_compile": bool(compile_model)}


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


def lm_step_record(torch, dist, rank, world, local_rank, steps, warmup, compile_model):
    """Times the data-parallel training step (the process group, if any, is already initialised). Returns the record
    on every rank (times are the maximum over ranks)."""
    from rbf_attention_b200 import lm

    device = torch.device("cuda", local_rank)
    model = lm_model("rbf_triton", torch.bfloat16, device)
    net = model
    if world > 1:
        net = torch.nn.parallel.DistributedDataParallel(model, device_ids=[local_rank], gradient_as_bucket_view=True)
    if compile_model:
        net = torch.compile(net)
    opt = torch.optim.AdamW(model.parameters(), lr=1e-4, fused=True)
    ids_host = lm.zipf_token_ids(LM["batch"], LM["seq"] + 1, LM["vocab"], seed=100 + rank).pin_memory()
    ids_dev = ids_host.to(device)
    loss_host = torch.zeros((), dtype=torch.float32).pin_memory()

    def step(ids):
        # the logits keep the vocabulary's padding to a multiple of 64 (-inf columns: same loss, no strided copies)
        logits, _ = net(ids[:, :-1], padded_logits=True)
        loss = lm.cross_entropy(logits, ids[:, 1:])         # loss and d(loss)/d(logits) from one kernel
        loss.backward()
        opt.step()
        opt.zero_grad(set_to_none=True)
        return loss

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(warmup, 3)):
        step(ids_dev)
    barrier()
    with ClockSampler(local_rank) as clocks:
        ms = time_loop(torch, lambda: step(ids_dev), steps)
    barrier()

    def e2e_step():
        ids = ids_host.to(device, non_blocking=True)
        loss_host.copy_(step(ids).detach(), non_blocking=True)

    e2e_steps = max(2, min(steps, 10))
    e2e_step()
    barrier()
    e2e_ms = time_loop(torch, e2e_step, e2e_steps)
    t = torch.tensor([ms, e2e_ms], device=device, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, e2e_ms = t.tolist()
    tokens = LM["batch"] * LM["seq"] * world
    graph_record = None
    if world == 1 and not compile_model:
        graph_record = lm_step_as_cuda_graph(torch, lm, model, ids_host, ids_dev, loss_host, steps, tokens)
    peak, peak_src = measured_peaks()
    n_params = sum(p.numel() for p in model.parameters())
    dense = 6.0 * (n_params - LM["vocab"] * LM["d_model"]) * LM["batch"] * LM["seq"]     # embedding lookup is free
    n_attn = LM["seq"] + LM["registers"]
    attn = LM["layers"] * 14.0 * LM["batch"] * LM["heads"] * n_attn * n_attn * 64 * 0.5
    achieved = (dense + attn) / (ms * 1e-3) / 1e12          # per GPU
    return {
        "metric": LM_METRIC, "value": tokens / (ms * 1e-3), "unit": LM_UNIT, "n_gpus": world, "steps": steps,
        "warmup": max(warmup, 3), "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "config": lm_config(world, compile_model),
        "roofline": {"bound": "tensor", "kernel": "whole step (cuBLAS GEMMs dominate; attention is ~9 % of the FLOPs)",
                     "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak, "traffic": None,
                     "peak_source": peak_src},
        "e2e": {"value": tokens / (e2e_ms * 1e-3), "unit": LM_UNIT, "h2d_bytes_per_step": ids_host.numel() * 8,
                "d2h_bytes_per_step": 4, "ms_per_step": e2e_ms},
        # the library's own launches per step: per layer 6 forward (2 LayerNorm, q/k preparation, attention, status
        # post, GELU) and 18 backward (GELU + its bias sum 2, three bias sums 6, 2 LayerNorm 4, attention pre-pass,
        # main kernel, dQ conversion, status post, position gradients 2); per model the last LayerNorm (1 + 2), the
        # loss kernel and its rescale
        "gpu_launches": (LM["layers"] * 24 + 5) * steps, "clocks": clocks.summary(),
        **({"cuda_graph": graph_record} if graph_record is not None else {})}


def lm_step_as_cuda_graph(torch, lm, model, ids_host, ids_dev, loss_host, steps, tokens):
    """The same training step (forward, loss, backward, AdamW) captured once into a CUDA graph and replayed: what the
    eager step loses to launch gaps between its ~700 kernels. One GPU only (the data-parallel wrapper is not captured).
    Returns a sub-record; a capture that fails is reported, not raised."""
    try:
        opt = torch.optim.AdamW(model.parameters(), lr=1e-4, fused=True, capturable=True)
        static_ids = ids_dev.clone()

        def step():
            logits, _ = model(static_ids[:, :-1], padded_logits=True)
            loss = lm.cross_entropy(logits, static_ids[:, 1:])
            loss.backward()
            opt.step()
            return loss

        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(3):
                opt.zero_grad(set_to_none=True)
                step()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        opt.zero_grad(set_to_none=True)
        with torch.cuda.graph(graph):
            static_loss = step()
        for _ in range(2):
            graph.replay()
        torch.cuda.synchronize()
        first = float(static_loss.detach())
        ms = time_loop(torch, graph.replay, steps)
        last = float(static_loss.detach())

        def e2e_step():
            static_ids.copy_(ids_host, non_blocking=True)
            graph.replay()
            loss_host.copy_(static_loss.detach(), non_blocking=True)

        e2e_step()
        e2e_ms = time_loop(torch, e2e_step, max(2, min(steps, 10)))
        import math
        return {"ms_per_step": ms, "value": tokens / (ms * 1e-3), "unit": LM_UNIT,
                "e2e": {"value": tokens / (e2e_ms * 1e-3), "unit": LM_UNIT, "ms_per_step": e2e_ms},
                "loss_before_and_after_the_timed_replays": [first, last],
                "trains": bool(math.isfinite(last) and last < first)}
    except Exception as exc:   # noqa: BLE001 - reported in the record
        return {"error": f"{type(exc).__name__}: {str(exc)[:300]}"}


def run_lm(args, rank, world, local_rank):
    import torch
    import torch.distributed as dist

    if args.impl == "reference":
        if rank != 0:
            return
        tps, threads, sample = lm_cpu_tokens_per_second(steps=max(1, min(args.steps, 3)))
        print(json.dumps({
            "impl": "reference", "metric": LM_METRIC, "value": tps, "unit": LM_UNIT, "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": None, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": lm_config(args.gpus, args.compile),
            "cpu_baseline": {"value": tps, "unit": LM_UNIT, "cores": threads, "kind": "port", "sample": sample},
            "e2e": {"value": tps, "unit": LM_UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}), flush=True)
        return

    device = torch.device("cuda", local_rank)
    torch.cuda.set_device(device)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    rec = lm_step_record(torch, dist, rank, world, local_rank, args.steps, args.warmup, args.compile)
    if rank == 0:
        cpu_tps, cores, sample = lm_cpu_tokens_per_second()
        rec["cpu_baseline"] = {"value": cpu_tps, "unit": LM_UNIT, "cores": cores, "kind": "port", "sample": sample}
        print(json.dumps(rec), flush=True)
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
    ap.add_argument("--compile", action="store_true", help="config5_lm: wrap the model in torch.compile")
    ap.add_argument("--no-also", dest="also", action="store_false",
                    help="headline workload only: skip the other configurations and the GPU comparison arms")
    ap.add_argument("--profile-case", action="store_true",
                    help="small case for profilers: a quarter of the workload's batch, kernels only, no JSON line")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.workload == "config5_lm":
        return run_lm(args, rank, world, local_rank)
    w = dict(WORKLOADS[args.workload])
    if args.profile_case:
        w["B"] = max(1, w["B"] // 4)
        return run_profile_case(args, w)
    if args.impl == "reference":
        run_reference(args, w, rank, world)
    else:
        run_ours(args, w, rank, world, local_rank)


if __name__ == "__main__":
    main()
