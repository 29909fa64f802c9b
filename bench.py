"""Benchmark of the gated-MLP hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--workload NAME]

One step = one pass of the hot path over one batch of synthetic input. The default
workload is the Llama-3-8B MLP forward in bf16 (M=8192 tokens, hidden 4096,
intermediate 14336), the configuration the headline metric is quoted on. With
N > 1 (launched by torch.distributed.run, one rank per GPU) every rank runs the
same per-GPU batch on replicated weights: token sharding, no data-path
collective, weak scaling.

Prints ONE JSON line (rank 0). `value` is device-timed throughput with inputs
resident in HBM; `e2e` is the same metric through the public module API with
pinned-host input and output buffers and both copies inside the timed region.
`--impl reference` times the CPU oracle (the restatement of the reference's
torch-eager path) on the host cores on a bounded sample of the same workload.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

WORKLOADS = {
    # name: (M, K, N, bias, dropout_p, mode)
    "llama3-8b-mlp-fwd-bf16": dict(M=8192, K=4096, N=14336, bias=False, p=0.0, mode="fwd"),
    "train-fwd-bwd-bf16": dict(M=16384, K=2048, N=8192, bias=True, p=0.1, mode="fwd+bwd"),
    "prefill-fwd-bf16": dict(M=65536, K=8192, N=28672, bias=False, p=0.0, mode="fwd"),
    "prefill-fwd-bwd-bf16": dict(M=65536, K=8192, N=28672, bias=False, p=0.0, mode="fwd+bwd"),
    # skinny-M inference through the weight-streaming kernels: HBM-bound, metric in GB/s
    "decode-m1-bf16": dict(M=1, K=8192, N=28672, bias=False, p=0.0, mode="decode"),
    "decode-m8-bf16": dict(M=8, K=8192, N=28672, bias=False, p=0.0, mode="decode"),
    "decode-m32-bf16": dict(M=32, K=8192, N=28672, bias=False, p=0.0, mode="decode"),
    "decode-m64-bf16": dict(M=64, K=8192, N=28672, bias=False, p=0.0, mode="decode"),
}
NOMINAL_HBM_GBS = 8000.0
FALLBACK_HBM_GBS = 6650.0
# DRAM bytes (read + write) of one decode forward at M=1 (gate/up kernel 946.6 MB + down projection
# 474.2 MB), from the ncu capture summarised in profiles/decode_stream_kernels_k8192_n28672.md.
DECODE_M1_DRAM_TRAFFIC_BYTES = 1.4208e9
NOMINAL_BF16_TFLOPS = 2250.0
FALLBACK_BF16_TFLOPS = 1590.0
# DRAM bytes (read + write) of one launch of the gate/up kernel at the default workload,
# from the ncu capture summarised in profiles/gateup_pair_kernel_llama8b_fwd.md.
K1_DRAM_TRAFFIC_BYTES = 1.265e9


def flops_per_step(w) -> float:
    mkn = w["M"] * w["K"] * w["N"]
    return (6.0 if w["mode"] in ("fwd", "decode") else 18.0) * mkn


def decode_bytes_per_step(w) -> float:
    """Algorithmic bytes of one decode forward: the three bf16 weight matrices once, x in, y out."""
    return 2.0 * (3.0 * w["K"] * w["N"] + 2.0 * w["M"] * w["K"])


def measured_hbm_peak():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return float(json.loads(p.read_text())["hbm_gbs"]), "measured copy bandwidth (MEASURED_PEAKS.json hbm_gbs)"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, "fallback (MEASURED_PEAKS.json absent)"


def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            d = json.loads(p.read_text())
            return float(d["bf16_tflops"]), "measured burst (MEASURED_PEAKS.json bf16_tflops)"
        except Exception:
            pass
    return FALLBACK_BF16_TFLOPS, "fallback (MEASURED_PEAKS.json absent)"


# ------------------------------------------------------------------ clocks --
class ClockSampler:
    """Samples SM clock and throttle reasons through NVML while the timed region runs."""

    def __init__(self, index: int, period_s: float = 0.02):
        self.index, self.period = index, period_s
        self.samples, self.reasons = [], set()
        self.max_mhz = None
        self._stop = threading.Event()
        self._thr = None
        try:
            import pynvml

            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _loop(self):
        nv = self.nv
        names = {
            "hw_slowdown": getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8),
            "sw_power_cap": getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4),
            "hw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40),
            "sw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20),
            "hw_power_brake": getattr(nv, "nvmlClocksEventReasonHwPowerBrakeSlowdown", 0x80),
        }
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                try:
                    mask = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                except Exception:
                    mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for k, bit in names.items():
                    if mask & bit:
                        self.reasons.add(k)
            except Exception:
                pass
            self._stop.wait(self.period)

    def __enter__(self):
        if self.nv is not None:
            self._thr = threading.Thread(target=self._loop, daemon=True)
            self._thr.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        if self._thr is not None:
            self._thr.join(timeout=2)

    def summary(self):
        return {
            "sm_mhz": statistics.median(self.samples) if self.samples else None,
            "sm_max_mhz": self.max_mhz,
            "reasons": sorted(self.reasons),
            "samples": len(self.samples),
        }


# ------------------------------------------------------------ CPU baseline --
def cpu_baseline(w, budget_s: float = 12.0):
    """Times the CPU oracle (fp32, all host threads) on a row sample of the workload."""
    from oracle import gated_mlp_oracle as orc

    torch.set_num_threads(os.cpu_count() or 1)
    ms = min(w["M"], 1024)
    case = orc.make_case(ms, w["K"], w["N"], w["bias"], torch.bfloat16, seed=0, w_std=0.02, dy_std=1e-2)
    x, wg, bg, wu, bu, wd, bd, dy = case.f32()
    fl = flops_per_step(w) * ms / w["M"]

    def run():
        if w["mode"] in ("fwd", "decode"):
            orc.forward(x, wg, bg, wu, bu, wd, bd)
        else:
            orc.forward(x, wg, bg, wu, bu, wd, bd)
            orc.backward(x, wg, bg, wu, bu, wd, bd, dy)

    run()  # warm-up
    times = []
    t_end = time.perf_counter() + budget_s
    while len(times) < 3 or (time.perf_counter() < t_end and len(times) < 20):
        t0 = time.perf_counter()
        run()
        times.append(time.perf_counter() - t0)
    t = statistics.median(times)
    if w["mode"] == "decode":
        # the whole batch fits the sample; fp32 weights, so the CPU streams twice the bf16 bytes the metric counts
        return {
            "value": decode_bytes_per_step(w) / t / 1e9, "unit": "GB/s", "cores": torch.get_num_threads(),
            "kind": "port",
            "sample": f"all {ms} token rows, full K and N, fp32 torch CPU, median of {len(times)} runs "
                      f"({t * 1e3:.0f} ms each); bytes counted as for the bf16 path",
        }, t, ms
    return {
        "value": fl / t / 1e12, "unit": "TFLOP/s", "cores": torch.get_num_threads(), "kind": "port",
        "sample": f"{ms} of {w['M']} token rows, full K and N, fp32 torch CPU, median of {len(times)} runs "
                  f"({t * 1e3:.0f} ms each)",
    }, t, ms


def run_reference(args, w, name):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    base, t, ms = cpu_baseline(w, budget_s=max(5.0, min(60.0, 0.5 * (args.steps + args.warmup))))
    decode = w["mode"] == "decode"
    line = {
        "impl": "reference",
        "metric": "gated_mlp_decode_hbm_gbs" if decode else f"gated_mlp_{w['mode'].replace('+', '_')}_tflops",
        "value": base["value"], "unit": base["unit"], "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": t * 1e3 * w["M"] / ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": name, "M": w["M"], "K": w["K"], "N": w["N"], "bias": w["bias"],
                   "dropout_p": w["p"], "pass": w["mode"],
                   "note": "CPU restatement of the reference's torch-eager path (the reference is Python and "
                           "is not present on this machine); ms_per_step extrapolated linearly from the row sample"},
        "cpu_baseline": base,
        "e2e": {"value": base["value"], "unit": base["unit"], "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------- decode ----
def run_decode(args, w, name):
    """M <= 64 tokens through the module's decode path; the metric is algorithmic GB/s of the weight stream.

    Two weight sets alternate between steps, so nothing a step reads was left in L2 by the step before
    (one set is 1.4 GB against 126 MB of L2 anyway). With N > 1 every rank decodes its own batch on
    replicated weights (replicas, no collective)."""
    import __graft_entry__ as entry

    pkg = entry.load_package()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    dist_on = world > 1
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if dist_on:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=dev)
    M, K, N = w["M"], w["K"], w["N"]
    dt = torch.bfloat16
    wgen = torch.Generator(device=dev).manual_seed(7)
    sets = []
    for _ in range(2):
        mlp = pkg.FusedGatedMLP(K, N, bias=w["bias"]).to(dev).to(dt).eval()
        with torch.no_grad():
            for p_ in mlp.parameters():
                p_.copy_((torch.randn(p_.shape, device=dev, generator=wgen) * 0.02).to(dt))
        sets.append(mlp)
    x = torch.randn((M, K), device=dev, dtype=dt, generator=torch.Generator(device=dev).manual_seed(1234 + rank))

    def barrier():
        torch.cuda.synchronize()
        if dist_on:
            dist.barrier()
        torch.cuda.synchronize()

    with torch.no_grad():
        for i in range(max(args.warmup, 3) * 2):
            sets[i & 1](x)
        assert sets[0]._decode_scratch is not None, "the decode path was not taken"
        barrier()
        with ClockSampler(local) as clocks:
            t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            t0.record()
            for i in range(args.steps):
                sets[i & 1](x)
            t1.record()
            barrier()
    elapsed_ms = t0.elapsed_time(t1)

    # end to end: x from pinned host memory, y back to pinned host memory, every step
    x_host = torch.empty((M, K), dtype=dt).pin_memory()
    x_host.copy_(x.cpu())
    y_host = torch.empty((M, K), dtype=dt).pin_memory()
    flip = [0]

    def api_step(x_dev):
        flip[0] ^= 1
        with torch.no_grad():
            return sets[flip[0]](x_dev)

    pipe = pkg.host_pipeline.HostPipeline(api_step, dev, depth=3)
    e2e_steps = max(3, min(args.steps, 200))
    for _ in range(4):
        pipe.submit(y_host, x_host)
    pipe.drain()
    barrier()
    s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s0.record(pipe.s_in)
    for _ in range(e2e_steps):
        pipe.submit(y_host, x_host)
    s1.record(pipe.s_out)
    pipe.drain()
    barrier()
    e2e_ms = s0.elapsed_time(s1)
    status = pkg._lib.status_read(dev)
    if dist_on:
        t = torch.tensor([elapsed_ms, e2e_ms, float(status)], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        elapsed_ms, e2e_ms, status = t[0].item(), t[1].item(), int(t[2].item())
    assert status == 0, f"a kernel recorded a device-side timeout (code {status})"

    if rank == 0:
        nbytes = decode_bytes_per_step(w)
        ms_step = elapsed_ms / args.steps
        value = world * nbytes / (ms_step * 1e-3) / 1e9
        peak, peak_src = measured_hbm_peak()
        line = {
            "metric": "gated_mlp_decode_hbm_gbs", "value": value, "unit": "GB/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": name, "M_per_gpu": M, "K": K, "N": N, "bias": w["bias"], "pass": "decode forward",
                       "parallelism": f"independent replicas x{world}, no collective",
                       "l2": "two weight sets alternate between steps; one set (1.4 GB) exceeds the 126 MB L2"},
            "frac_of_nominal_hbm_peak": value / world / NOMINAL_HBM_GBS,
            "frac_of_measured_hbm_peak": value / world / peak,
            "e2e": {"value": world * nbytes / (e2e_ms / e2e_steps * 1e-3) / 1e9, "unit": "GB/s",
                    "h2d_bytes_per_step": x_host.numel() * 2, "d2h_bytes_per_step": y_host.numel() * 2,
                    "steps": e2e_steps, "ms_per_step": e2e_ms / e2e_steps},
            "gpu_launches": 2 * args.steps,
            "clocks": clocks.summary(),
            "roofline": {
                "kernel": "decode_stream_kernel<MPAD, gate+up> then <MPAD, down>, chained by programmatic dependent "
                          "launch (timed together: timing them apart would break the chain)",
                "bound": "hbm", "achieved": value / world, "peak": peak, "unit": "GB/s", "frac": value / world / peak,
                "peak_source": peak_src, "frac_of_nominal": value / world / NOMINAL_HBM_GBS,
                "traffic": DECODE_M1_DRAM_TRAFFIC_BYTES if M == 1 else None,
                "ms_per_launch": ms_step, "algorithmic_bytes_per_launch": nbytes,
            },
        }
        if world == 1 and not args.no_cpu_baseline:
            base, _, _ = cpu_baseline(w)
            line["cpu_baseline"] = base
        print(json.dumps(line), flush=True)
    if dist_on:
        dist.barrier()
        dist.destroy_process_group()


# ------------------------------------------------------------------- GPU ----
def run_gpu(args, w, name):
    import __graft_entry__ as entry

    pkg = entry.load_package()
    K_ = pkg.ops.kernels
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    dist_on = world > 1
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if dist_on:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=dev)

    M, K, N = w["M"], w["K"], w["N"]
    dt = torch.bfloat16
    g = torch.Generator(device=dev).manual_seed(1234 + rank)
    # synthetic data of the configuration's shape and distributions, created once
    mlp = pkg.FusedGatedMLP(K, N, bias=w["bias"], dropout_p=w["p"], parallel_mode="token" if dist_on else "none",
                            philox_seed=0x5EED)
    mlp = mlp.to(dev).to(dt)
    wgen = torch.Generator(device=dev).manual_seed(7)   # same weights on every rank
    with torch.no_grad():
        for p_ in mlp.parameters():
            p_.copy_((torch.randn(p_.shape, device=dev, generator=wgen) * 0.02).to(dt))
    mlp.token_row0 = rank * M
    train = w["mode"] != "fwd"
    mlp.train(train)
    x = torch.randn((M, K), device=dev, dtype=dt, generator=g)
    dy = (torch.randn((M, K), device=dev, dtype=dt, generator=g) * 1e-2) if train else None
    wg, wu, wd = mlp.gate_proj.weight, mlp.up_proj.weight, mlp.down_proj.weight
    bgt, but, bdt = mlp.gate_proj.bias, mlp.up_proj.bias, mlp.down_proj.bias

    k1_events = []

    def step_device(record: bool):
        """The hot path on resident inputs, kernel by kernel (what FusedGatedMLP.forward/backward enqueue)."""
        if not train:
            if record:
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
            h = K_.hidden_fwd(x, wg, bgt, wu, but)
            if record:
                e1.record()
                k1_events.append((e0, e1))
            return K_.down_fwd(h, wd, bdt)
        xx = x.detach().requires_grad_(True)
        y = mlp(xx)
        y.backward(dy)
        return xx.grad

    launches_per_step = 2 if not train else (2 + 4 + (3 if w["bias"] else 0) * 2)

    def barrier():
        torch.cuda.synchronize()
        if dist_on:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        step_device(False)
    barrier()
    with ClockSampler(local) as clocks:
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        for _ in range(args.steps):
            step_device(True)
        t1.record()
        barrier()
    elapsed_ms = t0.elapsed_time(t1)
    k1_ms = statistics.mean(a.elapsed_time(b) for a, b in k1_events) if k1_events else None

    # ---- end to end through the module API with pinned host buffers: every step copies
    # its input(s) from pinned host memory and its result back, inside the timed region.
    # The copies of neighbouring steps overlap the compute (HostPipeline: three streams).
    x_host = torch.empty((M, K), dtype=dt).pin_memory()
    x_host.copy_(x.cpu())
    y_host = torch.empty((M, K), dtype=dt).pin_memory()
    if train:
        dy_host = torch.empty((M, K), dtype=dt).pin_memory()
        dy_host.copy_(dy.cpu())

        def api_step(x_dev, dy_dev):
            xx = x_dev.detach().requires_grad_(True)
            mlp(xx).backward(dy_dev)
            return xx.grad

        host_inputs = (x_host, dy_host)
    else:
        def api_step(x_dev):
            with torch.no_grad():
                return mlp(x_dev)

        host_inputs = (x_host,)
    pipe = pkg.host_pipeline.HostPipeline(api_step, dev, depth=3)
    e2e_steps = max(3, min(args.steps, 50))
    for _ in range(3):
        pipe.submit(y_host, *host_inputs)
    pipe.drain()
    barrier()
    s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s0.record(pipe.s_in)          # before the first host->device copy
    for _ in range(e2e_steps):
        pipe.submit(y_host, *host_inputs)
    s1.record(pipe.s_out)         # after the last device->host copy
    pipe.drain()
    barrier()
    e2e_ms = s0.elapsed_time(s1)
    status = pkg._lib.status_read(dev)

    if dist_on:
        t = torch.tensor([elapsed_ms, e2e_ms, float(status)], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        elapsed_ms, e2e_ms, status = t[0].item(), t[1].item(), int(t[2].item())
    assert status == 0, f"a kernel recorded a device-side timeout (code {status})"

    if rank == 0:
        fl = flops_per_step(w)
        ms_step = elapsed_ms / args.steps
        value = world * fl / (ms_step * 1e-3) / 1e12
        e2e_value = world * fl / (e2e_ms / e2e_steps * 1e-3) / 1e12
        peak, peak_src = measured_peaks()
        line = {
            "metric": f"gated_mlp_{w['mode'].replace('+', '_')}_tflops", "value": value, "unit": "TFLOP/s",
            "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_step,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": name, "M_per_gpu": M, "K": K, "N": N, "bias": w["bias"], "dropout_p": w["p"],
                       "pass": w["mode"], "parallelism": f"token-sharded x{world}, replicated weights, no collective",
                       "l2": "working set (x + weights + H > 650 MB) exceeds the 126 MB L2; no flush needed"},
            "frac_of_nominal_bf16_peak": value / world / NOMINAL_BF16_TFLOPS,
            "frac_of_measured_bf16_peak": value / world / peak,
            "e2e": {"value": e2e_value, "unit": "TFLOP/s", "h2d_bytes_per_step": x_host.numel() * 2 * (2 if train else 1),
                    "d2h_bytes_per_step": y_host.numel() * 2, "steps": e2e_steps,
                    "ms_per_step": e2e_ms / e2e_steps},
            "gpu_launches": launches_per_step * args.steps,
            "clocks": clocks.summary(),
        }
        if k1_ms is not None:
            k1_flops = 4.0 * M * K * N
            ach = k1_flops / (k1_ms * 1e-3) / 1e12
            line["roofline"] = {
                "kernel": "gemm_tcgen05_pair_kernel<256, K-major, K-major, EPI_SWIGLU> (gate/up GEMM + SiLU*up epilogue)", "bound": "tensor",
                "achieved": ach, "peak": peak, "unit": "TFLOP/s", "frac": ach / peak, "peak_source": peak_src,
                "frac_of_nominal": ach / NOMINAL_BF16_TFLOPS,
                "traffic": K1_DRAM_TRAFFIC_BYTES if name == "llama3-8b-mlp-fwd-bf16" else None,
                "ms_per_launch": k1_ms, "algorithmic_flops_per_launch": k1_flops,
            }
        else:
            line["roofline"] = None
        if world == 1 and not args.no_cpu_baseline:
            base, _, _ = cpu_baseline(w)
            line["cpu_baseline"] = base
        print(json.dumps(line), flush=True)
    if dist_on:
        dist.barrier()
        dist.destroy_process_group()


def run_sweep(args):
    """The reference's own benchmark (src/triton_gated_mlp/benchmark.py:26-123): M = N = K = 2**5 .. 2**12, fp16,
    bias=False, dropout 0, one step = forward + out.sum().backward(), TFLOP/s = 18*M*N*K / t (:86) and peak
    memory (:96-116), for torch-eager (cuBLAS) and for this engine. One JSON line per size."""
    import __graft_entry__ as entry

    pkg = entry.load_package()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)

    def eager_module(K, N):
        class Eager(torch.nn.Module):   # the reference's EagerGatedMLP, restated with torch modules
            def __init__(self):
                super().__init__()
                self.gate_proj = torch.nn.Linear(K, N, bias=False)
                self.up_proj = torch.nn.Linear(K, N, bias=False)
                self.down_proj = torch.nn.Linear(N, K, bias=False)

            def forward(self, x):
                return self.down_proj(torch.nn.functional.silu(self.gate_proj(x)) * self.up_proj(x))
        return Eager()

    def measure(mod, x):
        def step():
            mod.zero_grad(set_to_none=True)
            x.grad = None
            mod(x).sum().backward()
        for _ in range(5):
            step()
        torch.cuda.synchronize()
        torch.cuda.reset_peak_memory_stats(dev)
        times = []
        for _ in range(20):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            step()
            e1.record()
            torch.cuda.synchronize()
            times.append(e0.elapsed_time(e1))
        times.sort()
        return times[len(times) // 2], times[len(times) // 5], times[(4 * len(times)) // 5], \
            torch.cuda.max_memory_allocated(dev) / 2 ** 20

    for e in range(5, 13):
        n = 2 ** e
        x = torch.randn((n, n), device=dev, dtype=torch.float16, requires_grad=True)
        row = {"M": n, "N": n, "K": n, "dtype": "fp16"}
        for name, mod in (("torch_eager", eager_module(n, n)), ("b200", pkg.FusedGatedMLP(n, n, bias=False))):
            mod = mod.to(dev).to(torch.float16)
            ms, lo, hi, mem = measure(mod, x)
            row[name] = {"ms": ms, "ms_p20": lo, "ms_p80": hi, "tflops": 18.0 * n ** 3 / (ms * 1e-3) / 1e12,
                         "peak_mem_mib": mem}
        print(json.dumps(row), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true", help="skip the CPU oracle timing (profiling runs)")
    ap.add_argument("--sweep", action="store_true",
                    help="run the reference benchmark's M=N=K sweep (fp16, fwd+bwd) instead of the headline workload")
    ap.add_argument("--workload", default="llama3-8b-mlp-fwd-bf16", choices=sorted(WORKLOADS))
    args = ap.parse_args()
    w = WORKLOADS[args.workload]
    if args.sweep:
        return run_sweep(args)
    if args.impl == "reference":
        run_reference(args, w, args.workload)
    elif w["mode"] == "decode":
        run_decode(args, w, args.workload)
    else:
        run_gpu(args, w, args.workload)


if __name__ == "__main__":
    main()
