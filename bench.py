"""Benchmark of the gated-MLP hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--workload NAME]

One step = one pass of the hot path over one batch of synthetic input. The default
workload is the Llama-3-8B MLP forward in bf16 (M=8192 tokens, hidden 4096,
intermediate 14336), the configuration the headline metric is quoted on. With
N > 1 (launched by torch.distributed.run, one rank per GPU) every rank runs the
same per-GPU batch on replicated weights (token sharding, no data-path collective,
weak scaling), and the default workload then also runs the tensor-parallel mode over
the N ranks (parity against the CPU oracle, decode and prefill step times, the
all-reduce alone) and reports it under "tp".

Prints ONE JSON line (rank 0):
  value       device-timed throughput of exactly K steps, inputs resident in HBM
  e2e         the same metric through the public module API with pinned-host input and
              output buffers and both copies inside the timed region
  roofline    the dominant kernel against the measured peak
  sustained   the same step repeated for about two seconds, with the clocks sampled
              meanwhile and time x clock per step (kernels compared per clock)
  gpu_eager   the torch-eager (cuBLAS) module on the same box in the same process, timed the
              same two ways: a comparator, never the value
  check       sampled rows of the last timed output against the CPU oracle
  cpu_baseline  the reference's CPU path on a bounded sample (N = 1 only)
`--impl reference` times the reference's torch-eager CPU path on the host cores on a
bounded sample of the same workload.
"""
from __future__ import annotations

import argparse
import datetime
import json
import math
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
    # name: M, K, N, bias, dropout p, mode, dtype
    "llama3-8b-mlp-fwd-bf16": dict(M=8192, K=4096, N=14336, bias=False, p=0.0, mode="fwd"),
    "llama3-8b-mlp-fwd-bwd-bf16": dict(M=8192, K=4096, N=14336, bias=False, p=0.0, mode="fwd+bwd"),
    "train-fwd-bwd-bf16": dict(M=16384, K=2048, N=8192, bias=True, p=0.1, mode="fwd+bwd"),
    "prefill-fwd-bf16": dict(M=65536, K=8192, N=28672, bias=False, p=0.0, mode="fwd"),
    "prefill-fwd-bwd-bf16": dict(M=65536, K=8192, N=28672, bias=False, p=0.0, mode="fwd+bwd"),
    # the reference README's shape: launch-bound, reported in microseconds per step as well
    "readme-fwd-bwd-fp16": dict(M=128, K=512, N=256, bias=False, p=0.0, mode="fwd+bwd", dtype="fp16"),
    # skinny-M inference through the weight-streaming kernels: HBM-bound, metric in GB/s
    "decode-m1-bf16": dict(M=1, K=8192, N=28672, bias=False, p=0.0, mode="decode"),
    "decode-m8-bf16": dict(M=8, K=8192, N=28672, bias=False, p=0.0, mode="decode"),
    "decode-m32-bf16": dict(M=32, K=8192, N=28672, bias=False, p=0.0, mode="decode"),
    "decode-m64-bf16": dict(M=64, K=8192, N=28672, bias=False, p=0.0, mode="decode"),
    # the same with e4m3 weights (one scale per weight row) and per-token e4m3 activations
    # the same through the one-launch kernel (both weight streams in one persistent kernel)
    "decode-m1-bf16-one-launch": dict(M=1, K=8192, N=28672, bias=False, p=0.0, mode="decode", one_launch=True),
    "decode-m8-bf16-one-launch": dict(M=8, K=8192, N=28672, bias=False, p=0.0, mode="decode", one_launch=True),
    "decode-m32-bf16-one-launch": dict(M=32, K=8192, N=28672, bias=False, p=0.0, mode="decode", one_launch=True),
    "decode-m64-bf16-one-launch": dict(M=64, K=8192, N=28672, bias=False, p=0.0, mode="decode", one_launch=True),
    "decode-m1-fp8": dict(M=1, K=8192, N=28672, bias=False, p=0.0, mode="decode", fp8=True),
    "decode-m8-fp8": dict(M=8, K=8192, N=28672, bias=False, p=0.0, mode="decode", fp8=True),
    "decode-m64-fp8": dict(M=64, K=8192, N=28672, bias=False, p=0.0, mode="decode", fp8=True),
}
DEFAULT_WORKLOAD = "llama3-8b-mlp-fwd-bf16"
NOMINAL_HBM_GBS = 8000.0
FALLBACK_HBM_GBS = 6650.0
NOMINAL_BF16_TFLOPS = 2250.0
FALLBACK_BF16_TFLOPS = 1590.0
FALLBACK_BF16_TFLOPS_SUSTAINED = 1400.0
SUSTAINED_SECONDS = 2.0
# DRAM bytes per launch of each workload's dominant kernel, from ncu captures; written next to
# the capture summaries.
TRAFFIC_FILE = ROOT / "profiles" / "dram_traffic.json"


def wl_dtype(w) -> torch.dtype:
    return torch.float16 if w.get("dtype") == "fp16" else torch.bfloat16


def flops_per_step(w) -> float:
    mkn = w["M"] * w["K"] * w["N"]
    return (6.0 if w["mode"] in ("fwd", "decode") else 18.0) * mkn


def decode_bytes_per_step(w) -> float:
    """Algorithmic bytes of one decode forward: the three weight matrices once (2 bytes per element, or 1 plus
    a 4-byte scale per weight row with e4m3 weights), x in, y out."""
    if w.get("fp8"):
        return 3.0 * w["K"] * w["N"] + 4.0 * (2 * w["N"] + w["K"]) + 2.0 * 2.0 * w["M"] * w["K"]
    return 2.0 * (3.0 * w["K"] * w["N"] + 2.0 * w["M"] * w["K"])


def _peaks_file():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return json.loads(p.read_text())
        except Exception:
            pass
    return None


def measured_hbm_peak():
    d = _peaks_file()
    if d and "hbm_gbs" in d:
        return float(d["hbm_gbs"]), "measured copy bandwidth (MEASURED_PEAKS.json hbm_gbs)"
    return FALLBACK_HBM_GBS, "fallback (MEASURED_PEAKS.json absent)"


def measured_peaks():
    d = _peaks_file()
    if d and "bf16_tflops" in d:
        return float(d["bf16_tflops"]), "measured burst (MEASURED_PEAKS.json bf16_tflops)"
    return FALLBACK_BF16_TFLOPS, "fallback (MEASURED_PEAKS.json absent)"


def measured_sustained_peak():
    d = _peaks_file()
    if d and "bf16_tflops_sustained" in d:
        return float(d["bf16_tflops_sustained"]), "measured sustained (MEASURED_PEAKS.json bf16_tflops_sustained)"
    return FALLBACK_BF16_TFLOPS_SUSTAINED, "fallback (MEASURED_PEAKS.json absent)"


def dram_traffic(name: str):
    """(bytes per launch, note) for the workload's dominant kernel from the tracked capture record, else (None, None)."""
    try:
        rec = json.loads(TRAFFIC_FILE.read_text()).get(name)
        if rec:
            return float(rec["dram_bytes_per_launch"]), rec.get("note")
    except Exception:
        pass
    return None, None


# ------------------------------------------------------------------ clocks --
class ClockSampler:
    """Samples SM clock and throttle reasons through NVML while a timed region runs."""

    def __init__(self, index: int, period_s: float = 0.005):
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
            "sm_mhz_min": min(self.samples) if self.samples else None,
            "sm_max_mhz": self.max_mhz,
            "reasons": sorted(self.reasons),
            "samples": len(self.samples),
        }


# ------------------------------------------------------------ CPU baseline --
def _reference_module():
    """The reference's own EagerGatedMLP, if the build step extracted it from the reference's sources
    (oracle/make_ref.py; the extract is not tracked and exists only where the reference was present at
    build time); None otherwise."""
    try:
        from oracle._ref import eager_reference

        return eager_reference.EagerGatedMLP
    except Exception:
        return None


def cpu_baseline(w, budget_s: float = 12.0, steps: int = 0, warmup: int = 1):
    """Times the reference's torch-eager CPU path (fp32, all host threads) on a row sample of the workload:
    the reference's own EagerGatedMLP class when its extract is present, else the oracle's restatement.
    steps = 0: as many repetitions as fit the budget (3 to 20); steps > 0: exactly that many after `warmup`
    untimed ones, cut short only if the budget runs out."""
    from oracle import gated_mlp_oracle as orc

    torch.set_num_threads(os.cpu_count() or 1)
    ms = min(w["M"], 1024)
    case = orc.make_case(ms, w["K"], w["N"], w["bias"], wl_dtype(w), seed=0, w_std=0.02, dy_std=1e-2)
    x, wg, bg, wu, bu, wd, bd, dy = case.f32()
    fl = flops_per_step(w) * ms / w["M"]
    ref_cls = _reference_module()
    kind = "reference" if ref_cls is not None else "port"
    train = w["mode"] not in ("fwd", "decode")
    if ref_cls is not None:
        mod = ref_cls(w["K"], w["N"], bias=w["bias"])
        mod.load_state_dict(case.state_dict())
        mod.train(False)

        def run():
            if train:
                xx = x.clone().requires_grad_(True)
                mod.zero_grad(set_to_none=True)
                mod(xx).backward(dy)
            else:
                with torch.no_grad():
                    mod(x)
    else:
        def run():
            orc.forward(x, wg, bg, wu, bu, wd, bd)
            if train:
                orc.backward(x, wg, bg, wu, bu, wd, bd, dy)

    for _ in range(max(1, warmup)):
        run()
    times = []
    t_end = time.perf_counter() + budget_s
    want = steps if steps > 0 else 20
    while len(times) < min(3, want) or (time.perf_counter() < t_end and len(times) < want):
        t0 = time.perf_counter()
        run()
        times.append(time.perf_counter() - t0)
    t = statistics.median(times)
    what = "the reference's EagerGatedMLP" if kind == "reference" else "CPU restatement of the reference's eager path"
    if w["mode"] == "decode":
        # the whole batch fits the sample; fp32 weights, so the CPU streams twice the bf16 bytes the metric counts
        return {
            "value": decode_bytes_per_step(w) / t / 1e9, "unit": "GB/s", "cores": torch.get_num_threads(),
            "kind": kind, "runs": len(times),
            "sample": f"{what}: all {ms} token rows, full K and N, fp32 torch CPU, median of {len(times)} runs "
                      f"({t * 1e3:.0f} ms each); bytes counted as for the bf16 path",
        }, t, ms, sum(times)
    return {
        "value": fl / t / 1e12, "unit": "TFLOP/s", "cores": torch.get_num_threads(), "kind": kind, "runs": len(times),
        "sample": f"{what}: {ms} of {w['M']} token rows, full K and N, fp32 torch CPU, median of {len(times)} runs "
                  f"({t * 1e3:.0f} ms each)",
    }, t, ms, sum(times)


def workload_config(name, w, world, decode=False):
    """The `config` object both arms print (same keys, so the two lines can be compared)."""
    return {"workload": name, "M_per_gpu": w["M"], "K": w["K"], "N": w["N"], "bias": w["bias"],
            "dropout_p": w["p"], "pass": "decode forward" if decode else w["mode"],
            "parallelism": (f"independent replicas x{world}, no collective" if decode
                            else f"token-sharded x{world}, replicated weights, no collective"),
            "l2": ("two weight sets alternate between steps; one set (1.4 GB) exceeds the 126 MB L2" if decode
                   else "working set (x + weights + H) exceeds the 126 MB L2; no flush needed"
                   if w["M"] * w["N"] * 2 > 126e6 else "working set fits L2: launch-bound shape, reported as is")}


def run_reference(args, w, name):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    base, t, ms, busy_s = cpu_baseline(w, budget_s=150.0, steps=args.steps, warmup=args.warmup)
    decode = w["mode"] == "decode"
    world = int(os.environ.get("WORLD_SIZE", "1"))
    line = {
        "impl": "reference",
        "metric": "gated_mlp_decode_hbm_gbs" if decode else f"gated_mlp_{w['mode'].replace('+', '_')}_tflops",
        "value": base["value"], "unit": base["unit"], "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "steps_timed": base.pop("runs"),
        # one "step" of this arm is the bounded row sample, not the full batch
        "ms_per_step": t * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": workload_config(name, w, world, decode),
        "sample_rows_per_step": ms, "timed_seconds": busy_s,
        "cpu_baseline": base,
        "e2e": {"value": base["value"], "unit": base["unit"], "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------ value check --
def sampled_rows_check(x, y, mlp, rows=16, seed=5):
    """Rows of the engine's output y = mlp(x) against the fp32 CPU oracle fed the same 16-bit inputs.
    Returns the literal and the contract's error figures; token rows are independent, so a row sample
    checks the whole pipeline at any M."""
    from oracle import gated_mlp_oracle as orc

    g = torch.Generator().manual_seed(seed)
    idx = torch.randperm(x.shape[0], generator=g)[:min(rows, x.shape[0])].sort().values
    f = lambda t: None if t is None else t.detach().float().cpu()
    want = orc.forward(f(x[idx.to(x.device)]), f(mlp.gate_proj.weight), f(mlp.gate_proj.bias), f(mlp.up_proj.weight),
                       f(mlp.up_proj.bias), f(mlp.down_proj.weight), f(mlp.down_proj.bias))
    got = y[idx.to(y.device)].float().cpu()
    return parity_record(got, want, y.dtype, rows=int(idx.numel()))


def parity_record(got, want, out_dtype, low_precision_sum_over=1, **extra):
    """One comparison against the oracle as a JSON record. low_precision_sum_over = g: the value is a sum of g
    per-rank partial results that NCCL added in the 16-bit format, rounding at every hop of its ring (2g - 1
    roundings instead of the one the contract allows for): the max-abs bound is widened by sqrt(g / 2) and the record
    says so. Sums taken in fp32 (the peer-memory sum) and everything that crosses no rank keep the plain bound."""
    from oracle import gated_mlp_oracle as orc

    scaled, mean_rel = orc.parity_errors(got, want, orc.HALF_ULP_REL.get(out_dtype, 2.0 ** -8))
    tol = orc.MAX_ABS_TOL * max(1.0, (low_precision_sum_over / 2.0) ** 0.5)
    rec = {"max_abs": (got.double() - want.double()).abs().max().item(), "max_abs_scaled": scaled,
           "mean_rel": mean_rel, "rms_want": want.double().pow(2).mean().sqrt().item(), "max_abs_tol": tol,
           "ok": bool(scaled <= tol and mean_rel <= orc.MEAN_REL_TOL)}
    if low_precision_sum_over > 2:
        rec["tol_note"] = f"sum of {low_precision_sum_over} partials in the 16-bit format: bound x sqrt(ranks / 2)"
    rec.update(extra)
    return rec


# ------------------------------------------------------------ comparators --
def eager_module(K, N, bias, dt, dev, src=None):
    """torch-eager (cuBLAS) gated MLP with the reference's EagerGatedMLP semantics: the on-GPU comparator."""
    class Eager(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.gate_proj = torch.nn.Linear(K, N, bias=bias)
            self.up_proj = torch.nn.Linear(K, N, bias=bias)
            self.down_proj = torch.nn.Linear(N, K, bias=bias)

        def forward(self, x):
            return self.down_proj(torch.nn.functional.silu(self.gate_proj(x)) * self.up_proj(x))

    m = Eager().to(dev).to(dt)
    if src is not None:
        m.load_state_dict({k: v for k, v in src.state_dict().items()})
    return m


def timed_steps(step, n, barrier, clocks_index=None):
    """Milliseconds for n back-to-back calls of step() (CUDA events on the current stream), and the clock record."""
    barrier()
    sampler = ClockSampler(clocks_index) if clocks_index is not None else None
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if sampler is not None:
        sampler.__enter__()
    t0.record()
    for _ in range(n):
        step()
    t1.record()
    barrier()
    if sampler is not None:
        sampler.__exit__()
    return t0.elapsed_time(t1), (sampler.summary() if sampler is not None else None)


def sustained_run(step, ms_step_estimate, fl, barrier, local, peak_sustained):
    """The step repeated back to back for about SUSTAINED_SECONDS: throughput under the power cap, the clocks
    seen meanwhile and time x clock per step (what the step costs in SM cycles, whatever the clock did)."""
    n = max(10, int(math.ceil(SUSTAINED_SECONDS * 1e3 / max(ms_step_estimate, 1e-3))))
    n = min(n, 20000)
    ms, clk = timed_steps(step, n, barrier, clocks_index=local)
    ms_step = ms / n
    rec = {"seconds": ms * 1e-3, "steps": n, "ms_per_step": ms_step, "value": fl / (ms_step * 1e-3) / 1e12,
           "unit": "TFLOP/s", "clocks": clk}
    if clk and clk.get("sm_mhz"):
        rec["mcycles_per_step"] = ms_step * 1e-3 * clk["sm_mhz"]   # ms x MHz = thousands of cycles; /1e3 -> Mcycles
        rec["flop_per_cycle_per_gpu"] = fl / (ms_step * 1e-3 * clk["sm_mhz"] * 1e6)
    rec["frac_of_sustained_peak"] = rec["value"] / peak_sustained
    return rec


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
        if w.get("fp8"):
            mlp.quantize_decode_weights()
        mlp.decode_one_launch = bool(w.get("one_launch"))
        sets.append(mlp)
    x = torch.randn((M, K), device=dev, dtype=dt, generator=torch.Generator(device=dev).manual_seed(1234 + rank))

    def barrier():
        torch.cuda.synchronize()
        if dist_on:
            dist.barrier()
        torch.cuda.synchronize()

    # A serving loop replays its decode steps from a CUDA graph; so does the timed region here (two steps per
    # graph, one per weight set), because at 2 launches per ~0.2 ms an eager Python loop is not reliably
    # faster than the GPU and the figure would measure the host. Exactly `steps` steps are replayed.
    with torch.no_grad():
        for i in range(max(args.warmup, 3) * 2):
            sets[i & 1](x)
        assert sets[0]._decode_scratch is not None, "the decode path was not taken"
        torch.cuda.synchronize()
        side = torch.cuda.Stream(dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        y_pair = [None, None]
        with torch.cuda.stream(side):
            pair_graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(pair_graph, stream=side):
                y_pair[0] = sets[0](x)
                y_pair[1] = sets[1](x)
        torch.cuda.current_stream(dev).wait_stream(side)
        for _ in range(3):
            pair_graph.replay()
        barrier()
        with ClockSampler(local, period_s=0.02) as clocks:
            t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            t0.record()
            for _ in range(args.steps // 2):
                pair_graph.replay()
            if args.steps % 2:
                sets[0](x)
            t1.record()
            barrier()
        elapsed_ms = t0.elapsed_time(t1)
        check = sampled_rows_check(x, y_pair[1], sets[1], rows=M)
        if w.get("fp8"):
            # against the UNQUANTISED module's oracle this measures the quantisation itself (weights and
            # activations to e4m3): a few percent, held to 8e-2 mean relative; the kernels' own parity under
            # the quantisation contract is the test suite's business
            check["ok"] = bool(check["mean_rel"] <= 8e-2)
            check["note"] = "vs the 16-bit oracle: measures e4m3 quantisation of weights and activations"

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
        t = torch.tensor([elapsed_ms, e2e_ms, float(status), 0.0 if check["ok"] else 1.0], device=dev,
                         dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        elapsed_ms, e2e_ms, status = t[0].item(), t[1].item(), int(t[2].item())
        check["ok_all_ranks"] = t[3].item() == 0.0
    assert status == 0, f"a kernel recorded a device-side timeout (code {status})"

    if rank == 0:
        nbytes = decode_bytes_per_step(w)
        ms_step = elapsed_ms / args.steps
        value = world * nbytes / (ms_step * 1e-3) / 1e9
        peak, peak_src = measured_hbm_peak()
        traffic, traffic_note = dram_traffic(name)
        line = {
            "metric": "gated_mlp_decode_hbm_gbs", "value": value, "unit": "GB/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "e4m3 x e4m3 -> f32" if w.get("fp8") else "bf16",
            "data": "synthetic",
            "config": workload_config(name, w, world, decode=True),
            "frac_of_nominal_hbm_peak": value / world / NOMINAL_HBM_GBS,
            "frac_of_measured_hbm_peak": value / world / peak,
            "e2e": {"value": world * nbytes / (e2e_ms / e2e_steps * 1e-3) / 1e9, "unit": "GB/s",
                    "h2d_bytes_per_step": x_host.numel() * 2, "d2h_bytes_per_step": y_host.numel() * 2,
                    "steps": e2e_steps, "ms_per_step": e2e_ms / e2e_steps},
            "gpu_launches": (4 if w.get("fp8") else 1 if w.get("one_launch") else 2) * args.steps,
            "launch_mode": "CUDA graph of two steps (one per weight set) replayed steps/2 times",
            "clocks": clocks.summary(),
            "check": check,
            "roofline": {
                "kernel": ("decode_fused_kernel<MPAD>: gate+up and down streams from one persistent kernel"
                           if w.get("one_launch") else
                           "decode_stream_kernel<MPAD, gate+up> then <MPAD, down>, chained by programmatic dependent "
                           "launch (timed together: timing them apart would break the chain)"),
                "bound": "hbm", "achieved": value / world, "peak": peak, "unit": "GB/s", "frac": value / world / peak,
                "peak_source": peak_src, "frac_of_nominal": value / world / NOMINAL_HBM_GBS,
                "traffic": traffic, "traffic_note": traffic_note,
                "ms_per_launch": ms_step, "algorithmic_bytes_per_launch": nbytes,
            },
        }
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline(w)[0]
        print(json.dumps(line), flush=True)
    if dist_on:
        dist.barrier()
        dist.destroy_process_group()
    assert check["ok"], f"decode output outside the parity tolerance: {check}"


# ------------------------------------------------------- tensor parallel ----
def graph_timed(fn, dev, dist, inner=20, reps=10):
    """Milliseconds per call of fn on the device: `inner` calls captured in one CUDA graph (so the host's launch
    cost is out of the picture), `reps` replays timed with events, max over ranks."""
    side = torch.cuda.Stream(dev)
    side.wait_stream(torch.cuda.current_stream(dev))
    with torch.cuda.stream(side):
        for _ in range(3):
            fn()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            for _ in range(inner):
                fn()
    torch.cuda.current_stream(dev).wait_stream(side)
    graph.replay()
    torch.cuda.synchronize()
    dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        graph.replay()
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / (reps * inner)], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.item()


def event_timed(fn, n, dev, dist):
    """Milliseconds per call, max over ranks (device events, barrier on both sides, 3 warm-up calls)."""
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(n):
        fn()
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / n], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.item()


def tp_section(pkg, dev, rank, world, dist):
    """Tensor-parallel mode over all ranks at the decode and prefill configurations' K and N (8192, 28672 split over
    the ranks): parity against the CPU oracle (rank 0 computes it), decode step times with the NCCL sum and with the
    peer-memory sum, prefill forward and forward+backward times, and the all-reduce alone."""
    from oracle import gated_mlp_oracle as orc

    K, N = 8192, 28672
    dt = torch.bfloat16
    if N % (world * 128) != 0:
        return {"skipped": f"N={N} does not split into {world} shards of a multiple of 128 columns"}
    cols = N // world
    c0 = rank * cols
    out = {"K": K, "N_global": N, "N_per_gpu": cols, "ranks": world}

    def make_weights(std, seed):
        g = torch.Generator(device=dev).manual_seed(seed)   # the same full matrices on every rank
        return [(torch.randn(s, device=dev, generator=g) * std).to(dt) for s in ((N, K), (N, K), (K, N))]

    def shard_module(wg, wu, wd, group=None):
        m = pkg.FusedGatedMLP(K, cols, bias=False, parallel_mode="tp", process_group=group).to(dev).to(dt)
        with torch.no_grad():
            m.gate_proj.weight.copy_(wg[c0:c0 + cols])
            m.up_proj.weight.copy_(wu[c0:c0 + cols])
            m.down_proj.weight.copy_(wd[:, c0:c0 + cols])
        return m

    hbm_peak, _ = measured_hbm_peak()
    # ---------------------------------------------------------- decode: parity and step times
    wg, wu, wd = make_weights(0.02, 41)
    m = shard_module(wg, wu, wd).eval()
    x64 = torch.randn((64, K), device=dev, dtype=dt, generator=torch.Generator(device=dev).manual_seed(42))
    want = None
    if rank == 0:
        torch.set_num_threads(max(1, min(16, os.cpu_count() or 1)))   # torchrun pins OMP_NUM_THREADS to 1
        want = orc.forward(x64.float().cpu(), wg.float().cpu(), None, wu.float().cpu(), None, wd.float().cpu(), None)
    del wg, wu, wd
    decode = []
    comm = None
    try:
        with torch.no_grad():
            for M in (1, 8, 32, 64):
                x = x64[:M].contiguous()
                rec = {"M": M}
                m._peer = None
                y_nccl = m(x).clone()
                rec["step_us_nccl_sum"] = graph_timed(lambda: m(x), dev, dist) * 1e3
                y_buf = torch.empty((M, K), device=dev, dtype=dt)
                rec["sum_alone_us_nccl"] = graph_timed(lambda: dist.all_reduce(y_buf), dev, dist) * 1e3
                if comm is None:
                    comm = m.enable_peer_allreduce(64)
                else:
                    m._peer = comm
                y_peer = m(x).clone()
                rec["step_us_peer_sum"] = graph_timed(lambda: m(x), dev, dist) * 1e3
                rec["sum_alone_us_peer"] = graph_timed(lambda: comm.all_reduce(y_buf, out=y_buf), dev, dist) * 1e3
                nbytes = 2.0 * (3.0 * K * cols + 2.0 * M * K)   # per GPU: its weight shard once, x in, y out
                best = min(rec["step_us_nccl_sum"], rec["step_us_peer_sum"])
                rec["per_gpu_gbs"] = nbytes / (best * 1e-6) / 1e9
                rec["frac_of_measured_hbm_peak"] = rec["per_gpu_gbs"] / hbm_peak
                rec["frac_of_nominal_hbm_peak"] = rec["per_gpu_gbs"] / NOMINAL_HBM_GBS
                if rank == 0:
                    rec["parity_nccl_sum"] = parity_record(y_nccl.float().cpu(), want[:M], dt, low_precision_sum_over=world)
                    rec["parity_peer_sum"] = parity_record(y_peer.float().cpu(), want[:M], dt)
                decode.append(rec)
    finally:
        if comm is not None:
            comm.close()
    out["decode"] = decode
    del m

    # ---------------------------------------------------------- prefill / training: parity and step times
    M = 16384
    wg, wu, wd = make_weights(0.01, 43)
    g = torch.Generator(device=dev).manual_seed(44)   # x and dy are replicated: the same on every rank
    x = torch.randn((M, K), device=dev, dtype=dt, generator=g)
    dy = (torch.randn((M, K), device=dev, generator=g) * 1e-2).to(dt)
    rows = torch.randperm(M, generator=torch.Generator().manual_seed(45))[:32].sort().values
    units = torch.randperm(cols, generator=torch.Generator().manual_seed(46))[:16].sort().values  # of rank 0's shard
    want = {}
    if rank == 0:
        f = lambda t: t.float().cpu()
        wgf, wuf, wdf = f(wg), f(wu), f(wd)
        xr, dyr = f(x[rows.to(dev)]), f(dy[rows.to(dev)])
        want["y"] = orc.forward(xr, wgf, None, wuf, None, wdf, None)
        want["dx"] = orc.backward(xr, wgf, None, wuf, None, wdf, None, dyr)["dx"]
        xf, dyf = f(x), f(dy)
        h_s, g_s, u_s = orc.hidden_forward(xf, wgf[units], None, wuf[units], None)
        _, dwu_s, dwg_s, _, _ = orc.hidden_backward(xf, wgf[units], wuf[units], g_s, u_s, dyf @ wdf[:, units])
        want["dgate_proj.weight"], want["dup_proj.weight"] = dwg_s, dwu_s
        want["ddown_proj.weight"] = dyf.T @ h_s
        del wgf, wuf, wdf, xf, dyf
    opts = None
    try:
        opts = dist.ProcessGroupNCCL.Options()
        opts.config.max_ctas = 16   # the collective's CTAs must fit into the SMs the chunked GEMMs leave free
    except Exception:
        opts = None
    group16 = dist.new_group(list(range(world)), pg_options=opts) if opts is not None else None
    m = shard_module(wg, wu, wd, group=group16)
    del wg, wu, wd
    xg = x.clone().requires_grad_(True)
    y = m(xg)
    y.backward(dy)
    parity = {}
    if rank == 0:
        parity["y_rows"] = parity_record(y[rows.to(dev)].float().cpu(), want["y"], dt, low_precision_sum_over=world,
                                         rows=int(rows.numel()))
        parity["dx_rows"] = parity_record(xg.grad[rows.to(dev)].float().cpu(), want["dx"], dt,
                                          low_precision_sum_over=world, rows=int(rows.numel()))
        u_dev = units.to(dev)
        parity["dW_gate_units"] = parity_record(m.gate_proj.weight.grad[u_dev].float().cpu(),
                                                want["dgate_proj.weight"], dt, units=int(units.numel()))
        parity["dW_up_units"] = parity_record(m.up_proj.weight.grad[u_dev].float().cpu(),
                                              want["dup_proj.weight"], dt, units=int(units.numel()))
        parity["dW_down_units"] = parity_record(m.down_proj.weight.grad[:, u_dev].float().cpu(),
                                                want["ddown_proj.weight"], dt, units=int(units.numel()))
    want_y, want_dx = (want["y"], want["dx"]) if rank == 0 else (None, None)
    del y, xg, want
    m.zero_grad(set_to_none=True)

    def fwd():
        with torch.no_grad():
            m(x)

    xt = x.clone().requires_grad_(True)

    def fwd_bwd():
        m(xt).backward(dy)
        m.zero_grad(set_to_none=True)
        xt.grad = None

    pre = {"M": M, "parity": parity}
    pre["fwd_ms"] = event_timed(fwd, 10, dev, dist)
    pre["fwd_bwd_ms"] = event_timed(fwd_bwd, 5, dev, dist)
    m.tp_chunk_rows = 4096
    pre["fwd_bwd_ms_dx_chunks_of_4096_rows"] = event_timed(fwd_bwd, 5, dev, dist)
    m.tp_chunk_rows = 0
    buf = torch.empty((M, K), device=dev, dtype=dt)
    pre["allreduce_alone_ms"] = event_timed(lambda: dist.all_reduce(buf), 10, dev, dist)
    pre["allreduce_bytes"] = M * K * 2
    pre["allreduce_busbw_gbs"] = (2.0 * (world - 1) / world) * M * K * 2 / (pre["allreduce_alone_ms"] * 1e-3) / 1e9
    pre["fwd_tflops_whole_job"] = 6.0 * M * K * N / (pre["fwd_ms"] * 1e-3) / 1e12
    best_fb = min(pre["fwd_bwd_ms"], pre["fwd_bwd_ms_dx_chunks_of_4096_rows"])
    pre["fwd_bwd_tflops_whole_job"] = 18.0 * M * K * N / (best_fb * 1e-3) / 1e12
    pre["fwd_frac_of_nominal_per_gpu"] = pre["fwd_tflops_whole_job"] / world / NOMINAL_BF16_TFLOPS
    pre["fwd_bwd_frac_of_nominal_per_gpu"] = pre["fwd_bwd_tflops_whole_job"] / world / NOMINAL_BF16_TFLOPS
    # what the forward would take with the all-reduce fully hidden: names the limiter
    pre["fwd_ms_minus_allreduce"] = pre["fwd_ms"] - pre["allreduce_alone_ms"]
    # the same forward with the down projection pushing the other ranks' row blocks into their inboxes from its
    # epilogue (scatter overlapped with the GEMM) and one kernel per rank that sums and hands round: no NCCL call
    del buf
    torch.cuda.empty_cache()
    try:
        m.enable_peer_output_sum(max_tokens=M)
        with torch.no_grad():
            yp = m(x)
        if rank == 0:
            parity["y_rows_pushed_sum"] = parity_record(yp[rows.to(dev)].float().cpu(), want_y, dt,
                                                        rows=int(rows.numel()))
        del yp
        pre["fwd_ms_pushed_sum"] = event_timed(fwd, 10, dev, dist)
        pre["fwd_pushed_sum_tflops_whole_job"] = 6.0 * M * K * N / (pre["fwd_ms_pushed_sum"] * 1e-3) / 1e12
        # forward and backward without an NCCL call: y and dx both scattered from their GEMMs' epilogues, the
        # dx sum kernel enqueued behind the weight-gradient GEMMs
        pre["fwd_bwd_ms_pushed_sums"] = event_timed(fwd_bwd, 5, dev, dist)
        pre["fwd_bwd_pushed_sums_tflops_whole_job"] = 18.0 * M * K * N / (pre["fwd_bwd_ms_pushed_sums"] * 1e-3) / 1e12
        if rank == 0:
            xq = x.clone().requires_grad_(True)
            m(xq).backward(dy)
            parity["dx_rows_pushed_sum"] = parity_record(xq.grad[rows.to(dev)].float().cpu(), want_dx, dt,
                                                         rows=int(rows.numel()))
            m.zero_grad(set_to_none=True)
            del xq
        else:
            xq = x.clone().requires_grad_(True)
            m(xq).backward(dy)
            m.zero_grad(set_to_none=True)
            del xq
        m._peer_sum.close()
        m._peer_sum = None
    except Exception as e:   # the line must still be printed
        pre["pushed_sum_error"] = f"{type(e).__name__}: {e}"
    out["prefill"] = pre
    oks = [r[k]["ok"] for r in decode for k in ("parity_nccl_sum", "parity_peer_sum") if k in r]
    oks += [v["ok"] for v in parity.values()]
    out["parity_ok"] = all(oks) if rank == 0 else None
    return out


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
    pkg.host_pipeline.bind_host_thread_near(local)   # before any pinned allocation
    dist = None
    if dist_on:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=300))

    M, K, N = w["M"], w["K"], w["N"]
    dt = wl_dtype(w)
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

    def step_device(record: bool = False):
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
        # one training step's worth of work: gradients start from None, as after an optimiser's
        # zero_grad(set_to_none=True) (otherwise torch adds every new gradient into the old one,
        # three more passes over the weights that are not part of the hot path)
        mlp.zero_grad(set_to_none=True)
        xx = x.detach().requires_grad_(True)
        y = mlp(xx)
        y.backward(dy)
        return xx.grad

    launches_per_step = 2 if not train else 6   # bias gradients come out of the weight-gradient kernels

    def barrier():
        torch.cuda.synchronize()
        if dist_on:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- headline: W warm-up steps, then exactly K timed steps
    time.sleep(1.0)
    for _ in range(max(args.warmup, 3)):
        step_device()
    barrier()
    with ClockSampler(local) as clocks:
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        for _ in range(args.steps):
            last = step_device(True)
        t1.record()
        barrier()
    elapsed_ms = t0.elapsed_time(t1)
    k1_ms = statistics.mean(a.elapsed_time(b) for a, b in k1_events) if k1_events else None
    # a value check of what the timed loop computed (forward output rows; the backward's parity is the
    # test suite's business)
    with torch.no_grad():
        check = sampled_rows_check(x, last if not train else mlp.eval()(x), mlp) if (w["K"] * w["N"] <= 2 ** 27 or rank == 0) \
            else {"skipped": "weights too large to check on every rank's host; rank 0 checks"}
    mlp.train(train)

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
            mlp.zero_grad(set_to_none=True)
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
    # the copies alone, all ranks at once: the host-side ceiling of the end-to-end figure
    x_dev2 = torch.empty_like(x)
    h2d_ms, _ = timed_steps(lambda: x_dev2.copy_(x_host, non_blocking=True), 10, barrier)
    d2h_ms, _ = timed_steps(lambda: y_host.copy_(x_dev2, non_blocking=True), 10, barrier)
    # both directions at once (what the pipeline asks of the host in steady state), all ranks at once, no kernels
    x_dev3 = torch.empty_like(x)
    side = torch.cuda.Stream(dev)

    def both_ways():
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            y_host.copy_(x_dev3, non_blocking=True)
        for h in host_inputs:
            x_dev2.copy_(h, non_blocking=True)
        torch.cuda.current_stream(dev).wait_stream(side)

    duplex_ms, _ = timed_steps(both_ways, 10, barrier)
    del x_dev3
    status = pkg._lib.status_read(dev)

    # ---- comparator and sustained figures (default-size GEMM workloads; skipped for the largest shape)
    fl = flops_per_step(w)
    peak_sus, peak_sus_src = measured_sustained_peak()
    sustained = eager = None
    if not args.no_extras and M * N <= 16384 * 14336:
        ms_est = elapsed_ms / args.steps
        em = eager_module(K, N, w["bias"], dt, dev, src=mlp)
        em.train(False)

        def eager_step():
            if not train:
                with torch.no_grad():
                    return em(x)
            xx = x.detach().requires_grad_(True)
            em.zero_grad(set_to_none=True)
            em(xx).backward(dy)
            return xx.grad

        engine_step = step_device

        time.sleep(1.0)
        for _ in range(max(args.warmup, 3)):
            eager_step()
        e_ms, e_clk = timed_steps(eager_step, args.steps, barrier, clocks_index=local)
        eager = {"what": "torch-eager module (nn.Linear x3 on cuBLAS + elementwise kernels), same box, same process, "
                         "same weights and inputs: a comparator, not the value",
                 "burst": {"steps": args.steps, "ms_per_step": e_ms / args.steps,
                           "value": fl / (e_ms / args.steps * 1e-3) / 1e12, "unit": "TFLOP/s", "clocks": e_clk}}
        time.sleep(1.0)
        sustained = sustained_run(engine_step, ms_est, fl, barrier, local, peak_sus)
        sustained["peak_source"] = peak_sus_src
        time.sleep(1.0)
        eager["sustained"] = sustained_run(eager_step, e_ms / args.steps, fl, barrier, local, peak_sus)
        sustained["vs_gpu_eager_sustained"] = sustained["value"] / eager["sustained"]["value"]
        del em
        status = status or pkg._lib.status_read(dev)

    if dist_on:
        t = torch.tensor([elapsed_ms, e2e_ms, float(status), h2d_ms, d2h_ms,
                          0.0 if check.get("ok", True) else 1.0, duplex_ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        elapsed_ms, e2e_ms, status, h2d_ms, d2h_ms = t[0].item(), t[1].item(), int(t[2].item()), t[3].item(), t[4].item()
        check["ok_all_ranks"] = t[5].item() == 0.0
        duplex_ms = t[6].item()
    assert status == 0, f"a kernel recorded a device-side timeout (code {status})"

    tp = None
    if dist_on and name == DEFAULT_WORKLOAD and not args.no_tp:
        del x_dev2, pipe
        torch.cuda.empty_cache()
        try:
            tp = tp_section(pkg, dev, rank, world, dist)
        except Exception as e:  # the headline line must still be printed
            tp = {"error": f"{type(e).__name__}: {e}"}
        st = pkg._lib.status_read(dev)
        if st != 0:
            tp["device_status"] = st

    if rank == 0:
        ms_step = elapsed_ms / args.steps
        value = world * fl / (ms_step * 1e-3) / 1e12
        e2e_step = e2e_ms / e2e_steps
        e2e_value = world * fl / (e2e_step * 1e-3) / 1e12
        peak, peak_src = measured_peaks()
        h2d_bytes = x_host.numel() * x_host.element_size() * (2 if train else 1)
        d2h_bytes = y_host.numel() * y_host.element_size()
        line = {
            "metric": f"gated_mlp_{w['mode'].replace('+', '_')}_tflops", "value": value, "unit": "TFLOP/s",
            "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_step,
            "us_per_step": ms_step * 1e3,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "fp16" if dt == torch.float16 else "bf16", "data": "synthetic",
            "config": workload_config(name, w, world),
            "frac_of_nominal_bf16_peak": value / world / NOMINAL_BF16_TFLOPS,
            "frac_of_measured_bf16_peak": value / world / peak,
            "e2e": {"value": e2e_value, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d_bytes,
                    "d2h_bytes_per_step": d2h_bytes, "steps": e2e_steps, "ms_per_step": e2e_step,
                    # per rank, all ranks copying at once
                    "h2d_gbs_in_pipeline": h2d_bytes / (e2e_step * 1e-3) / 1e9,
                    "d2h_gbs_in_pipeline": d2h_bytes / (e2e_step * 1e-3) / 1e9,
                    "h2d_alone_gbs": x_host.numel() * x_host.element_size() / (h2d_ms / 10 * 1e-3) / 1e9,
                    "d2h_alone_gbs": d2h_bytes / (d2h_ms / 10 * 1e-3) / 1e9,
                    # one step's copies in both directions at once, nothing else running: what the host side
                    # (PCIe root, host memory) allows per step when every rank copies, i.e. the floor of e2e
                    "copies_both_ways_ms": duplex_ms / 10,
                    "copies_both_ways_gbs_per_direction": d2h_bytes / (duplex_ms / 10 * 1e-3) / 1e9,
                    "host_copy_floor_ms": duplex_ms / 10,
                    "frac_of_host_copy_floor": (duplex_ms / 10) / e2e_step,
                    "bound": "host copies" if duplex_ms / 10 > ms_step else "kernels"},
            "gpu_launches": launches_per_step * args.steps,
            "clocks": clocks.summary(),
            "check": check,
        }
        if k1_ms is not None:
            k1_flops = 4.0 * M * K * N
            ach = k1_flops / (k1_ms * 1e-3) / 1e12
            traffic, traffic_note = dram_traffic(name)
            line["roofline"] = {
                "kernel": "gemm_tcgen05_pair_kernel<256, K-major, K-major, EPI_SWIGLU> (gate/up GEMM + SiLU*up epilogue)",
                "bound": "tensor",
                "achieved": ach, "peak": peak, "unit": "TFLOP/s", "frac": ach / peak, "peak_source": peak_src,
                "frac_of_nominal": ach / NOMINAL_BF16_TFLOPS,
                "traffic": traffic, "traffic_note": traffic_note,
                "ms_per_launch": k1_ms, "algorithmic_flops_per_launch": k1_flops,
                "algorithmic_dram_bytes_per_launch": 2.0 * (M * K + 2 * N * K + M * N),
            }
        else:
            # fwd+bwd: the step as a whole against the tensor roofline (six GEMM kernels of comparable weight)
            line["roofline"] = {
                "kernel": "whole step: gate/up, down, dH, dX, dW_gate+dW_up, dW_down GEMM kernels", "bound": "tensor",
                "achieved": value / world, "peak": peak, "unit": "TFLOP/s", "frac": value / world / peak,
                "peak_source": peak_src, "frac_of_nominal": value / world / NOMINAL_BF16_TFLOPS, "traffic": None,
                "ms_per_launch": ms_step, "algorithmic_flops_per_launch": fl,
            }
        if sustained is not None:
            line["sustained"] = sustained
            line["gpu_eager"] = eager
        if tp is not None:
            line["tp"] = tp
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline(w)[0]
        print(json.dumps(line), flush=True)
    if dist_on:
        dist.barrier()
        dist.destroy_process_group()
    assert check.get("ok", True), f"output rows outside the parity tolerance: {check}"
    if rank == 0 and tp is not None:
        assert "error" not in tp, tp["error"]
        assert tp.get("parity_ok", True), "tensor-parallel outputs outside the parity tolerance"


def run_sweep(args):
    """The reference's own benchmark (src/triton_gated_mlp/benchmark.py:26-123): M = N = K = 2**5 .. 2**12, fp16,
    bias=False, dropout 0, one step = forward + out.sum().backward(), TFLOP/s = 18*M*N*K / t (:86) and peak
    memory (:96-116), for torch-eager (cuBLAS) and for this engine. One JSON line per size."""
    import __graft_entry__ as entry

    pkg = entry.load_package()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)

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
        for name, mod in (("torch_eager", eager_module(n, n, False, torch.float16, dev)),
                          ("b200", pkg.FusedGatedMLP(n, n, bias=False).to(dev).to(torch.float16))):
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
    ap.add_argument("--no-cpu-baseline", action="store_true", help="skip the CPU timing (profiling runs)")
    ap.add_argument("--no-extras", action="store_true",
                    help="skip the sustained and torch-eager comparator sections (profiling runs)")
    ap.add_argument("--no-tp", action="store_true", help="with N > 1: skip the tensor-parallel section")
    ap.add_argument("--sweep", action="store_true",
                    help="run the reference benchmark's M=N=K sweep (fp16, fwd+bwd) instead of the headline workload")
    ap.add_argument("--workload", default=DEFAULT_WORKLOAD, choices=sorted(WORKLOADS))
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
