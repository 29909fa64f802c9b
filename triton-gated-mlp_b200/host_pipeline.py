"""Streaming host batches through a FusedGatedMLP with copies and compute overlapped.

The reference has no counterpart: its benchmark creates inputs on the device
(src/triton_gated_mlp/benchmark.py:79). A caller whose activations live in host
memory pays two PCIe transfers per batch, each about as long as the forward pass of
the Llama-8B MLP shape itself; run back to back they triple the step time. This helper
keeps `depth` batches in flight on three CUDA streams (host->device, compute,
device->host), so a stream of batches runs at the pace of the slowest of the three.
"""
from __future__ import annotations

import os
from typing import Callable, List, Optional

import torch
from torch import Tensor


def bind_host_thread_near(device_index: int) -> Optional[List[int]]:
    """Restrict the calling process to the CPU cores the driver reports as closest to GPU
    `device_index` (NVML's CPU affinity for the device: the cores of the NUMA node its PCIe
    root hangs off), so that pinned buffers allocated afterwards land in that node's memory
    and the copy threads run beside it. With several ranks on one host this keeps each
    rank's host traffic on its own socket. Only the process's own affinity is changed; no
    setting of the GPU. Returns the cores chosen, or None when NVML or the affinity call is
    unavailable or reports nothing useful (the process then stays as it was)."""
    try:
        import pynvml

        pynvml.nvmlInit()
        h = pynvml.nvmlDeviceGetHandleByIndex(int(device_index))
        ncpu = os.cpu_count() or 1
        words = pynvml.nvmlDeviceGetCpuAffinity(h, (ncpu + 63) // 64)
        cores = [64 * i + b for i, wd in enumerate(words) for b in range(64) if (int(wd) >> b) & 1]
        allowed = os.sched_getaffinity(0)
        cores = sorted(c for c in cores if c in allowed)
        if not cores or len(cores) == len(allowed):
            return None
        os.sched_setaffinity(0, cores)
        return cores
    except Exception:
        return None


class HostPipeline:
    """step(x_dev, *extra_dev) -> result tensor, applied to pinned host batches.

    submit() enqueues one batch and returns immediately; the result lands in the pinned
    host tensor passed as `out` once drain() (or a later submit that reuses the slot) has
    synchronised with it.
    """

    def __init__(self, step: Callable[..., Tensor], device: torch.device, depth: int = 2):
        self.step, self.device, self.depth = step, torch.device(device), max(1, int(depth))
        self.s_in = torch.cuda.Stream(self.device)
        self.s_run = torch.cuda.Stream(self.device)
        self.s_out = torch.cuda.Stream(self.device)
        self._slots: List[Optional[dict]] = [None] * self.depth
        self._n = 0

    def _slot(self, host_inputs) -> dict:
        i = self._n % self.depth
        slot = self._slots[i]
        if slot is None or [t.shape for t in slot["dev_in"]] != [t.shape for t in host_inputs]:
            # The device inputs belong to the copy stream: allocate them there, and when a
            # slot is replaced (batch shape changed) let that stream wait for the run that
            # may still read the old buffers before their memory can be handed out again.
            with torch.cuda.stream(self.s_in):
                if slot is not None and slot["used"]:
                    self.s_in.wait_event(slot["run_done"])
                    for t in slot["dev_in"]:
                        t.record_stream(self.s_run)
                dev_in = [torch.empty(t.shape, dtype=t.dtype, device=self.device) for t in host_inputs]
            for t in dev_in:
                t.record_stream(self.s_run)
            slot = {
                "dev_in": dev_in,
                "in_done": torch.cuda.Event(), "run_done": torch.cuda.Event(), "out_done": torch.cuda.Event(),
                "used": False,
            }
            self._slots[i] = slot
        return slot

    def submit(self, out: Tensor, *host_inputs: Tensor) -> None:
        for t in (out, *host_inputs):
            if not t.is_pinned():
                raise ValueError("HostPipeline needs pinned host tensors (tensor.pin_memory())")
        slot = self._slot(host_inputs)
        with torch.cuda.stream(self.s_in):
            if slot["used"]:
                self.s_in.wait_event(slot["run_done"])      # the device inputs of this slot are free again
            for d, h in zip(slot["dev_in"], host_inputs):
                d.copy_(h, non_blocking=True)
            slot["in_done"].record(self.s_in)
        with torch.cuda.stream(self.s_run):
            self.s_run.wait_event(slot["in_done"])
            result = self.step(*slot["dev_in"])
            slot["run_done"].record(self.s_run)
        with torch.cuda.stream(self.s_out):
            self.s_out.wait_event(slot["run_done"])
            result.record_stream(self.s_out)
            out.copy_(result, non_blocking=True)
            slot["out_done"].record(self.s_out)
        slot["used"] = True
        self._n += 1

    def drain(self) -> None:
        self.s_out.synchronize()
        self.s_run.synchronize()
        self.s_in.synchronize()
