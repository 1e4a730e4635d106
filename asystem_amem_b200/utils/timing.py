"""CUDA-event timing with L2 flushes, nvidia-smi clock sampling, measured-peak lookup.

Reference parity: the reference times pause and resume with std::chrono around the calls and
prints milliseconds (amem_nccl_plugin/amem_nccl.cpp:490,563-569,602,668-674); nothing is timed
on the device there.
"""
from __future__ import annotations

import json
import os
import statistics
import subprocess
import threading

_FLUSH = None


def flush_l2() -> None:
    """Writes a buffer larger than the 126 MB L2 so the next kernel starts cold."""
    import torch
    global _FLUSH
    if _FLUSH is None:
        _FLUSH = torch.empty(192 << 20, dtype=torch.uint8, device="cuda")
    _FLUSH.zero_()


def cuda_time_ms(fn, iters: int = 10, warmup: int = 3, flush: bool = True) -> dict:
    """Times fn() with CUDA events on the current stream; returns best / mean / all in ms."""
    import torch
    for _ in range(max(3, warmup)):
        fn()
    torch.cuda.synchronize()
    times = []
    for _ in range(iters):
        if flush:
            flush_l2()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        times.append(s.elapsed_time(e))
    return {"best": min(times), "mean": statistics.mean(times), "all": times}


def max_over_ranks(value: float, group=None) -> float:
    import torch
    import torch.distributed as dist
    if not (dist.is_available() and dist.is_initialized()):
        return value
    t = torch.tensor([value], dtype=torch.float64)
    if dist.get_backend(group) == "nccl":
        t = t.cuda()
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return float(t.item())


def load_measured_peaks(root: str | None = None) -> dict:
    """Measured copy bandwidth / cuBLAS throughput of the B200s at hand (MEASURED_PEAKS.json), or the documented
    fallback (6.65 TB/s, 1.59 PFLOP/s) when the file is absent."""
    root = root or os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    p = os.path.join(root, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        d["source"] = "measured"
        return d
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and clock-event reasons while a timed region runs (read-only queries).

    NVML is initialised in the constructor, i.e. BEFORE the timed region: starting a fresh
    ``nvidia-smi`` process per sample (which initialises the management library every time) was
    measured to stall the memory-management calls of the benchmark itself (one cuMemUnmap of 940 ms
    in a region that otherwise takes 2 ms).  In-process NVML queries take microseconds; the
    ``nvidia-smi`` loop is kept as a fallback when the Python binding is missing."""

    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int = 0, period_s: float | None = 0.05):
        """``period_s=None``: no background thread, the caller takes samples with ``sample_now()``
        at moments of its choosing (management-library queries contend with the driver's
        memory-management calls: polled at 50 Hz from two ranks they stretched a 13 ms
        pause + resume to 87 ms, so a latency benchmark samples between those calls, not across)."""
        self.index, self.samples, self._stop, self.period_s = index, [], threading.Event(), period_s
        self._nvml = self._handle = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self._handle = pynvml.nvmlDeviceGetHandleByIndex(self._physical_index(index))
            self._nvml = pynvml
        except Exception:  # noqa: BLE001
            self._nvml = self._handle = None
        self._t = threading.Thread(target=self._run, daemon=True)

    @staticmethod
    def _physical_index(index: int) -> int:
        vis = os.environ.get("CUDA_VISIBLE_DEVICES", "")
        parts = [p for p in vis.split(",") if p.strip()]
        if parts and index < len(parts) and parts[index].strip().isdigit():
            return int(parts[index])
        return index

    def _sample_nvml(self):
        n, h = self._nvml, self._handle
        sm = n.nvmlDeviceGetClockInfo(h, n.NVML_CLOCK_SM)
        mx = n.nvmlDeviceGetMaxClockInfo(h, n.NVML_CLOCK_SM)
        try:
            mask = n.nvmlDeviceGetCurrentClocksEventReasons(h)
        except Exception:  # noqa: BLE001
            mask = n.nvmlDeviceGetCurrentClocksThrottleReasons(h)
        flag = lambda bit: "Active" if mask & bit else "Not Active"  # noqa: E731
        return [str(sm), str(mx), flag(n.nvmlClocksEventReasonHwSlowdown), flag(n.nvmlClocksEventReasonHwThermalSlowdown),
                flag(n.nvmlClocksEventReasonSwThermalSlowdown), flag(n.nvmlClocksEventReasonSwPowerCap)]

    def sample_now(self) -> None:
        """One synchronous sample (no-op without the Python binding)."""
        if self._nvml is not None:
            try:
                self.samples.append(self._sample_nvml())
            except Exception:  # noqa: BLE001
                pass

    def _run(self):
        while not self._stop.is_set():
            try:
                if self._nvml is not None:
                    self.samples.append(self._sample_nvml())
                else:
                    out = subprocess.run(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-i", str(self.index)],
                                         capture_output=True, text=True, timeout=5).stdout.strip()
                    if out:
                        self.samples.append([f.strip() for f in out.split(",")])
            except Exception:  # noqa: BLE001
                pass
            self._stop.wait(self.period_s if self._nvml is not None else 0.2)

    def __enter__(self):
        if self.period_s is not None:
            self._t.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        if self._t.is_alive():
            self._t.join(timeout=6)

    def summary(self) -> dict:
        def num(s):
            try:
                return float(s)
            except ValueError:
                return None
        sm = [v for v in (num(s[0]) for s in self.samples if s) if v is not None]
        mx = [v for v in (num(s[1]) for s in self.samples if len(s) > 1) if v is not None]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({names[i] for s in self.samples for i in range(4) if len(s) >= 6 and s[2 + i].lower().startswith("active")})
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(self.samples)}
