"""CUDA-event phase timers and an nvidia-smi clock sampler.

``PhaseTimers`` keeps the seven per-group columns that the reference's
communication thread prints every 100 samples (allreducer.py:334-387:
backward, merge, compression, allreduce, demerge, d2h, h2d), measured here with
CUDA events on the stream that runs the phase instead of host wall clock
around device synchronisations.
"""
from __future__ import annotations

import contextlib
import statistics
import subprocess
import threading
from collections import defaultdict
from typing import Dict, List, Optional

import torch

from .. import settings


def nvtx_push(name: str) -> None:
    if settings.NVTX and torch.cuda.is_available():
        torch.cuda.nvtx.range_push(name)


def nvtx_pop() -> None:
    if settings.NVTX and torch.cuda.is_available():
        torch.cuda.nvtx.range_pop()


@contextlib.contextmanager
def nvtx_range(name: str):
    """NVTX range when ``settings.NVTX`` is on; nothing otherwise."""
    nvtx_push(name)
    try:
        yield
    finally:
        nvtx_pop()


class CudaTimer:
    """start()/stop() pairs on the current stream; elapsed times are resolved
    lazily so that timing never synchronises the hot path."""

    def __init__(self, enabled: bool = True):
        self.enabled = enabled and torch.cuda.is_available()
        self._pending: List = []
        self._done: List[float] = []
        self._open = None

    def start(self) -> None:
        if not self.enabled:
            return
        ev = torch.cuda.Event(enable_timing=True)
        ev.record()
        self._open = ev

    def stop(self) -> None:
        if not self.enabled or self._open is None:
            return
        ev = torch.cuda.Event(enable_timing=True)
        ev.record()
        self._pending.append((self._open, ev))
        self._open = None

    def resolve(self) -> List[float]:
        """Seconds of every finished interval (keeps unfinished ones pending)."""
        keep = []
        for a, b in self._pending:
            if b.query():
                self._done.append(a.elapsed_time(b) * 1e-3)
            else:
                keep.append((a, b))
        self._pending = keep
        return self._done

    def drain(self) -> List[float]:
        if self._pending:
            torch.cuda.synchronize()
        out = list(self.resolve())
        self._done = []
        return out


class PhaseTimers:
    PHASES = ("backward", "merge", "compression", "allreduce", "demerge", "d2h", "h2d")

    def __init__(self, enabled: bool = True):
        self.enabled = enabled
        self._t: Dict[str, Dict[str, CudaTimer]] = defaultdict(dict)
        self._host: Dict[str, Dict[str, List[float]]] = defaultdict(lambda: defaultdict(list))

    def timer(self, group: str, phase: str) -> CudaTimer:
        d = self._t[group]
        if phase not in d:
            d[phase] = CudaTimer(self.enabled)
        return d[phase]

    def start(self, group: str, phase: str) -> None:
        nvtx_push("gtopk/" + phase)
        if self.enabled:
            self.timer(group, phase).start()

    def stop(self, group: str, phase: str) -> None:
        if self.enabled:
            self.timer(group, phase).stop()
        nvtx_pop()

    def add_host(self, group: str, phase: str, seconds: float) -> None:
        if self.enabled:
            self._host[group][phase].append(seconds)

    def samples(self, group: str) -> int:
        t = self._t.get(group, {}).get("allreduce")
        host = len(self._host.get(group, {}).get("allreduce", []))
        return host + (len(t._pending) + len(t._done) if t is not None else 0)

    def means(self, group: str) -> Dict[str, float]:
        out = {}
        for ph in self.PHASES:
            vals = list(self._host.get(group, {}).get(ph, []))
            t = self._t.get(group, {}).get(ph)
            if t is not None:
                vals += t.drain()
            out[ph] = statistics.fmean(vals) if vals else 0.0
        self._host.pop(group, None)
        return out


_QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
          "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
          "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a timed
    region runs (read-only; never changes a GPU setting)."""

    def __init__(self, gpu_index: int = 0, period_ms: int = 200):
        self.gpu_index, self.period_ms = gpu_index, period_ms
        self._proc: Optional[subprocess.Popen] = None
        self._lines: List[str] = []
        self._thread: Optional[threading.Thread] = None

    def start(self) -> None:
        try:
            self._proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.gpu_index), "--query-gpu=" + _QUERY, "--format=csv,noheader,nounits",
                 "-lms", str(self.period_ms)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self._proc = None
            return

        def pump():
            assert self._proc is not None and self._proc.stdout is not None
            for line in self._proc.stdout:
                self._lines.append(line.strip())

        self._thread = threading.Thread(target=pump, daemon=True)
        self._thread.start()

    def stop(self) -> dict:
        if self._proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self._proc.terminate()
        try:
            self._proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self._proc.kill()
        if self._thread is not None:
            self._thread.join(timeout=2)
        sm, mx, power, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        if not self._lines:  # the region was shorter than nvidia-smi's start-up: one query right after it
            try:
                out = subprocess.run(["nvidia-smi", "-i", str(self.gpu_index), "--query-gpu=" + _QUERY,
                                      "--format=csv,noheader,nounits"], capture_output=True, text=True, timeout=10)
                self._lines = [l.strip() for l in out.stdout.splitlines() if l.strip()]
            except (OSError, subprocess.TimeoutExpired):
                pass
        for line in self._lines:
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
                power.append(float(f[3]))
            except ValueError:
                continue
            for name, val in zip(names, f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        busy = [s for s, p in zip(sm, power) if p >= 0.5 * max(power)] or sm
        return {"sm_mhz": statistics.median(busy), "sm_max_mhz": max(mx), "power_w_max": max(power),
                "samples": len(sm), "reasons": sorted(reasons)}
