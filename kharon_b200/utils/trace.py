"""Phase tracing: CUDA-event timelines, NVTX ranges and a roofline report.

``Tracer.range(name)`` brackets a region with CUDA events on the current stream (and an NVTX range
when running under a profiler that shows them); ``report()`` sums device time per name after one
synchronisation, so tracing adds no host-device sync inside the step.  ``roofline()`` turns an
achieved FLOP or byte rate into a fraction of the measured peaks (``MEASURED_PEAKS.json`` at the repo
root, else the stated fall-back: 6.65 TB/s copy bandwidth and 1.59 PFLOP/s bf16, an earlier
measurement on the same pool).  The reference only had ad-hoc cudaEvent windows and differential
timing (src/pp_train.c:119-176).
"""
from __future__ import annotations

import contextlib
import json
import os
import time
from collections import defaultdict

import torch

_FALLBACK = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


def measured_peaks():
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "MEASURED_PEAKS.json")
    try:
        d = json.load(open(path))
        d["source"] = "measured"
        return d
    except Exception:
        return dict(_FALLBACK)


def roofline(flops: float = 0.0, bytes_: float = 0.0, ms: float = 1.0, sustained: bool = False):
    """Fractions of the measured tensor and memory peaks reached by a region that took ``ms``."""
    pk = measured_peaks()
    tf = pk["bf16_tflops_sustained" if sustained else "bf16_tflops"]
    out = {"of": pk["source"], "ms": ms}
    if flops:
        out["tflops"] = flops / ms / 1e9
        out["tensor_frac"] = out["tflops"] / tf
    if bytes_:
        out["gbs"] = bytes_ / ms / 1e6
        out["hbm_frac"] = out["gbs"] / pk["hbm_gbs"]
    return out


class Tracer:
    def __init__(self, enabled=True, nvtx=True):
        self.enabled = enabled
        self.cuda = torch.cuda.is_available()
        self.nvtx = nvtx and self.cuda
        self.pending = []                  # (name, start event | float, end event | float)
        self.totals = defaultdict(float)
        self.counts = defaultdict(int)

    @contextlib.contextmanager
    def range(self, name: str):
        if not self.enabled:
            yield
            return
        if self.cuda:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            if self.nvtx:
                torch.cuda.nvtx.range_push(name)
            e0.record()
            try:
                yield
            finally:
                e1.record()
                if self.nvtx:
                    torch.cuda.nvtx.range_pop()
                self.pending.append((name, e0, e1))
        else:
            t0 = time.perf_counter()
            try:
                yield
            finally:
                self.pending.append((name, t0, time.perf_counter()))

    def flush(self):
        if self.cuda and self.pending:
            torch.cuda.synchronize()
        for name, a, b in self.pending:
            ms = a.elapsed_time(b) if self.cuda else (b - a) * 1e3
            self.totals[name] += ms
            self.counts[name] += 1
        self.pending.clear()

    def report(self, reset=True):
        """{name: (calls, total ms)} since the last report."""
        self.flush()
        out = {k: (self.counts[k], self.totals[k]) for k in self.totals}
        if reset:
            self.totals.clear()
            self.counts.clear()
        return out

    def format(self, rep=None):
        rep = self.report() if rep is None else rep
        tot = sum(v[1] for v in rep.values()) or 1.0
        return "\n".join("  %-24s %6d calls %10.3f ms %5.1f %%" % (k, n, ms, 100 * ms / tot)
                         for k, (n, ms) in sorted(rep.items(), key=lambda kv: -kv[1][1]))


class JsonlLogger:
    """Appends one JSON object per call to a file (machine-readable twin of the printed log lines)."""

    def __init__(self, path):
        self.path = path
        if path:
            os.makedirs(os.path.dirname(path) or ".", exist_ok=True)

    def log(self, **kv):
        if not self.path:
            return
        kv.setdefault("time", time.time())
        with open(self.path, "a") as f:
            f.write(json.dumps(kv) + "\n")
