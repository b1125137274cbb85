"""Timing primitives for the decode path on one GPU.

B200 restatement of the four primitives of the reference's measurement harness that
its numbers rest on (benchmark.py): ``bench_graph`` (:556-612, "hot": one cache,
CUDA-graph replay of back-to-back calls), ``bench_graph_rotating`` (:641-694, "cold":
one graph holding one call per distinct cache copy, working set >= 3x L2),
``replicas_for`` (:625-638) and ``stats`` (:697-728), plus a clock sampler in place
of its ``ClockMonitor`` (:130-300).  The laptop-specific clock gating, ramping and
preload logic of the original is not reproduced: a B200 holds its clocks.

Everything is timed on the device with CUDA events on the launching stream.
"""

from __future__ import annotations

import statistics
import subprocess
import threading
import time

import torch


def stats(xs: list[float]) -> dict:
    """Median / quartiles / IQR of per-call times in ms."""
    s = sorted(xs)
    n = len(s)

    def q(f: float) -> float:
        if n == 1:
            return s[0]
        i = f * (n - 1)
        lo = int(i)
        hi = min(lo + 1, n - 1)
        return s[lo] + (s[hi] - s[lo]) * (i - lo)

    med = statistics.median(s)
    p25, p75 = q(0.25), q(0.75)
    return {
        "mean_ms": statistics.fmean(s),
        "std_ms": statistics.pstdev(s) if n > 1 else 0.0,
        "median_ms": med,
        "p25_ms": p25,
        "p75_ms": p75,
        "iqr_ms": p75 - p25,
        "iqr_frac_of_median": (p75 - p25) / med if med else None,
        "min_ms": s[0],
        "max_ms": s[-1],
        "n": n,
    }


def replicas_for(cache_bytes: int, l2_bytes: int, factor: float = 3.0,
                 max_replicas: int = 4096, max_total_bytes: int = 16 << 30) -> int:
    """How many distinct copies of a cache to rotate through so the set cannot sit in
    L2: ``factor`` x L2 (read from the device, 126 MB on B200).  The reference caps
    this at 512 copies / 400 MB for an 8 GB card; with 180 GB of HBM the caps are
    lifted to 4096 copies / 16 GiB so the smallest caches still reach 3x L2."""
    if cache_bytes <= 0:
        return 1
    target = int(factor * (l2_bytes or 0))
    want = -(-target // cache_bytes)
    by_bytes = max(1, max_total_bytes // cache_bytes)
    return int(max(1, min(max_replicas, want, by_bytes)))


def _capture(fns, repeat: int = 1):
    """Warm up on a side stream, then capture ``repeat`` passes over ``fns``."""
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for f in fns:
            f()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for _ in range(repeat):
            for f in fns:
                f()
    torch.cuda.synchronize()
    return g


def _sample_graph(g, calls_per_replay: int, samples: int, min_seconds: float,
                  max_seconds: float = 6.0, warm_replays: int = 3) -> list[float]:
    for _ in range(warm_replays):
        g.replay()
    torch.cuda.synchronize()
    out = []
    t0 = time.time()
    while True:
        s = torch.cuda.Event(enable_timing=True)
        e = torch.cuda.Event(enable_timing=True)
        s.record()
        g.replay()
        e.record()
        e.synchronize()
        out.append(s.elapsed_time(e) / calls_per_replay)
        el = time.time() - t0
        if len(out) >= samples and (el >= min_seconds or el >= max_seconds):
            break
    return out


def bench_graph(fn, samples: int = 30, iters: int = 50, min_seconds: float = 0.1) -> list[float]:
    """Hot regime: per-call ms of ``iters`` back-to-back calls on one cache, replayed
    as one CUDA graph (launch overhead removed, cache resident in L2 if it fits)."""
    g = _capture([fn], repeat=iters)
    return _sample_graph(g, iters, samples, min_seconds)


def bench_graph_rotating(fns, samples: int = 30, min_seconds: float = 0.1) -> list[float]:
    """Cold regime: per-call ms of one graph holding one call per distinct cache copy."""
    g = _capture(fns, repeat=1)
    return _sample_graph(g, len(fns), samples, min_seconds)


class StepGraphs:
    """EXACTLY ``K`` steps as CUDA-graph replays: ``K // L`` replays of an ``L``-call
    graph plus one remainder graph, the calls cycling over ``fns``."""

    def __init__(self, fns, K: int, max_len: int = 1000):
        n = len(fns)
        L = min(K, max(n, (max_len // n) * n))
        self.full_len = L
        self.n_full = K // L
        self.rem = K - self.n_full * L
        seq = [fns[i % n] for i in range(L)]
        self.g_full = _capture(seq)
        self.g_rem = _capture(seq[: self.rem]) if self.rem else None
        self.K = K

    def run(self):
        for _ in range(self.n_full):
            self.g_full.replay()
        if self.g_rem is not None:
            self.g_rem.replay()


def time_region(run, sync_barrier=None) -> float:
    """ms of ``run()`` on the current stream, CUDA events, synchronised on both sides."""
    torch.cuda.synchronize()
    if sync_barrier is not None:
        sync_barrier()
    s = torch.cuda.Event(enable_timing=True)
    e = torch.cuda.Event(enable_timing=True)
    s.record()
    run()
    e.record()
    torch.cuda.synchronize()
    return s.elapsed_time(e)


_REASONS = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]


class ClockSampler:
    """Samples ``nvidia-smi`` (read-only queries) every ``period_ms`` in a child
    process while a measurement runs; never changes a GPU setting."""

    def __init__(self, gpu_index: int = 0, period_ms: int = 100):
        self.rows: list[list[str]] = []
        self.proc = None
        self.thread = None
        fields = ("clocks.sm,clocks.max.sm,power.draw,utilization.gpu,"
                  + ",".join(f"clocks_event_reasons.{r}" for r in _REASONS))
        self.cmd = ["nvidia-smi", f"--id={gpu_index}", f"--query-gpu={fields}",
                    "--format=csv,noheader,nounits", "-lms", str(period_ms)]

    def start(self):
        try:
            self.proc = subprocess.Popen(self.cmd, stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
        except Exception:
            self.proc = None
            return self

        def reader():
            for line in self.proc.stdout:
                parts = [p.strip() for p in line.split(",")]
                if len(parts) >= 4 + len(_REASONS):
                    self.rows.append(parts)

        self.thread = threading.Thread(target=reader, daemon=True)
        self.thread.start()
        return self

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        self.proc.terminate()  # the exact child started above
        try:
            self.proc.wait(timeout=5)
        except Exception:
            pass
        if self.thread is not None:
            self.thread.join(timeout=2)
        sm, smax, reasons, power = [], [], set(), []
        for r in self.rows:
            try:
                util = float(r[3])
                clk = float(r[0])
            except ValueError:
                continue
            smax.append(float(r[1]))
            if util >= 20.0:
                sm.append(clk)
                try:
                    power.append(float(r[2]))
                except ValueError:
                    pass
                for name, flag in zip(_REASONS, r[4:4 + len(_REASONS)]):
                    if flag.lower().startswith("active"):
                        reasons.add(name)
        return {
            "sm_mhz": statistics.median(sm) if sm else None,
            "sm_max_mhz": max(smax) if smax else None,
            "power_w_max": max(power) if power else None,
            "reasons": sorted(reasons),
            "samples": len(self.rows),
            "samples_under_load": len(sm),
        }
