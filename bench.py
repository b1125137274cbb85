#!/usr/bin/env python
"""Benchmark of the packed-KV decode-attention path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--workload llama8b-b64|qwen-b1|llama70b-128k|ragged-b16|l2-sweep]
                    [--nbits 4|2] [--ctx N] [--batch B] [--samples 30]

One "step" is one decode step: one call of ``fused_decode_attention`` over the whole
cache of the workload.  The metric is the algorithmic HBM bandwidth of that step
(cache bytes / step time; ``ms_per_step`` carries the step time), in the COLD regime:
the K timed steps rotate over R distinct cache copies whose total size is >= 3x L2,
replayed as CUDA graphs so launch overhead is not part of the number.  The K-step
region is timed ``--samples`` times (CUDA events, barrier + synchronize on both sides,
max over ranks per sample); the line reports the median and the interquartile range.

Default workload: Llama-3-8B-shaped decode attention, batch 64, ctx 4096, 4-bit, group 32.
Under torchrun (N > 1) the batch is sharded over the ranks with no data-path collective
(strong scaling).  The same JSON line carries, for the same shape, the same-split fp16
control (hot and cold), the 2-bit cell, a ``history_split`` record (Llama-3-70B shape,
ctx 131072, 2-bit, the history split over the N ranks with an exchange of (acc, m, l)
partials and a log-sum-exp merge) and, at N = 1, the single-sequence sweep ``rows``.
At N > 1 the sharded paths are first checked against the CPU oracle
(``parity_vs_oracle``).

``--impl reference`` times the CPU path the reference itself runs (dequantise the
cache in fp32, then fp32 attention) through the C restatement under ``oracle/`` on
all host cores, for the same workload, inputs and metric.
"""

from __future__ import annotations

import argparse
import json
import math
import os
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "decode-step algorithmic HBM GB/s, fused packed-KV attention, cold (rotating >=3x L2)"
GS = 32
FALLBACK_HBM_GBS = 6650.0
CHUNK = 4096  # tokens per independently seeded piece of a host-generated sequence

WORKLOADS = {
    # name: (B, HQ, HKV, D, default ctx, default nbits, value distribution, description)
    "llama8b-b64": (64, 32, 8, 128, 4096, 4, "normal", "Llama-3-8B shape, batch 64, ctx 4096"),
    "qwen-b1": (1, 12, 2, 128, 65536, 4, "channel", "Qwen2.5-1.5B attention shape, batch 1"),
    "llama70b-128k": (1, 64, 8, 128, 131072, 2, "normal", "Llama-3-70B shape, batch 1, ctx 131072"),
    # ragged batch: per-sequence lengths uniform in [1024, ctx] from the seed; bytes counted
    # are those of the valid tokens only
    "ragged-b16": (16, 32, 8, 128, 32768, 4, "entry", "ragged batch 16, lengths uniform in [1024, 32768]"),
    # fp16 cache footprint from 0.125x to 12x the L2 size, fused 4-bit vs the fp16 control
    "l2-sweep": (1, 12, 2, 128, 0, 4, "channel", "Qwen2.5-1.5B shape, contexts placed by fp16 footprint / L2"),
}

# DRAM traffic of the split kernel relative to its algorithmic bytes, from the ncu captures
# summarised under profiles/ (dram__bytes_read.sum + dram__bytes_write.sum per launch over the
# cache bytes of that launch).  Traffic grows in proportion to the cache (every byte is read
# once, L2 hit rate 1-2 %), so the ratio measured at the capture size carries to the bench size.
NCU_TRAFFIC_RATIO = {
    # profiles/splitk_fused_4bit_llama8b_batch16.md: (84.07 MB read + 2.57 MB written) / 83.89 MB
    ("llama8b-b64", 4): (84_073_216 + 2_570_752) / 83_886_080,
    # profiles/splitk_fused_2bit_llama8b_batch16.md: (50.51 MB read + 2.05 MB written) / 50.33 MB
    ("llama8b-b64", 2): (50_514_688 + 2_048_000) / 50_331_648,
    # profiles/splitk_fused_4bit_qwen_ctx65536.md: 21.02 MB read / 20.97 MB
    ("qwen-b1", 4): 21_023_488 / 20_971_520,
}


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    # 20-step regions (about a millisecond) by default: the copy peak the roofline is stated
    # against was measured as a burst of that length; regions of hundreds of steps hold the
    # board at its power cap and read about 10 % lower
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="llama8b-b64", choices=sorted(WORKLOADS))
    ap.add_argument("--nbits", type=int, default=None)
    ap.add_argument("--ctx", type=int, default=None)
    ap.add_argument("--batch", type=int, default=None, help="override the workload's batch size")
    ap.add_argument("--samples", type=int, default=30, help="timed repeats of the K-step region")
    ap.add_argument("--no-table", action="store_true", help="skip the single-sequence sweep rows")
    ap.add_argument("--no-extras", action="store_true",
                    help="skip the fp16 control, 2-bit and history-split records")
    ap.add_argument("--light", action="store_true",
                    help="timed region only: no extras, CPU baseline, end-to-end leg or oracle "
                         "check (for profiler captures)")
    ap.add_argument("--seed", type=int, default=0)
    return ap.parse_args()


def fused_bytes(B, HKV, S, D, nbits, gs=GS):
    return B * HKV * S * (2 * D * nbits // 8 + 8 * (D // gs))


def fp16_bytes(B, HKV, S, D):
    return B * HKV * S * 4 * D


def measured_peak():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(p) as f:
            return float(json.load(f)["hbm_gbs"]), "measured (MEASURED_PEAKS.json)"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


def workload_config(name, B, HQ, HKV, D, ctx, nbits, n_gpus):
    """The ``config`` object of the JSON line: the whole job, identical for both arms."""
    desc = WORKLOADS[name][7]
    if name == "llama70b-128k":
        part = "history split over the ranks, exchange of (acc, m, l), log-sum-exp merge"
    elif name == "llama8b-b64":
        part = "batch sharded over the ranks, no data-path collective"
    else:
        part = "one copy of the workload per rank, no data-path collective"
    return {"workload": f"{name}: {desc}; B={B} HQ={HQ} HKV={HKV} D={D} ctx={ctx}, {nbits}-bit, group {GS}",
            "partition": part if n_gpus > 1 else "single GPU"}


# ------------------------------------------------------------------ seeded host inputs


def _gen(seed, *key):
    import torch

    s = seed & 0x7fffffff
    for k in key:
        s = (s * 1_000_003 + (k + 7)) & 0x7fffffffffff
    return torch.Generator(device="cpu").manual_seed(s)


def host_sequence(name, b, t0, t1, seed):
    """Tokens [t0, t1) of sequence ``b`` of workload ``name``: (k, v) fp16 CPU tensors
    (HKV, t1-t0, D).  Generated in independently seeded chunks of CHUNK tokens, so any
    token range of any sequence is reproducible on its own -- the GPU arm (whatever the
    number of ranks and whichever shard a rank owns) and the CPU arm see the same values."""
    import torch

    _, HQ, HKV, D, _, _, dist_kind, _ = WORKLOADS[name]
    ks, vs = [], []
    for c in range(t0 // CHUNK, (t1 + CHUNK - 1) // CHUNK):
        g = _gen(seed, b, c)
        k = torch.randn(HKV, CHUNK, D, generator=g, dtype=torch.float32)
        v = torch.randn(HKV, CHUNK, D, generator=g, dtype=torch.float32)
        if dist_kind == "entry":  # 1 % of the K entries (only K) x20
            k = torch.where(torch.rand(HKV, CHUNK, D, generator=g) < 0.01, k * 20.0, k)
        lo, hi = max(t0, c * CHUNK) - c * CHUNK, min(t1, (c + 1) * CHUNK) - c * CHUNK
        ks.append(k[:, lo:hi])
        vs.append(v[:, lo:hi])
    k = torch.cat(ks, dim=1) if len(ks) > 1 else ks[0]
    v = torch.cat(vs, dim=1) if len(vs) > 1 else vs[0]
    if dist_kind == "channel":  # per-channel lognormal(0, 0.5) factors on K: outlier channels
        chan = torch.exp(0.5 * torch.randn(HKV, D, generator=_gen(seed, -1, -1), dtype=torch.float32))
        k = k * chan[:, None, :]
    return k.half().contiguous(), v.half().contiguous()


def host_query(name, b, seed):
    import torch

    _, HQ, _, D = WORKLOADS[name][:4]
    return torch.randn(HQ, D, generator=_gen(seed, b, -2), dtype=torch.float32).half()


def host_batch(name, b_lo, b_hi, t0, t1, seed):
    """q (nb, HQ, D), k, v (nb, HKV, t1-t0, D) fp16 CPU tensors of sequences [b_lo, b_hi)."""
    import torch

    qs, ks, vs = [], [], []
    for b in range(b_lo, b_hi):
        k, v = host_sequence(name, b, t0, t1, seed)
        qs.append(host_query(name, b, seed))
        ks.append(k)
        vs.append(v)
    return torch.stack(qs), torch.stack(ks), torch.stack(vs)


# ----------------------------------------------------------------------------- CPU arm


def time_cpu(q, kq, vq, S, D, nbits, steps, warmup, budget_s):
    """Time the reference's CPU path (C restatement, all host cores): dequantise K and V to
    fp32, then fp32 softmax attention.  ``q`` (B, HQ, D) float32, ``kq``/``vq`` = (packed,
    scale, zero) numpy arrays of the whole cache.  If ``steps + warmup`` steps of the whole
    cache do not fit ``budget_s`` the sample is the first ``B_s`` sequences (whole
    sequences) or, for a single sequence, its first ``S_s`` tokens.
    Returns (GB/s, seconds per step, info)."""
    from oracle import c_oracle

    c_oracle.use_all_cores()
    B, HQ, _ = q.shape
    HKV = kq[0].shape[1]

    def make(B_s, S_s):
        sl = [a[:B_s, :, :S_s].copy() for a in (*kq, *vq)]
        step = c_oracle.DecodeStep(B_s, HQ, HKV, S_s, D, nbits, GS)
        qs = q[:B_s].copy()
        return lambda: step(qs, *sl)

    probe_S = min(S, 1024)
    run = make(1, probe_S)
    run()
    t0 = time.perf_counter()
    for _ in range(3):
        run()
    per_token = (time.perf_counter() - t0) / 3 / probe_S  # one sequence, per token
    n = max(1, steps + warmup)
    whole = per_token * S * B * n
    B_s, S_s = B, S
    if whole > budget_s:
        if B > 1:
            B_s = int(max(1, min(B, budget_s / (per_token * S * n))))
        if B_s == 1 and per_token * S * n > budget_s:
            S_s = int(max(256, budget_s / (per_token * n)))
            S_s = max(16, min(S, (S_s // 16) * 16))
    run = make(B_s, S_s)
    for _ in range(max(1, warmup)):
        run()
    t0 = time.perf_counter()
    for _ in range(steps):
        run()
    dt = (time.perf_counter() - t0) / steps
    nbytes = fused_bytes(B_s, HKV, S_s, D, nbits)
    what = ("the whole configuration" if (B_s, S_s) == (B, S) else
            f"the first {B_s} of {B} sequences, first {S_s} of {S} tokens of each")
    info = {
        "cores": c_oracle.num_threads(),
        "kind": "port",
        "sample": f"{what}; {steps} steps after {max(1, warmup)} warm-up; dequantise K,V to fp32 "
                  f"then fp32 softmax attention (oracle/tkv_oracle.c, OpenMP)",
    }
    return nbytes / dt / 1e9, dt, info


def host_quantized(name, B, S, nbits, seed):
    """Replica 0 of the workload on the host: q float32 (B, HQ, D), (packed, scale, zero) of K and V."""
    import numpy as np

    from oracle import c_oracle

    c_oracle.use_all_cores()
    qs, kqs, vqs = [], [], []
    for b in range(B):  # per sequence: bounds the fp32 temporaries
        q, k, v = host_batch(name, b, b + 1, 0, S, seed)
        qs.append(q.float().numpy())
        kqs.append(c_oracle.quantize_groupwise(k.float().numpy(), nbits, GS))
        vqs.append(c_oracle.quantize_groupwise(v.float().numpy(), nbits, GS))
    cat = lambda parts: tuple(np.concatenate([p[i] for p in parts], axis=0) for i in range(3))
    return np.concatenate(qs, axis=0), cat(kqs), cat(vqs)


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    name = args.workload if args.workload != "l2-sweep" else "qwen-b1"
    B, HQ, HKV, D, ctx, nbits, _, _ = WORKLOADS[name]
    ctx = args.ctx or ctx
    nbits = args.nbits or nbits
    B = args.batch or B
    steps = max(1, args.steps)
    q, kq, vq = host_quantized(name, B, ctx, nbits, args.seed)
    gbs, dt, info = time_cpu(q, kq, vq, ctx, D, nbits, steps, args.warmup, budget_s=120.0)
    line = {
        "impl": "reference",
        "metric": METRIC, "value": gbs, "unit": "GB/s", "n_gpus": args.gpus, "steps": steps,
        "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": "strong" if name in ("llama8b-b64", "llama70b-128k") else "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(name, B, HQ, HKV, D, ctx, nbits, args.gpus),
        "cpu_baseline": {"value": gbs, "unit": "GB/s", **info},
        "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


# ----------------------------------------------------------------------------- GPU arm


class Ctx:
    """What every leg of the GPU arm needs: device, ranks, timing helpers."""

    def __init__(self, args):
        import torch

        from tritonkv_b200 import _cabi, harness

        self.torch, self.harness, self.args = torch, harness, args
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.rank = int(os.environ.get("RANK", "0"))
        self.local = int(os.environ.get("LOCAL_RANK", "0"))
        ok, why = _cabi.available()
        if not ok:
            raise RuntimeError(f"bench.py needs the CUDA library on a GPU: {why}")
        torch.cuda.set_device(self.local)
        self.device = torch.device("cuda", self.local)
        self.dist = None
        if self.world > 1:
            import torch.distributed as dist

            dist.init_process_group("nccl", device_id=self.device)
            self.dist = dist
        self.l2 = _cabi.device_info(self.local)["l2_bytes"]
        self.peak, self.peak_src = measured_peak()
        self.K, self.W = max(1, args.steps), max(3, args.warmup)
        self.samples = max(1, args.samples)

    def barrier(self):
        if self.dist is not None:
            self.dist.barrier()

    def max_over_ranks(self, x: float) -> float:
        if self.dist is None:
            return x
        t = self.torch.tensor([x], device=self.device, dtype=self.torch.float64)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t.item())

    def all_ok(self, ok: bool) -> bool:
        if self.dist is None:
            return ok
        t = self.torch.tensor([1 if ok else 0], device=self.device)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MIN)
        return bool(t.item())

    def time_steps(self, fns, K=None, W=None, graphs=True, samples=None):
        """EXACTLY ``K`` steps cycling over ``fns`` (one per distinct cache), timed ``samples``
        times after ``W`` warm-up steps: barrier + synchronize on both sides of every sample,
        CUDA events on the launching stream, max over ranks.  Returns the statistics of the
        per-sample times in ms (of the whole K-step region) and whether graphs were used."""
        h, torch = self.harness, self.torch
        K = K or self.K
        W = self.W if W is None else W
        samples = samples or self.samples
        if graphs:
            sg = h.StepGraphs(fns, K)
            wg = h.StepGraphs(fns, W) if W != K else sg
            # The first launch of an instantiated graph uploads it to the device (set-up
            # cost, not step time): replay once before the warm-up steps.
            sg.run()
            wg.run()
            run = sg.run
        else:
            n = len(fns)

            def run_n(count):
                for i in range(count):
                    fns[i % n]()
            run_n(W)
            run = lambda: run_n(K)
        torch.cuda.synchronize()
        xs = [self.max_over_ranks(h.time_region(run, self.barrier)) for _ in range(samples)]
        return h.stats(xs)


def device_replicas(cx, name, B, S, nbits, n_fused, n_fp16, seed, b_lo=0, t_lo=0):
    """``max(n_fused, n_fp16)`` distinct caches on the device.  Copy 0 holds the seeded host
    values of sequences [b_lo, b_lo+B), tokens [t_lo, t_lo+S) (``host_batch``: what the CPU arm
    and the parity checks use); the further copies, which only keep the working set out of L2,
    are drawn on the device from the same distribution."""
    torch = cx.torch
    from tritonkv_b200 import quantize as Q

    _, HQ, HKV, D, _, _, dist_kind, _ = WORKLOADS[name]
    dev = cx.device
    reps = []
    for i in range(max(n_fused, n_fp16, 1)):
        if i == 0:
            q, k, v = (t.to(dev) for t in host_batch(name, b_lo, b_lo + B, t_lo, t_lo + S, seed))
        else:
            g = torch.Generator(device=dev).manual_seed(seed * 7919 + 104729 * i + cx.rank)
            q = torch.randn(B, HQ, D, generator=g, device=dev, dtype=torch.float32).half()
            k = torch.randn(B, HKV, S, D, generator=g, device=dev, dtype=torch.float32)
            if dist_kind == "channel":
                k *= torch.exp(0.5 * torch.randn(HKV, D, generator=g, device=dev))[None, :, None, :]
            elif dist_kind == "entry":
                k = torch.where(torch.rand(B, HKV, S, D, generator=g, device=dev) < 0.01, k * 20.0, k)
            k = k.half()
            v = torch.randn(B, HKV, S, D, generator=g, device=dev, dtype=torch.float32).half()
        rep = {"q": q}
        if i < n_fused:
            rep["kq"], rep["vq"] = Q.quantize_kv(k, v, nbits, GS)
        if i < n_fp16:
            rep["k"], rep["v"] = k, v
        reps.append(rep)
        del k, v
    return reps


def oracle_check(q, kq, vq, got, seq_lens=None, rows=None):
    """Compare ``got`` (B, HQ, D) with the CPU oracle (the checker) on the quantised caches the
    kernel read; ``rows``: the sequences to check (all if None)."""
    import numpy as np

    from oracle import c_oracle
    from oracle import tkv_oracle as O

    idx = list(range(q.shape[0])) if rows is None else list(rows)
    it = cx_index(idx, q.device)
    h = lambda t: t.index_select(0, it).cpu().numpy()
    hm = lambda t: h(t).view(np.uint16)
    sl = None if seq_lens is None else seq_lens.index_select(0, it).cpu().numpy()
    ref = c_oracle.decode_step(h(q.float()), h(kq.packed), hm(kq.scale), hm(kq.zero), h(vq.packed),
                               hm(vq.scale), hm(vq.zero), kq.nbits, kq.group_size, seq_lens=sl)
    rep = O.allclose_report(h(got), ref)
    return {k: (bool(rep[k]) if k == "ok" else float(rep[k])) for k in ("ok", "max_abs_err", "rel_l2")}


def cx_index(idx, device):
    import torch

    return torch.tensor(idx, device=device, dtype=torch.long)


def multi_gpu_parity(cx):
    """N > 1, before any timing: the sharded paths against the CPU oracle.  A shortened
    Llama-3-70B history split (HQ 64 / HKV 8, 2-bit, ctx 6016 per rank) through both exchanges
    and a batch-sharded slice of the Llama-3-8B shape (2 sequences per rank, ctx 4096); every
    rank checks what it computed, the verdicts are all-reduced, the device status word is read."""
    torch = cx.torch
    from tritonkv_b200 import _cabi
    from tritonkv_b200 import parallel as P
    from tritonkv_b200 import quantize as Q
    from tritonkv_b200.kernels import fused_decode_attention

    res = {}
    name = "llama70b-128k"
    _, HQ, HKV, D = WORKLOADS[name][:4]
    S = 6016 * cx.world
    lo, hi = P.history_shard(S, cx.world, cx.rank)
    q, k, v = (t.to(cx.device) for t in host_batch(name, 0, 1, 0, S, cx.args.seed + 11))
    kq, vq = Q.quantize_kv(k, v, 2, GS)
    cut = lambda t: Q.QuantizedTensor(t.packed[:, :, lo:hi].contiguous(), t.scale[:, :, lo:hi].contiguous(),
                                      t.zero[:, :, lo:hi].contiguous(), 2, GS, D)
    kq_l, vq_l = cut(kq), cut(vq)
    for exchange in ("peer", "nccl"):
        key = f"history_split_{exchange}"
        try:
            dec = P.HistorySplitDecoder(1, HQ, D, cx.device, exchange=exchange)
        except Exception as exc:  # e.g. no symmetric memory on this system: every rank raises
            res[key] = f"unavailable: {exc!r}"[:300]
            continue
        outs = [dec.step(q, kq_l, vq_l).clone() for _ in range(3)]  # the buffers are reused per step
        torch.cuda.synchronize()
        rep = oracle_check(q, kq, vq, outs[0])  # every rank holds the merged result
        ok = rep["ok"] and all(torch.equal(outs[0], o) for o in outs[1:])
        res[key] = {"ok": cx.all_ok(ok), "max_abs_err": cx.max_over_ranks(rep["max_abs_err"]),
                    "ctx": S, "exchange": dec.exchange}
        dec.close()
        del dec
    name = "llama8b-b64"
    _, HQ, HKV, D = WORKLOADS[name][:4]
    Bt = 2 * cx.world
    b_lo, b_hi = P.batch_shard(Bt, cx.world, cx.rank)
    q, k, v = (t.to(cx.device) for t in host_batch(name, b_lo, b_hi, 0, 4096, cx.args.seed + 12))
    kq, vq = Q.quantize_kv(k, v, 4, GS)
    rep = oracle_check(q, kq, vq, fused_decode_attention(q, kq, vq))
    res["batch_shard"] = {"ok": cx.all_ok(rep["ok"]), "max_abs_err": cx.max_over_ranks(rep["max_abs_err"]),
                          "sequences": Bt, "ctx": 4096}
    res["device_status"] = int(cx.max_over_ranks(float(_cabi.device_status())))
    bad = [k for k, r in res.items() if isinstance(r, dict) and not r["ok"]]
    if bad or res["device_status"] != 0:
        raise RuntimeError(f"multi-GPU parity against the oracle failed: {res}")
    return res


def fused_cell(cx, name, B, S, nbits, seed, b_lo=0, want_fp16=False, seq_lens=None, valid_frac=1.0):
    """Build the rotating caches of one (shape, nbits) cell and return the closures of the
    step, of the split kernel alone and (optionally) of the fp16 control."""
    torch, h = cx.torch, cx.harness
    from tritonkv_b200.kernels import fp16_decode_attention, fused_decode_attention

    _, HQ, HKV, D = WORKLOADS[name][:4]
    cbytes = int(fused_bytes(B, HKV, S, D, nbits) * valid_frac)
    R = max(2, h.replicas_for(cbytes, cx.l2))
    R16 = max(2, h.replicas_for(fp16_bytes(B, HKV, S, D), cx.l2)) if want_fp16 else 0
    reps = device_replicas(cx, name, B, S, nbits, R, min(R16, R), seed, b_lo=b_lo)
    outs = [torch.empty(B, HQ, D, device=cx.device) for _ in range(R)]
    ws, ws2, ws16 = {}, {}, {}
    step = [(lambda r=r, o=o: fused_decode_attention(r["q"], r["kq"], r["vq"], out=o, _workspace=ws,
                                                     seq_lens=seq_lens)) for r, o in zip(reps, outs)]
    split = [(lambda r=r, o=o: fused_decode_attention(r["q"], r["kq"], r["vq"], out=o, _workspace=ws2,
                                                      _partials_only=True, seq_lens=seq_lens))
             for r, o in zip(reps, outs)]
    ctl = [(lambda r=r, o=o: fp16_decode_attention(r["q"], r["k"], r["v"], out=o, _workspace=ws16,
                                                   seq_lens=seq_lens))
           for r, o in zip(reps[:min(R16, R)], outs)]
    for f in step + split + ctl:  # first calls allocate the workspaces
        f()
    torch.cuda.synchronize()
    return {"reps": reps, "outs": outs, "ws": ws, "step": step, "split": split, "ctl": ctl,
            "bytes": cbytes, "bytes16": fp16_bytes(B, HKV, S, D), "R": R, "R16": min(R16, R)}


def per_channel_cell(cx, name, B, S, seed, b_lo, world):
    """The same shape with 2-bit keys quantised per channel over 32-token groups and 2-bit
    per-token values (``kernels.kivi_decode_attention``; the format the reference lists as
    future work): cold step time, same byte count per token as the 2-bit per-token cache."""
    torch, h = cx.torch, cx.harness
    from tritonkv_b200.kernels import kivi_decode_attention, quantize_kv_kivi

    _, HQ, HKV, D = WORKLOADS[name][:4]
    cbytes = fused_bytes(B, HKV, S, D, 2)
    R = max(2, h.replicas_for(cbytes, cx.l2))
    reps = device_replicas(cx, name, B, S, 2, 0, R, seed, b_lo=b_lo)
    caches = [(r["q"], quantize_kv_kivi(r.pop("k"), r.pop("v"), 2)) for r in reps]
    outs = [torch.empty(B, HQ, D, device=cx.device) for _ in range(R)]
    ws: dict = {}
    fns = [(lambda q=q, c=c, o=o: kivi_decode_attention(q, c, out=o, _workspace=ws))
           for (q, c), o in zip(caches, outs)]
    for f in fns:
        f()
    torch.cuda.synchronize()
    st = cx.time_steps(fns)
    return {"cold_us": us(st, cx.K), "GBps": cbytes * world * cx.K / (st["median_ms"] * 1e-3) / 1e9,
            "iqr_frac": st["iqr_frac_of_median"], "launches_per_step": 2,
            "what": "split kernel on per-channel keys + merge of its partials (no fp16 tail at this length)"}


def write_side_record(cx, name, B, S, nbits):
    """The cache's write side on the workload's shape: (a) quantise + pack the whole K tensor
    into a preallocated cache (what a prefill does; ``quantize.append_groupwise`` with all S
    tokens: the one-launch quantiser writing in place, no allocation), timed cold by size
    (the fp16 input alone is several times L2), against its algorithmic bytes
    ``2*D + D*nbits/8 + 4*D/gs`` per token row; (b) the decode loop's append of one new token
    per sequence to K and V (two launches)."""
    torch = cx.torch
    from tritonkv_b200 import quantize as Q

    _, HQ, HKV, D = WORKLOADS[name][:4]
    g = torch.Generator(device=cx.device).manual_seed(7)
    x = torch.randn(B, HKV, S, D, generator=g, device=cx.device, dtype=torch.float32).half()
    cache = Q.empty_cache(B, HKV, S, D, nbits, GS, cx.device)
    fns = [lambda: Q.append_groupwise(cache, x, 0)]
    st = cx.time_steps(fns, K=10, W=3, graphs=False)
    rows = B * HKV * S
    byt = rows * (2 * D + D * nbits // 8 + 4 * D // GS)
    t_us = us(st, 10)
    rec = {"quantize_pack_us": t_us, "tokens_rows": rows, "bytes": byt,
           "GBps": byt / (t_us * 1e-6) / 1e9, "frac_of_peak": byt / (t_us * 1e-6) / 1e9 / cx.peak,
           "what": f"fp16 (B,HKV,S,D) -> {nbits}-bit packed cache in place, one launch"}
    del x
    kq, vq = cache, Q.empty_cache(B, HKV, S, D, nbits, GS, cx.device)
    kn = torch.randn(B, HKV, 1, D, device=cx.device, dtype=torch.float16)
    vn = torch.randn_like(kn)
    pos = torch.full((B,), S // 2, device=cx.device, dtype=torch.int32)
    st = cx.time_steps([lambda: Q.append_kv(kq, vq, kn, vn, pos)])
    rec["append_one_token_us"] = us(st, cx.K)
    return rec


def us(stats, K):
    return stats["median_ms"] * 1e3 / K


def history_split_record(cx, seed):
    """Llama-3-70B shape, batch 1, ctx 131072, 2-bit: the history split over the ranks (peer
    exchange where symmetric memory is available, else one NCCL all-gather), strong scaling.
    On one GPU the same shape through ``fused_decode_attention``."""
    torch, h = cx.torch, cx.harness
    from tritonkv_b200 import parallel as P
    from tritonkv_b200.kernels import fused_decode_attention

    name = "llama70b-128k"
    B, HQ, HKV, D, S, nbits = WORKLOADS[name][:6]
    lo, hi = P.history_shard(S, cx.world, cx.rank)
    S_loc = hi - lo
    cbytes = fused_bytes(B, HKV, S_loc, D, nbits)
    R = max(2, h.replicas_for(cbytes, cx.l2))
    reps = device_replicas(cx, name, B, S_loc, nbits, R, 0, seed, t_lo=lo)
    for r in reps[1:]:  # the query is the same on every rank
        r["q"] = reps[0]["q"]
    K = cx.K
    rec = {"workload": workload_config(name, B, HQ, HKV, D, S, nbits, cx.world)["workload"],
           "tokens_per_rank": S_loc, "replicas": R}
    dec = None
    if cx.world > 1:
        dec = P.HistorySplitDecoder(B, HQ, D, cx.device)
        steps = [(lambda r=r: dec.step(r["q"], r["kq"], r["vq"])) for r in reps]
        out_dev = dec.out
        rec["exchange"] = ("stores into peer memory, tagged {value, step} pairs, one kernel"
                           if dec.exchange == "peer" else "one NCCL all-gather")
        # split kernel + the exchange kernel; with NCCL: split, local merge, all-gather, merge
        launches = 2 if dec.exchange == "peer" else 4
    else:
        out_dev = torch.empty(B, HQ, D, device=cx.device)
        ws: dict = {}
        steps = [(lambda r=r: fused_decode_attention(r["q"], r["kq"], r["vq"], out=out_dev, _workspace=ws))
                 for r in reps]
        rec["exchange"] = "none (one GPU)"
        launches = 2
    for s in steps:
        s()
    torch.cuda.synchronize()
    graphs = True
    if dec is not None and dec.exchange == "nccl":
        try:  # the step holds an NCCL all-gather: capture it, or fall back on every rank together
            h.StepGraphs(steps[:1], 1)
        except Exception as exc:
            graphs = False
            sys.stderr.write(f"[bench] graph capture of the NCCL step failed ({exc!r}); direct launches\n")
        graphs = cx.all_ok(graphs)
    st = cx.time_steps(steps, K, graphs=graphs)
    ws2: dict = {}
    o2 = torch.empty(B, HQ, D, device=cx.device)
    split = [(lambda r=r: fused_decode_attention(r["q"], r["kq"], r["vq"], out=o2, _workspace=ws2,
                                                 _partials_only=True)) for r in reps]
    for s in split:
        s()
    st_split = cx.time_steps(split, K)
    total = fused_bytes(B, HKV, S, D, nbits)
    rec.update({"us_per_step": us(st, K), "iqr_frac": st["iqr_frac_of_median"],
                "GBps": total / (st["median_ms"] * 1e-3 / K) / 1e9,
                "split_kernel_us": us(st_split, K), "graphs": graphs, "launches_per_step": launches})
    # end to end: q from pinned host memory, the step, out to pinned host memory, stream sync
    q_host = reps[0]["q"].cpu().pin_memory()
    q_dev = torch.empty_like(reps[0]["q"])
    out_host = torch.empty(B, HQ, D, dtype=torch.float32).pin_memory()
    stream = torch.cuda.current_stream()
    if dec is not None:
        call = [(lambda r=r: dec.step(q_dev, r["kq"], r["vq"])) for r in reps]
    else:
        call = [(lambda r=r: fused_decode_attention(q_dev, r["kq"], r["vq"], out=out_dev, _workspace=ws))
                for r in reps]

    def e2e_steps(n):
        for i in range(n):
            q_dev.copy_(q_host, non_blocking=True)
            call[i % R]()
            out_host.copy_(out_dev, non_blocking=True)
            stream.synchronize()

    Ke = min(K, 500)
    e2e_steps(20)
    xs = [cx.max_over_ranks(h.time_region(lambda: e2e_steps(Ke), cx.barrier)) for _ in range(5)]
    ms_e = h.stats(xs)["median_ms"]
    rec["e2e"] = {"value": total * Ke / (ms_e * 1e-3) / 1e9, "unit": "GB/s", "us_per_step": ms_e * 1e3 / Ke,
                  "h2d_bytes_per_step": int(q_dev.numel() * q_dev.element_size()),
                  "d2h_bytes_per_step": int(out_host.numel() * 4), "steps": Ke,
                  "path": "direct calls: q H2D, step, out D2H, stream sync, on every rank"}
    if dec is not None:
        torch.cuda.synchronize()
        cx.barrier()
        dec.close()
    return rec


def run_ours(args):
    import numpy as np
    import torch

    from tritonkv_b200 import _cabi

    cx = Ctx(args)
    h = cx.harness
    world, rank, device = cx.world, cx.rank, cx.device
    if args.workload == "l2-sweep":
        return run_l2_sweep(cx)
    name = args.workload
    B, HQ, HKV, D, ctx, nbits, _, _ = WORKLOADS[name]
    ctx = args.ctx or ctx
    nbits = args.nbits or nbits
    B_total = args.batch or B
    if args.light:
        args.no_table = args.no_extras = True
    K, W = cx.K, cx.W
    config = workload_config(name, B_total, HQ, HKV, D, ctx, nbits, world)

    sampler = h.ClockSampler(cx.local).start()
    parity = {}
    if world > 1 and not args.light:
        parity = multi_gpu_parity(cx)

    history_split = name == "llama70b-128k" and world > 1
    batch_sharded = name == "llama8b-b64" and world > 1
    scaling = "strong" if name in ("llama8b-b64", "llama70b-128k") else "weak"
    if history_split:
        # the headline IS the history split: its record carries the numbers
        rec = history_split_record(cx, args.seed)
        clocks = sampler.stop()
        if rank == 0:
            line = {"metric": METRIC, "value": rec["GBps"], "unit": "GB/s", "n_gpus": world, "steps": K,
                    "warmup": W, "ms_per_step": rec["us_per_step"] / 1e3, "higher_is_better": True,
                    "scaling": "strong", "vs_baseline": None, "dtype": "f16 operands / f32 accumulate",
                    "data": "synthetic", "config": config, "history_split": rec, "e2e": rec["e2e"],
                    "roofline": None, "cpu_baseline": None, "gpu_launches": rec["launches_per_step"] * K,
                    "clocks": clocks, "parity_vs_oracle": parity, "samples": cx.samples}
            print(json.dumps(line), flush=True)
        return teardown(cx)

    from tritonkv_b200 import parallel as P

    b_lo, b_hi = (P.batch_shard(B_total, world, rank) if batch_sharded else (0, B_total))
    B_loc = b_hi - b_lo
    seed = args.seed + (0 if batch_sharded or world == 1 else 1000 * rank)
    seq_lens, valid_frac = None, 1.0
    S_loc = ctx
    if name == "ragged-b16":
        g = torch.Generator(device="cpu").manual_seed(seed)  # lengths uniform in [1024, ctx]
        lens = torch.randint(1024, ctx + 1, (B_loc,), generator=g, dtype=torch.int64).to(torch.int32)
        S_loc = int(lens.max())
        seq_lens = lens.to(device)
        valid_frac = float(lens.sum()) / (B_loc * S_loc)
    cell = fused_cell(cx, name, B_loc, S_loc, nbits, seed, b_lo=b_lo,
                      want_fp16=not args.no_extras and name != "ragged-b16", seq_lens=seq_lens,
                      valid_frac=valid_frac)
    cbytes, R = cell["bytes"], cell["R"]
    if world > 1:
        t = torch.tensor([float(cbytes)], device=device, dtype=torch.float64)
        cx.dist.all_reduce(t)
        total_bytes = int(t.item())
    else:
        total_bytes = cbytes

    # ---- parity of copy 0 against the CPU oracle (the checker, not the timed thing) ----
    if not args.light:
        r0 = cell["reps"][0]
        cell["step"][0]()
        got = cell["outs"][0]
        nseq = min(B_loc, 8)  # sampled sequences at the full size (the C twin takes ~5 ms per MB)
        rows = sorted({(i * B_loc) // nseq for i in range(nseq)})
        rep = oracle_check(r0["q"], r0["kq"], r0["vq"], got, seq_lens=seq_lens, rows=rows)
        rep["sequences_checked"] = [b_lo + i for i in rows]
        rep["ok"] = cx.all_ok(rep["ok"])
        parity["headline_copy0"] = rep
        if not rep["ok"]:
            raise RuntimeError(f"parity against the oracle failed: {rep}")

    # ---- the headline: K steps, `samples` times ----
    st = cx.time_steps(cell["step"])
    ms = st["median_ms"]
    value = total_bytes * K / (ms * 1e-3) / 1e9
    nslots = (cell["ws"].get("key") or (0, 0, 1, 0))[2]
    launches_per_step = 1 if cell["ws"].get("key") is None else 2

    # ---- roofline of the dominant kernel: the split kernel alone, same geometry ----
    st_split = cx.time_steps(cell["split"])
    roofline = None
    if rank == 0:
        achieved = cbytes * K / (st_split["median_ms"] * 1e-3) / 1e9
        ratio = NCU_TRAFFIC_RATIO.get((name, nbits))
        roofline = {"bound": "hbm", "achieved": achieved, "peak": cx.peak, "unit": "GB/s",
                    "frac": achieved / cx.peak,
                    "traffic": None if ratio is None else int(ratio * cbytes),
                    "peak_source": cx.peak_src, "kernel": "splitk_kernel<FusedPolicy>",
                    "algorithmic_bytes_per_launch": cbytes,
                    "us_per_launch": us(st_split, K), "iqr_frac": st_split["iqr_frac_of_median"],
                    "frac_of_8TBps_spec": achieved / 8000.0,
                    "step_frac": cbytes * K / (ms * 1e-3) / 1e9 / cx.peak}

    # ---- same shape: fused hot, fp16 control cold and hot, the 2-bit cell ----
    extras = {}
    if not args.no_extras:
        hot = cx.time_steps(cell["step"][:1])
        extras["fused_cold_us"] = us(st, K)
        extras["fused_hot_us"] = us(hot, K)
        if cell["ctl"]:
            c_cold = cx.time_steps(cell["ctl"])
            c_hot = cx.time_steps(cell["ctl"][:1])
            extras.update({"fp16_cold_us": us(c_cold, K), "fp16_hot_us": us(c_hot, K),
                           "fp16_cold_GBps": cell["bytes16"] * K / (c_cold["median_ms"] * 1e-3) / 1e9,
                           "fp16_replicas": cell["R16"],
                           "speedup_cold": c_cold["median_ms"] / st["median_ms"],
                           "speedup_hot": c_hot["median_ms"] / hot["median_ms"],
                           "byte_ratio": cell["bytes16"] / cbytes})
        if nbits == 4 and name != "ragged-b16":
            c2 = fused_cell(cx, name, B_loc, S_loc, 2, seed, b_lo=b_lo)
            s2 = cx.time_steps(c2["step"])
            s2s = cx.time_steps(c2["split"])
            two = {"cold_us": us(s2, K), "split_kernel_us": us(s2s, K),
                   "GBps": c2["bytes"] * world * K / (s2["median_ms"] * 1e-3) / 1e9,
                   "split_frac_of_peak": c2["bytes"] * K / (s2s["median_ms"] * 1e-3) / 1e9 / cx.peak,
                   "iqr_frac": s2["iqr_frac_of_median"]}
            if "fp16_cold_us" in extras:
                two["speedup_cold_vs_fp16"] = extras["fp16_cold_us"] / two["cold_us"]
                two["byte_ratio"] = cell["bytes16"] / c2["bytes"]
            extras["two_bit"] = two
            del c2
            extras["per_channel_keys_2bit"] = per_channel_cell(cx, name, B_loc, S_loc, seed, b_lo, world)
            if rank == 0 and world == 1:
                torch.cuda.empty_cache()
                extras["write_side"] = write_side_record(cx, name, B_loc, S_loc, nbits)
        torch.cuda.empty_cache()
    cx.barrier()

    # ---- end to end through the public Python API with host buffers ----
    e2e = None
    if not args.light:
        e2e = e2e_leg(cx, name, B_loc, HQ, D, nbits, seed, b_lo, S_loc, seq_lens, valid_frac, total_bytes)

    # ---- the long single-sequence history split over the same ranks ----
    hist = None
    if not args.no_extras and name == "llama8b-b64":
        del cell
        torch.cuda.empty_cache()
        hist = history_split_record(cx, args.seed + 5)

    # ---- single-sequence sweep (rank 0, one GPU): hot and cold, fused 4/2-bit vs fp16 control ----
    rows = []
    if rank == 0 and world == 1 and not args.no_table and name in ("llama8b-b64", "qwen-b1"):
        rows = sweep_rows(cx, (2048, 8192, 16384, 65536), args.seed)

    # ---- the reference's Triton kernels, JIT-compiled on this GPU (rank 0, one GPU) ----
    triton = None
    if rank == 0 and world == 1 and not args.light and not args.no_table:
        torch.cuda.empty_cache()
        cells = [{"B": B_loc, "HQ": HQ, "HKV": HKV, "S": S_loc, "D": D, "nbits": [4, 2], "gs": GS,
                  "dist": WORKLOADS[name][6]}] if name == "llama8b-b64" else []
        qB, qHQ, qHKV, qD = WORKLOADS["qwen-b1"][:4]
        cells += [{"B": qB, "HQ": qHQ, "HKV": qHKV, "S": c, "D": qD, "nbits": [4, 2], "gs": GS,
                   "dist": "channel"} for c in sorted({r["ctx"] for r in rows})]
        tr, why = triton_rows(cells)
        triton = {"rows": tr, "unavailable": why,
                  "what": "the reference's fused_decode_attention / fp16_decode_attention (Triton, JIT on "
                          "this GPU) under the same hot / cold graph protocol, in a separate process"}
        for t in tr or []:  # next to our own numbers of the same cell
            for r in rows:
                if (r["ctx"], qB, qHQ) == (t["S"], t["B"], t["HQ"]):
                    r["triton_fused_cold_us"] = t.get(f"triton_fused_{r['nbits']}b_cold_us")
                    r["triton_fused_hot_us"] = t.get(f"triton_fused_{r['nbits']}b_hot_us")
                    r["triton_fp16_cold_us"] = t.get("triton_fp16_cold_us")
                    r["triton_fp16_hot_us"] = t.get("triton_fp16_hot_us")
            if name == "llama8b-b64" and (t["B"], t["S"], t["HQ"]) == (B_loc, S_loc, HQ) and extras:
                extras["triton_fused_cold_us"] = t.get(f"triton_fused_{nbits}b_cold_us")
                extras["triton_fused_2bit_cold_us"] = t.get("triton_fused_2b_cold_us")
                extras["triton_fp16_cold_us"] = t.get("triton_fp16_cold_us")

    clocks = sampler.stop()

    # ---- CPU baseline on this box's host cores (rank 0, single GPU only) ----
    cpu = None
    if rank == 0 and world == 1 and not args.light:
        r0 = fused_cell_host_copy(cx, name, B_loc, S_loc, nbits, seed)
        gbs, dt, cinfo = time_cpu(*r0, S_loc, D, nbits, steps=10, warmup=2, budget_s=20.0)
        cpu = {"value": gbs, "unit": "GB/s", **cinfo}

    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": world, "steps": K,
            "warmup": W, "ms_per_step": ms / K, "higher_is_better": True, "scaling": scaling,
            "vs_baseline": None, "dtype": "f16 operands / f32 accumulate", "data": "synthetic",
            "config": config,
            "run": {
                "per_gpu": f"B={B_loc} ctx={S_loc}",
                "regime": f"cold: inputs larger than L2 ({R} distinct caches, "
                          f"{R * cbytes / 1e6:.0f} MB >= 3 x {cx.l2 / 1e6:.0f} MB L2), CUDA-graph replay",
                "timing": f"median of {cx.samples} timed regions of {K} steps each (CUDA events, barrier + "
                          f"synchronize around every region, max over ranks)",
                "iqr_frac": st["iqr_frac_of_median"], "min_ms_per_step": st["min_ms"] / K,
                "max_ms_per_step": st["max_ms"] / K,
                "partial_slots_per_head": nslots,
                "untimed_steps_before_timing": K + W,
            },
            "roofline": roofline, "cpu_baseline": cpu, "e2e": e2e,
            "gpu_launches": launches_per_step * K, "clocks": clocks, "parity_vs_oracle": parity,
            "same_shape": extras, "history_split": hist, "rows": rows, "reference_triton": triton,
        }
        print(json.dumps(line), flush=True)
    teardown(cx)


def fused_cell_host_copy(cx, name, B, S, nbits, seed):
    """Host copy of cache 0 of the workload (the values ``device_replicas`` put on the GPU),
    quantised by the oracle: the CPU baseline's input."""
    return host_quantized(name, B, S, nbits, seed)


def e2e_leg(cx, name, B, HQ, D, nbits, seed, b_lo, S, seq_lens, valid_frac, total_bytes):
    """The same metric through the public Python API with host buffers: per step ``q`` pinned
    host -> device, the call, ``out`` device -> pinned host, stream synchronise.  The KV cache
    is the op's resident state (like weights) and is not copied per step."""
    torch, h = cx.torch, cx.harness
    from tritonkv_b200 import GraphedDecodeStep
    from tritonkv_b200.kernels import fused_decode_attention

    cell = fused_cell(cx, name, B, S, nbits, seed, b_lo=b_lo, seq_lens=seq_lens, valid_frac=valid_frac)
    reps, R, ws = cell["reps"], cell["R"], cell["ws"]
    out_dev = cell["outs"][0]
    K_e2e = min(cx.K, 500)
    q_host = [r["q"].cpu().pin_memory() for r in reps]
    q_dev = torch.empty_like(reps[0]["q"])
    out_host = torch.empty(B, HQ, D, dtype=torch.float32).pin_memory()
    stream = torch.cuda.current_stream()

    def direct(n):
        for i in range(n):
            r = reps[i % R]
            q_dev.copy_(q_host[i % R], non_blocking=True)
            fused_decode_attention(q_dev, r["kq"], r["vq"], out=out_dev, _workspace=ws, seq_lens=seq_lens)
            out_host.copy_(out_dev, non_blocking=True)
            stream.synchronize()  # the host reads this step's result before the next one

    direct(min(50, K_e2e))
    n_s = min(cx.samples, 10)
    ms_direct = h.stats([cx.max_over_ranks(h.time_region(lambda: direct(K_e2e), cx.barrier))
                         for _ in range(n_s)])["median_ms"]
    # The same step as a serving loop would run it: the two copies and the two kernels captured
    # once per cache (tritonkv_b200.GraphedDecodeStep), one graph launch per step.
    gsteps = [GraphedDecodeStep(r["kq"], r["vq"], HQ, q_dtype=r["q"].dtype, seq_lens=seq_lens) for r in reps]
    for g, qh in zip(gsteps, q_host):
        g.q_host.copy_(qh)

    def graphed(n):
        for i in range(n):
            g = gsteps[i % R]
            g.run()
            g.result()

    graphed(min(50, K_e2e))
    q_dev.copy_(q_host[0])
    fused_decode_attention(q_dev, reps[0]["kq"], reps[0]["vq"], out=out_dev, _workspace=ws, seq_lens=seq_lens)
    gsteps[0].run(q_host[0])
    if not torch.equal(gsteps[0].result(), out_dev.cpu()):
        raise RuntimeError("graphed step and direct call disagree")
    ms_graphed = h.stats([cx.max_over_ranks(h.time_region(lambda: graphed(K_e2e), cx.barrier))
                          for _ in range(n_s)])["median_ms"]
    # The same graph without the copy nodes: the last kernel writes out to the pinned host
    # buffer itself (GraphedDecodeStep(zero_copy=True)); the bytes that cross the bus per step
    # are the same.
    zsteps = [GraphedDecodeStep(r["kq"], r["vq"], HQ, q_dtype=r["q"].dtype, seq_lens=seq_lens,
                                zero_copy=True) for r in reps]
    for g, qh in zip(zsteps, q_host):
        g.q_host.copy_(qh)

    def zero_copy(n):
        for i in range(n):
            g = zsteps[i % R]
            g.run()
            g.result()

    zero_copy(min(50, K_e2e))
    zsteps[0].run(q_host[0])
    if not torch.equal(zsteps[0].result(), out_dev.cpu()):
        raise RuntimeError("zero-copy step and direct call disagree")
    ms_zero = h.stats([cx.max_over_ranks(h.time_region(lambda: zero_copy(K_e2e), cx.barrier))
                       for _ in range(n_s)])["median_ms"]
    ms_e2e = min(ms_graphed, ms_direct, ms_zero)
    path = {ms_graphed: "graphed", ms_direct: "direct", ms_zero: "graphed, zero-copy"}[ms_e2e]
    return {"value": total_bytes * K_e2e / (ms_e2e * 1e-3) / 1e9, "unit": "GB/s",
            "h2d_bytes_per_step": int(q_dev.numel() * q_dev.element_size()),
            "d2h_bytes_per_step": int(out_host.numel() * 4), "steps": K_e2e,
            "us_per_step": ms_e2e * 1e3 / K_e2e,
            "path": path,
            "graphed_us_per_step": ms_graphed * 1e3 / K_e2e,
            "zero_copy_us_per_step": ms_zero * 1e3 / K_e2e,
            "direct_call_us_per_step": ms_direct * 1e3 / K_e2e,
            "note": "per step: q pinned-host->device, fused_decode_attention (split + combine), "
                    "out device->pinned-host, stream sync; the KV cache is resident state. "
                    "graphed: tritonkv_b200.GraphedDecodeStep (the copies and kernels captured as "
                    "one CUDA graph, one launch per step); zero-copy: the same graph without the device-to-host copy node, "
                    "the last kernel writes out to pinned host memory itself; direct: the "
                    f"four host calls issued one by one; value = the fastest; median of {n_s} regions"}


def teardown(cx):
    if cx.dist is None:
        return
    # Graphs that hold captured NCCL kernels and the peer mappings are gone by now (the
    # legs close what they open).  A watchdog ends the process with a failure code if the
    # teardown itself blocks; the result line is already out.
    import gc
    import threading

    threading.Timer(60.0, lambda: os._exit(3)).start()
    gc.collect()
    cx.torch.cuda.synchronize()
    cx.dist.barrier()
    cx.dist.destroy_process_group()
    sys.stdout.flush()
    os._exit(0)


def sweep_rows(cx, contexts, seed, nbits_list=(4, 2), name="qwen-b1"):
    """Single-sequence sweep: nbits x contexts, fused vs the same-split fp16 control, hot (one
    cache, graph of 50 calls) and cold (one graph with one call per distinct cache), median
    and IQR over >= 30 replays (the reference's protocol, benchmark.py:556-728)."""
    torch, h = cx.torch, cx.harness
    from tritonkv_b200.kernels import fp16_decode_attention as fp16
    from tritonkv_b200.kernels import fused_decode_attention as fused

    B, HQ, HKV, D = WORKLOADS[name][:4]
    rows = []
    for ctx in contexts:
        b16 = fp16_bytes(B, HKV, ctx, D)
        R16 = max(2, h.replicas_for(b16, cx.l2))
        per = {}
        for nbits in nbits_list:
            bq = fused_bytes(B, HKV, ctx, D, nbits)
            Rq = max(2, h.replicas_for(bq, cx.l2))
            first = nbits == nbits_list[0]
            reps = device_replicas(cx, name, B, ctx, nbits, Rq, R16 if first else 0, seed + 7)
            outs = [torch.empty(B, HQ, D, device=cx.device) for _ in range(max(Rq, R16))]
            ws: dict = {}
            fq = [(lambda r=r, o=o: fused(r["q"], r["kq"], r["vq"], out=o, _workspace=ws))
                  for r, o in zip(reps[:Rq], outs)]
            hot = h.stats(h.bench_graph(fq[0]))
            cold = h.stats(h.bench_graph_rotating(fq))
            per[nbits] = (hot, cold, bq, Rq)
            if first:
                ws16: dict = {}
                f16 = [(lambda r=r, o=o: fp16(r["q"], r["k"], r["v"], out=o, _workspace=ws16))
                       for r, o in zip(reps[:R16], outs)]
                hot16 = h.stats(h.bench_graph(f16[0]))
                cold16 = h.stats(h.bench_graph_rotating(f16))
            del reps
        for nbits in nbits_list:
            hot, cold, bq, Rq = per[nbits]
            rows.append({
                "ctx": ctx, "nbits": nbits,
                "fused_hot_us": hot["median_ms"] * 1e3, "fused_cold_us": cold["median_ms"] * 1e3,
                "fp16_hot_us": hot16["median_ms"] * 1e3, "fp16_cold_us": cold16["median_ms"] * 1e3,
                "fused_cold_GBps": bq / cold["median_ms"] / 1e6,
                "fp16_cold_GBps": b16 / cold16["median_ms"] / 1e6,
                "fused_cold_frac_of_peak": bq / cold["median_ms"] / 1e6 / cx.peak,
                "speedup_cold": cold16["median_ms"] / cold["median_ms"],
                "speedup_hot": hot16["median_ms"] / hot["median_ms"],
                "cold_iqr_frac": cold["iqr_frac_of_median"], "hot_iqr_frac": hot["iqr_frac_of_median"],
                "replicas": Rq, "footprint_over_l2": Rq * bq / cx.l2,
                "fp16_cache_over_l2": b16 / cx.l2,
            })
        torch.cuda.empty_cache()
    return rows


def triton_rows(cells, timeout_s=900):
    """The reference's own Triton kernels on this GPU, timed by ``baseline/triton_leg.py`` in a
    separate process (it imports the reference's modules from the git-ignored
    ``baseline/_ref``, placed there by ``baseline/fetch_ref.py``; this process never imports
    them).  Returns (rows, reason): rows is None with a reason when the leg cannot run."""
    import subprocess

    leg = os.path.join(ROOT, "baseline", "triton_leg.py")
    if not os.path.isdir(os.path.join(ROOT, "baseline", "_ref")):
        return None, "baseline/_ref is absent: the reference's modules were not placed on this box"
    try:
        r = subprocess.run([sys.executable, leg, json.dumps(cells)], capture_output=True, text=True,
                           timeout=timeout_s)
    except subprocess.TimeoutExpired:
        return None, f"the Triton leg did not finish in {timeout_s} s"
    if r.returncode != 0:
        return None, "the Triton leg failed: " + r.stderr.strip().splitlines()[-1][:300] if r.stderr.strip() else "the Triton leg failed"
    try:
        res = json.loads(r.stdout.strip().splitlines()[-1])
    except Exception as exc:
        return None, f"unreadable output of the Triton leg: {exc!r}"
    if isinstance(res, dict):
        return None, res.get("unavailable", "unavailable")
    return res, None


L2_SWEEP_FACTORS = (0.125, 0.25, 0.5, 1.0, 2.0, 4.0, 8.0, 12.0)


def l2_sweep_contexts(l2_bytes, HKV, D, factors=L2_SWEEP_FACTORS):
    """Contexts that put the fp16 cache of ONE sequence at ``factor`` x the L2 size (a multiple
    of 256 tokens), the placement rule of the reference's long-context sweep
    (l2_sweep.py:196-304, docs/preregistration_l2.md:36-38)."""
    out = []
    for f in factors:
        ctx = int(f * l2_bytes / (4 * D * HKV))
        out.append(max(256, (ctx // 256) * 256))
    return out


def run_l2_sweep(cx):
    """``--workload l2-sweep``: fused 4-bit vs the fp16 control, hot and cold, at contexts that
    place the fp16 cache from 0.125x to 12x the L2 size read from the device."""
    args = cx.args
    name = "qwen-b1"
    B, HQ, HKV, D = WORKLOADS[name][:4]
    sampler = cx.harness.ClockSampler(cx.local).start()
    contexts = l2_sweep_contexts(cx.l2, HKV, D)
    rows = sweep_rows(cx, contexts, args.seed, nbits_list=(args.nbits or 4,)) if cx.rank == 0 else []
    clocks = sampler.stop()
    if cx.rank == 0:
        head = rows[-1]
        line = {"metric": METRIC, "value": head["fused_cold_GBps"], "unit": "GB/s", "n_gpus": cx.world,
                "steps": head["replicas"], "warmup": 3, "ms_per_step": head["fused_cold_us"] / 1e3,
                "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
                "dtype": "f16 operands / f32 accumulate", "data": "synthetic",
                "config": {"workload": f"l2-sweep: {WORKLOADS['l2-sweep'][7]}; headline = the longest context "
                                       f"(ctx {head['ctx']}, fp16 cache {head['fp16_cache_over_l2']:.1f} x L2)",
                           "partition": "rank 0 only"},
                "l2_bytes": cx.l2, "l2_sweep": rows, "clocks": clocks, "roofline": None,
                "cpu_baseline": None, "e2e": None, "gpu_launches": 2 * head["replicas"]}
        print(json.dumps(line), flush=True)
    teardown(cx)


def main():
    args = parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
