"""Time the reference's own Triton kernels on this GPU (a separate process started by
``bench.py``; nothing else imports this file, and it imports nothing of ``tritonkv_b200``).

    python baseline/triton_leg.py '<json list of cells>'

Each cell is ``{"B", "HQ", "HKV", "S", "D", "nbits": [..], "gs", "dist"}``; for each the script
quantises seeded caches with the reference's ``quantize_kv``, JIT-compiles its
``fused_decode_attention`` and ``fp16_decode_attention`` (``baseline/_ref``, placed by
``baseline/fetch_ref.py``) and times them under the reference's two protocols: hot (one
cache, a CUDA graph of 50 back-to-back calls) and cold (one graph with one call per
distinct cache, working set >= 3x L2), median over >= 30 replays (benchmark.py:556-728 of
the reference).  Prints one JSON list.  No kernel or helper of this repository runs here.
"""

from __future__ import annotations

import json
import os
import statistics
import sys
import time

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.path.join(HERE, "_ref")


def replicas_for(nbytes, l2, factor=3.0, cap_bytes=16 << 30):
    want = -(-int(factor * l2) // nbytes)
    return int(max(2, min(4096, want, max(1, cap_bytes // nbytes))))


def main():
    cells = json.loads(sys.argv[1])
    if not os.path.isdir(REF):
        print(json.dumps({"unavailable": "baseline/_ref is absent (run baseline/fetch_ref.py)"}))
        return
    sys.dont_write_bytecode = True
    sys.path.insert(0, REF)
    import torch
    import quantize as rq
    from kernels import fp16_decode_attention, fused_decode_attention, triton_available

    ok, why = triton_available()
    if not ok:
        print(json.dumps({"unavailable": f"reference reports Triton unusable: {why}"}))
        return
    dev = torch.device("cuda")
    l2 = torch.cuda.get_device_properties(dev).L2_cache_size

    def capture(fns, repeat):
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

    def sample(g, calls, samples=30, min_s=0.1, max_s=6.0):
        for _ in range(3):
            g.replay()
        torch.cuda.synchronize()
        xs, t0 = [], time.time()
        while True:
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            g.replay()
            e.record()
            e.synchronize()
            xs.append(s.elapsed_time(e) / calls)
            el = time.time() - t0
            if len(xs) >= samples and (el >= min_s or el >= max_s):
                return statistics.median(xs) * 1e3  # us

    out = []
    for c in cells:
        B, HQ, HKV, S, D, gs = (c[k] for k in ("B", "HQ", "HKV", "S", "D", "gs"))
        b16 = B * HKV * S * 4 * D
        R16 = replicas_for(b16, l2)
        row = dict(c)
        for j, nbits in enumerate(c["nbits"]):
            bq = B * HKV * S * (2 * D * nbits // 8 + 8 * (D // gs))
            Rq = replicas_for(bq, l2)
            n16 = R16 if j == 0 else 0  # the control is timed once per shape
            reps = []
            for i in range(max(Rq, n16)):
                g = torch.Generator(device=dev).manual_seed(1000 + i)
                q = torch.randn(B, HQ, D, generator=g, device=dev).half()
                k = torch.randn(B, HKV, S, D, generator=g, device=dev)
                if c.get("dist") == "channel":
                    k *= torch.exp(0.5 * torch.randn(HKV, D, generator=g, device=dev))[None, :, None, :]
                k = k.half()
                v = torch.randn(B, HKV, S, D, generator=g, device=dev).half()
                r = {"q": q}
                if i < Rq:
                    r["kq"], r["vq"] = rq.quantize_kv(k, v, nbits, gs)
                if i < n16:
                    r["k"], r["v"] = k, v
                reps.append(r)
                del k, v
            outs = [torch.empty(B, HQ, D, device=dev) for _ in range(max(Rq, n16))]
            ws, ws16 = {}, {}
            fq = [(lambda r=r, o=o: fused_decode_attention(r["q"], r["kq"], r["vq"], out=o, _workspace=ws))
                  for r, o in zip(reps[:Rq], outs)]
            row[f"triton_fused_{nbits}b_hot_us"] = sample(capture(fq[:1], 50), 50)
            row[f"triton_fused_{nbits}b_cold_us"] = sample(capture(fq, 1), len(fq))
            if n16:
                f16 = [(lambda r=r, o=o: fp16_decode_attention(r["q"], r["k"], r["v"], out=o, _workspace=ws16))
                       for r, o in zip(reps[:n16], outs)]
                row["triton_fp16_hot_us"] = sample(capture(f16[:1], 50), 50)
                row["triton_fp16_cold_us"] = sample(capture(f16, 1), len(f16))
                del f16
            del reps, outs, fq
            torch.cuda.empty_cache()
        out.append(row)
    print(json.dumps(out))


if __name__ == "__main__":
    main()
