"""Generate the golden fixtures in this directory from the reference project.

Run once, in a container where the reference checkout is available:

    TRITON_INTERPRET=1 python tests/golden/make_golden.py /path/to/reference

It imports the reference's ``quantize.py`` / ``reference.py`` unmodified (CPU
tensors) and, through Triton's CPU interpreter, launches the reference's own
``_fused_decode_attn_split`` / ``_combine_splits`` / ``_fp16_decode_attn_split``
kernels on tiny inputs, then stores inputs and outputs as ``.npz`` files.  The
fixtures travel with the repository; the reference does not have to.

Nothing in the library, the tests or the benchmark imports this script.
"""

from __future__ import annotations

import math
import os
import sys

os.environ.setdefault("TRITON_INTERPRET", "1")

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def all_f16_patterns(order: str, seed: int = 5) -> np.ndarray:
    """All 65536 fp16 bit patterns as a (1, 2, 256, 128) tensor: ``sorted`` (finite values in
    ascending order, then the non-finite ones: a group holds neighbouring values),
    ``shuffled``, or ``finite_shuffled`` (non-finite patterns replaced by repeats).  -0 is
    replaced by +0: which zero a minimum over {-0, +0} returns is not something to pin."""
    bits = np.arange(65536, dtype=np.uint16)
    bits[0x8000] = 0
    vals = bits.view(np.float16)
    if order == "sorted":
        finite = vals[np.isfinite(vals)]
        finite = finite[np.argsort(finite.astype(np.float32), kind="stable")]
        vals = np.concatenate([finite, vals[~np.isfinite(vals)]])
    else:
        if order == "finite_shuffled":
            vals = vals[np.isfinite(vals)]
            vals = np.concatenate([vals, vals[: 65536 - len(vals)]])
        vals = np.random.default_rng(seed).permutation(vals)
    return np.ascontiguousarray(vals.reshape(1, 2, 256, 128))


def main(ref_root: str) -> None:
    sys.dont_write_bytecode = True
    sys.path.insert(0, ref_root)
    import quantize as rq
    import reference as rr

    torch.manual_seed(0)
    out: dict[str, np.ndarray] = {}

    # ---- 1. split-P packing ------------------------------------------------
    out["pack4_known_codes"] = np.arange(1, 9, dtype=np.uint8)
    out["pack4_known_packed"] = rq.pack_codes(torch.arange(1, 9, dtype=torch.uint8), 4).numpy()
    c2 = torch.tensor([0, 1, 2, 3, 0, 1, 2, 3], dtype=torch.uint8)
    out["pack2_known_codes"] = c2.numpy()
    out["pack2_known_packed"] = rq.pack_codes(c2, 2).numpy()
    g = torch.Generator().manual_seed(1234)
    for nbits in (2, 4):
        for D in (64, 128):
            codes = torch.randint(0, 1 << nbits, (3, 5, D), dtype=torch.uint8, generator=g)
            packed = rq.pack_codes(codes, nbits)
            assert torch.equal(rq.unpack_codes(packed, nbits, D), codes)
            out[f"pack_codes_n{nbits}_d{D}"] = codes.numpy()
            out[f"pack_packed_n{nbits}_d{D}"] = packed.numpy()
    np.savez_compressed(os.path.join(HERE, "pack.npz"), **out)

    # ---- 2. quantiser ------------------------------------------------------
    out = {}
    g = torch.Generator().manual_seed(4321)
    x = torch.randn(48, 128, generator=g)
    m = torch.rand(48, 128, generator=g) < 0.02
    x = torch.where(m, x * 8.0, x)
    x[3, :32] = 3.5            # constant group
    x[4, 32:64] = 0.0          # constant zero group
    x[5, :] *= 1e-3            # small range
    x[6, :] *= 300.0           # large range
    x[7, 64:96] = torch.linspace(-1, 1, 32)      # exact half-way candidates
    x[8, :32] = torch.arange(32) * 0.5            # ties (x.5 codes)
    cases = {"f32": x, "f16": x.half(), "bf16": x.bfloat16()}
    for name, xin in cases.items():
        out[f"x_{name}"] = (xin.view(torch.int16).numpy() if xin.dtype == torch.bfloat16
                            else xin.numpy())
        for nbits in (2, 4):
            for gs in (16, 32, 64, 128):
                qt = rq.quantize_groupwise(xin, nbits, gs)
                key = f"{name}_n{nbits}_g{gs}"
                out[f"packed_{key}"] = qt.packed.numpy()
                out[f"scale_{key}"] = qt.scale.numpy()
                out[f"zero_{key}"] = qt.zero.numpy()
                if name == "f16":
                    out[f"deq_{key}"] = rq.dequantize_groupwise(qt, torch.float32).numpy()
    x64 = torch.randn(16, 64, generator=g).half()
    out["x64_f16"] = x64.numpy()
    for nbits in (2, 4):
        for gs in (16, 32, 64):
            qt = rq.quantize_groupwise(x64, nbits, gs)
            key = f"d64_n{nbits}_g{gs}"
            out[f"packed_{key}"] = qt.packed.numpy()
            out[f"scale_{key}"] = qt.scale.numpy()
            out[f"zero_{key}"] = qt.zero.numpy()
    np.savez_compressed(os.path.join(HERE, "quantize.npz"), **out)

    # ---- 2b. quantiser edges the reference's own tests do not pin --------
    # group ranges that underflow fp16 (scale rounds to a subnormal or to 0, codes
    # collapse to {0, qmax}), a constant group, +inf / -inf / NaN inside a group
    out = {}
    g = torch.Generator().manual_seed(99)
    xe = torch.zeros(6, 128)
    xe[0] = torch.randn(128, generator=g) * 1e-7
    xe[1] = 1.0 + torch.randn(128, generator=g) * 1e-8
    xe[2] = torch.randn(128, generator=g)
    xe[2, 5] = float("inf")
    xe[3] = torch.randn(128, generator=g)
    xe[3, 40] = float("-inf")
    xe[4] = torch.randn(128, generator=g)
    xe[4, 70] = float("nan")
    xe[5] = torch.randn(128, generator=g) * 1e-5
    out["x_edges"] = xe.numpy()
    for nbits in (2, 4):
        for gs in (32, 128):
            qt = rq.quantize_groupwise(xe, nbits, gs)
            key = f"edges_n{nbits}_g{gs}"
            out[f"packed_{key}"] = qt.packed.numpy()
            out[f"scale_{key}"] = qt.scale.numpy()
            out[f"zero_{key}"] = qt.zero.numpy()
    np.savez_compressed(os.path.join(HERE, "quantize_edges.npz"), **out)

    # ---- 2c. every fp16 bit pattern through the reference's quantiser ------
    # (what the CUDA quantiser's reciprocal-with-redo arithmetic has to reproduce bit for bit:
    # exact ties, ranges that underflow fp16, infinities and NaNs in every position)
    out = {}
    for order in ("sorted", "shuffled", "finite_shuffled"):
        x16 = all_f16_patterns(order)
        out[f"x_{order}"] = x16.view(np.uint16)
        xt = torch.from_numpy(x16)
        for nbits in (2, 4):
            for gs in (8, 32):
                qt = rq.quantize_groupwise(xt, nbits, gs)
                key = f"{order}_n{nbits}_g{gs}"
                out[f"packed_{key}"] = qt.packed.numpy()
                out[f"scale_{key}"] = qt.scale.numpy().view(np.uint16)
                out[f"zero_{key}"] = qt.zero.numpy().view(np.uint16)
    np.savez_compressed(os.path.join(HERE, "quantize_allbits.npz"), **out)

    # ---- 3. attention ground truth ----------------------------------------
    out = {}
    att_cases = [
        # name, B, HQ, HKV, S, D, nbits, gs, seed, outlier_frac
        ("cfg1", 1, 12, 2, 512, 128, 4, 32, 0, 0.0),
        ("qwen_s17_2b", 1, 12, 2, 17, 128, 2, 32, 1, 0.01),
        ("mha_d64", 1, 8, 8, 96, 64, 4, 32, 2, 0.01),
        ("llama_b2_d64_g64", 2, 32, 8, 80, 64, 4, 64, 3, 0.01),
        ("gqa8_g128_2b", 1, 8, 1, 130, 128, 2, 128, 4, 0.01),
        ("gqa4_g16", 2, 8, 2, 33, 128, 4, 16, 5, 0.01),
    ]
    for name, B, HQ, HKV, S, D, nbits, gs, seed, of in att_cases:
        q, k, v = rr.make_random_kv(B, HQ, HKV, S, D, device="cpu", seed=seed, outlier_frac=of)
        kq, vq = rq.quantize_kv(k, v, nbits, gs)
        kd = rq.dequantize_groupwise(kq, torch.float32)
        vd = rq.dequantize_groupwise(vq, torch.float32)
        ref = rr.reference_decode_attention(q, kd, vd)
        out[f"{name}_meta"] = np.array([B, HQ, HKV, S, D, nbits, gs, seed], dtype=np.int64)
        out[f"{name}_q"] = q.numpy()
        for t, qt in (("k", kq), ("v", vq)):
            out[f"{name}_{t}packed"] = qt.packed.numpy()
            out[f"{name}_{t}scale"] = qt.scale.numpy()
            out[f"{name}_{t}zero"] = qt.zero.numpy()
        out[f"{name}_out"] = ref.numpy()
        if name in ("qwen_s17_2b", "mha_d64"):
            out[f"{name}_k16"] = k.numpy()
            out[f"{name}_v16"] = v.numpy()
            out[f"{name}_out_fp16cache"] = rr.reference_decode_attention(q, k, v).numpy()
    np.savez_compressed(os.path.join(HERE, "attention.npz"), **out)

    # ---- 4. the reference's own Triton kernels under the CPU interpreter ---
    out = {}
    try:
        import triton
        from kernels import fused_decode_attn as rk
        from kernels import fp16_decode_attn as rf

        def launch_fused(q, kq, vq, block_n, num_splits):
            B, HQ, D = q.shape
            _, HKV, S, DP = kq.packed.shape
            group = HQ // HKV
            sm_scale = 1.0 / math.sqrt(D)
            block_n = min(block_n, max(16, rk._next_pow2(S)))
            n_blocks = triton.cdiv(S, block_n)
            num_splits = max(1, min(num_splits, n_blocks))
            bps = triton.cdiv(n_blocks, num_splits)
            num_splits = triton.cdiv(n_blocks, bps)
            split_size = bps * block_n
            o = torch.zeros((B, HQ, D), dtype=torch.float32)
            acc = torch.zeros((B, HQ, num_splits, D), dtype=torch.float32)
            maxs = torch.zeros((B, HQ, num_splits), dtype=torch.float32)
            sums = torch.zeros((B, HQ, num_splits), dtype=torch.float32)
            kp, ks, kz = kq.packed, kq.scale, kq.zero
            vp, vs, vz = vq.packed, vq.scale, vq.zero
            rk._fused_decode_attn_split[(B * HKV, num_splits)](
                q, kp, ks, kz, vp, vs, vz, acc, maxs, sums, o, sm_scale, S,
                q.stride(0), q.stride(1), q.stride(2),
                kp.stride(0), kp.stride(1), kp.stride(2), kp.stride(3),
                ks.stride(0), ks.stride(1), ks.stride(2), ks.stride(3),
                vp.stride(0), vp.stride(1), vp.stride(2), vp.stride(3),
                vs.stride(0), vs.stride(1), vs.stride(2), vs.stride(3),
                acc.stride(0), acc.stride(1), acc.stride(2), acc.stride(3),
                maxs.stride(0), maxs.stride(1), maxs.stride(2),
                o.stride(0), o.stride(1), o.stride(2),
                HKV=HKV, GROUP=group, D=D, DP=DP, NBITS=kq.nbits, GS=kq.group_size,
                NG=D // kq.group_size, BLOCK_H=max(16, rk._next_pow2(group)),
                BLOCK_N=block_n, SPLIT_SIZE=split_size, SINGLE_SPLIT=(num_splits == 1),
                BCAST_META=True, FOLD_ZP=False, DEQ_FP16=False,
            )
            if num_splits > 1:
                rk._combine_splits[(B * HQ,)](
                    acc, maxs, sums, o, num_splits,
                    acc.stride(0), acc.stride(1), acc.stride(2), acc.stride(3),
                    maxs.stride(0), maxs.stride(1), maxs.stride(2),
                    o.stride(0), o.stride(1), o.stride(2), HQ=HQ, D=D,
                )
            return o, acc, maxs, sums, num_splits, split_size

        for name, B, HQ, HKV, S, D, nbits, gs, seed, nsplit in [
            ("tk_qwen", 1, 12, 2, 80, 128, 4, 32, 11, 3),
            ("tk_2b_d64", 1, 8, 2, 48, 64, 2, 32, 12, 2),
        ]:
            q, k, v = rr.make_random_kv(B, HQ, HKV, S, D, device="cpu", seed=seed)
            kq, vq = rq.quantize_kv(k, v, nbits, gs)
            o, acc, maxs, sums, ns, ss = launch_fused(q, kq, vq, 16, nsplit)
            out[f"{name}_meta"] = np.array([B, HQ, HKV, S, D, nbits, gs, seed, ns, ss], np.int64)
            out[f"{name}_q"] = q.numpy()
            for t, qt in (("k", kq), ("v", vq)):
                out[f"{name}_{t}packed"] = qt.packed.numpy()
                out[f"{name}_{t}scale"] = qt.scale.numpy()
                out[f"{name}_{t}zero"] = qt.zero.numpy()
            out[f"{name}_out"] = o.numpy()
            out[f"{name}_acc"] = acc.numpy()
            out[f"{name}_maxs"] = maxs.numpy()
            out[f"{name}_sums"] = sums.numpy()
        out["triton_interpreter"] = np.array([1])
    except Exception as exc:  # interpreter unavailable: record why, keep the rest
        out["triton_interpreter"] = np.array([0])
        print(f"[make_golden] Triton CPU interpreter leg skipped: {exc!r}")
    np.savez_compressed(os.path.join(HERE, "triton_partials.npz"), **out)
    print("golden fixtures written to", HERE)


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: python tests/golden/make_golden.py <path to a checkout of the reference project>")
    main(sys.argv[1])
