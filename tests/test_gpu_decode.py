"""GPU parity of the decode kernels against the CPU oracle (dequantise in fp32, then
fp32 attention), through the C ABI.  The cases are the reference's kernel tests
(test_correctness.py:141-343) plus its audit checks (audit_claims.py:1905-2015),
with the elementwise bound |got-ref| <= 2e-3 + 1e-2*|ref| asserted next to the
reference's own cosine / rel-L2 thresholds."""

import os

import numpy as np
import pytest
import torch

from oracle import tkv_oracle as O
from tritonkv_b200 import quantize as Q
from tritonkv_b200.kernels import (combine_splits, fp16_decode_attention, fused_decode_attention,
                                   triton_available)
from oracle.workloads import make_random_kv, ragged_seq_lens

from util import ATOL, RTOL, assert_close, c_oracle_attention, oracle_attention, to_oracle

pytestmark = pytest.mark.gpu
DEV = "cuda"

SHAPES = [
    (1, 12, 2, 128),  # Qwen2.5-1.5B attention shape
    (1, 8, 8, 64),    # no GQA sharing (MHA)
    (2, 32, 8, 64),   # Llama-3.2-1B shape, batch 2
]
SEQ_LENS = [1, 17, 128, 512, 2048, 8192, 16384]


def _case(B, HQ, HKV, D, S, nbits, gs, seed, **kw):
    q, k, v = make_random_kv(B, HQ, HKV, S, D, device=DEV, seed=seed)
    kq, vq = Q.quantize_kv(k, v, nbits, gs)
    got = fused_decode_attention(q, kq, vq, **kw)
    return got, oracle_attention(q, kq, vq), (q, k, v, kq, vq)


def test_backend_reports_available():
    ok, why = triton_available()
    assert ok, why


@pytest.mark.parametrize("S", SEQ_LENS)
@pytest.mark.parametrize("seed", [0, 1, 2])
def test_kernel_matches_dequant_reference_4bit(S, seed):
    got, ref, _ = _case(1, 12, 2, 128, S, 4, 32, seed)
    assert_close(got, ref, f"S={S} seed={seed}")


@pytest.mark.parametrize("S", [512, 2048, 8192, 16384])
@pytest.mark.parametrize("seed", [0, 1])
def test_kernel_matches_dequant_reference_2bit(S, seed):
    got, ref, _ = _case(1, 12, 2, 128, S, 2, 32, seed)
    assert_close(got, ref, f"S={S} seed={seed}")


@pytest.mark.parametrize("shape", SHAPES)
@pytest.mark.parametrize("nbits", Q.SUPPORTED_BITS)
def test_kernel_shapes_and_gqa(shape, nbits):
    B, HQ, HKV, D = shape
    got, ref, _ = _case(B, HQ, HKV, D, 1024, nbits, 32, seed=3)
    assert_close(got, ref, f"{shape} {nbits}b")


@pytest.mark.parametrize("D,gs", [(128, 16), (128, 32), (128, 64), (128, 128), (64, 16), (64, 32),
                                  (64, 64)])
@pytest.mark.parametrize("nbits", Q.SUPPORTED_BITS)
def test_kernel_group_sizes(D, gs, nbits):
    got, ref, _ = _case(1, 12, 2, D, 2048, nbits, gs, seed=4)
    assert_close(got, ref, f"D={D} gs={gs} {nbits}b")


@pytest.mark.parametrize("HQ,HKV", [(8, 1), (32, 8), (64, 8), (4, 4), (24, 2), (9, 3)])
def test_gqa_group_sizes(HQ, HKV):
    """Groups of 1..12 query heads per KV head (12 spans two head chunks of a CTA)."""
    got, ref, _ = _case(2, HQ, HKV, 128, 777, 4, 32, seed=14)
    assert_close(got, ref, f"HQ/HKV={HQ}/{HKV}")


@pytest.mark.parametrize("num_splits", [1, 2, 5, 17, 64])
def test_split_count_does_not_change_the_answer(num_splits):
    got, ref, _ = _case(1, 12, 2, 128, 4096, 4, 32, seed=6, num_splits=num_splits)
    assert_close(got, ref, f"splits={num_splits}")


def test_split_counts_agree_with_each_other():
    """audit_claims.py:1962-1985: spread across split counts below 2% of mean |out|."""
    q, k, v = make_random_kv(1, 12, 2, 4096, 128, device=DEV, seed=21)
    kq, vq = Q.quantize_kv(k, v, 4, 32)
    outs = [fused_decode_attention(q, kq, vq, num_splits=n) for n in (1, 3, 8, 32)]
    stack = torch.stack(outs)
    spread = (stack.max(0).values - stack.min(0).values).max().item()
    assert spread < 0.02 * stack[0].abs().mean().item()


@pytest.mark.parametrize("block_n", [16, 32, 64, 128])
def test_block_sizes(block_n):
    got, ref, _ = _case(1, 12, 2, 128, 3000, 4, 32, seed=7, block_n=block_n)
    assert_close(got, ref, f"BLOCK_N={block_n}")


def test_output_is_finite_with_extreme_scores():
    q, k, v = make_random_kv(1, 12, 2, 2048, 128, device=DEV, seed=8)
    q = q * 50.0
    kq, vq = Q.quantize_kv(k, v, 4, 32)
    got = fused_decode_attention(q, kq, vq)
    assert torch.isfinite(got).all()
    rep = O.allclose_report(got.cpu().numpy(), oracle_attention(q, kq, vq))
    assert rep["cosine"] >= 0.99999 and rep["rel_l2"] <= 5e-3, rep


def test_single_token_cache():
    q, k, v = make_random_kv(1, 12, 2, 1, 128, device=DEV, seed=9)
    kq, vq = Q.quantize_kv(k, v, 4, 32)
    got = fused_decode_attention(q, kq, vq)
    v_deq = Q.dequantize_groupwise(vq, torch.float32)
    expect = v_deq[:, :, 0, :].repeat_interleave(6, dim=1)
    assert ((got - expect).norm() / expect.norm()).item() < 1e-3


def test_per_element_worst_case_not_hidden_by_aggregate():
    got, ref, _ = _case(1, 12, 2, 128, 8192, 4, 32, seed=10)
    err = np.abs(got.cpu().numpy() - ref)
    assert err.max() / max(np.abs(ref).mean(), 1e-6) < 0.05


def test_kernel_is_not_the_source_of_error():
    """Kernel error vs the unquantised cache no worse than 1.5x the error of
    dequantise-then-attend itself (test_correctness.py:202-217)."""
    for S in (512, 2048, 8192):
        got, ref_deq, (q, k, v, kq, vq) = _case(1, 12, 2, 128, S, 4, 32, seed=5)
        truth = O.reference_decode_attention(q.float().cpu().numpy(), k.float().cpu().numpy(),
                                             v.float().cpu().numpy())
        e_kernel = O.allclose_report(got.cpu().numpy(), truth)["rel_l2"]
        e_base = O.allclose_report(ref_deq, truth)["rel_l2"]
        assert e_kernel <= 1.5 * e_base, (S, e_kernel, e_base)


@pytest.mark.parametrize("S", [1, 17, 512, 2048])
@pytest.mark.parametrize("nbits", Q.SUPPORTED_BITS)
@pytest.mark.parametrize("gs", [16, 32, 64, 128])
def test_variant_flags_are_bitwise_identical(S, nbits, gs):
    """meta_bcast and dequant_fp16 must not change a single bit
    (test_correctness.py:292-343); fold_zp stays within tolerance."""
    q, k, v = make_random_kv(1, 12, 2, S, 128, device=DEV, seed=11)
    kq, vq = Q.quantize_kv(k, v, nbits, gs)
    base = fused_decode_attention(q, kq, vq)
    assert torch.equal(base, fused_decode_attention(q, kq, vq, meta_bcast=False))
    assert torch.equal(base, fused_decode_attention(q, kq, vq, dequant_fp16=True))
    assert torch.equal(base, fused_decode_attention(q, kq, vq, num_warps=8, num_stages=3))
    assert_close(fused_decode_attention(q, kq, vq, fold_zp=True), oracle_attention(q, kq, vq))


def test_heavy_outliers_and_peaked_softmax():
    """audit_claims.py:1905-2015: 5% of entries x20, and a query aligned with one key."""
    q, k, v = make_random_kv(1, 12, 2, 4096, 128, device=DEV, seed=31, outlier_frac=0.05,
                             outlier_scale=20.0)
    kq, vq = Q.quantize_kv(k, v, 4, 32)
    rep = O.allclose_report(fused_decode_attention(q, kq, vq).cpu().numpy(),
                            oracle_attention(q, kq, vq))
    assert rep["cosine"] >= 0.99999 and rep["rel_l2"] <= 5e-3, rep
    q2, k2, v2 = make_random_kv(1, 12, 2, 4096, 128, device=DEV, seed=32)
    q2[0, :, :] = k2[0, 0, 1234, :] * 3.0
    kq2, vq2 = Q.quantize_kv(k2, v2, 4, 32)
    rep = O.allclose_report(fused_decode_attention(q2, kq2, vq2).cpu().numpy(),
                            oracle_attention(q2, kq2, vq2))
    assert rep["rel_l2"] <= 5e-3, rep


@pytest.mark.parametrize("name", ["cfg1", "qwen_s17_2b", "mha_d64", "llama_b2_d64_g64",
                                  "gqa8_g128_2b", "gqa4_g16"])
def test_golden_attention_fixtures(golden_dir, name):
    """Inputs and outputs stored from the reference's own quantize.py/reference.py."""
    g = np.load(os.path.join(golden_dir, "attention.npz"))
    B, HQ, HKV, S, D, nbits, gs, seed = [int(x) for x in g[f"{name}_meta"]]
    def qt(t):
        return Q.QuantizedTensor(torch.from_numpy(g[f"{name}_{t}packed"]).to(DEV),
                                 torch.from_numpy(g[f"{name}_{t}scale"]).to(DEV),
                                 torch.from_numpy(g[f"{name}_{t}zero"]).to(DEV), nbits, gs, D)
    q = torch.from_numpy(g[f"{name}_q"]).to(DEV)
    got = fused_decode_attention(q, qt("k"), qt("v"))
    assert_close(got, g[f"{name}_out"], name)


@pytest.mark.parametrize("q_dtype", [torch.float16, torch.bfloat16, torch.float32])
def test_query_dtypes(q_dtype):
    q, k, v = make_random_kv(1, 12, 2, 1000, 128, device=DEV, seed=40)
    kq, vq = Q.quantize_kv(k, v, 4, 32)
    qq = q.to(q_dtype)
    got = fused_decode_attention(qq, kq, vq)
    # the kernel rounds q to fp16, as the reference does; compare on that value
    assert_close(got, oracle_attention(qq.to(torch.float16), kq, vq), str(q_dtype))


@pytest.mark.parametrize("nbits", [4, 2])
@pytest.mark.parametrize("k_first", [True, False])
@pytest.mark.parametrize("B,S", [(1, 4096), (16, 2048)])
def test_code_tensors_in_either_address_order(nbits, k_first, B, S):
    """The K and the V code tensor are fetched through ONE tensor map that spans both (the lower
    address first); whichever of the two lies higher, the result is the same bits."""
    HQ, HKV, D = 32, 8, 128
    q, k, v = make_random_kv(B, HQ, HKV, S, D, device=DEV, seed=91)
    kq, vq = Q.quantize_kv(k, v, nbits, 32)
    ref = fused_decode_attention(q, kq, vq)
    n = kq.packed.numel()
    buf = torch.empty(2 * n + 4096, dtype=torch.uint8, device=DEV)
    lo, hi = buf[:n].view(kq.packed.shape), buf[n + 4096:].view(kq.packed.shape)
    kp, vp = (lo, hi) if k_first else (hi, lo)
    kp.copy_(kq.packed)
    vp.copy_(vq.packed)
    assert (kp.data_ptr() < vp.data_ptr()) == k_first
    k2 = Q.QuantizedTensor(kp, kq.scale, kq.zero, nbits, 32, D)
    v2 = Q.QuantizedTensor(vp, vq.scale, vq.zero, nbits, 32, D)
    assert torch.equal(fused_decode_attention(q, k2, v2), ref)


def test_sm_scale_out_and_workspace_reuse():
    q, k, v = make_random_kv(2, 8, 2, 2048, 128, device=DEV, seed=41)
    kq, vq = Q.quantize_kv(k, v, 4, 32)
    out = torch.empty(2, 8, 128, device=DEV)
    ws = {}
    r = fused_decode_attention(q, kq, vq, sm_scale=0.05, out=out, _workspace=ws, num_splits=8)
    nslots = ws["key"][2]  # partial slots per head: num_splits x per-split CTA segments
    assert r is out and nslots % 8 == 0 and ws["key"] == (2, 8, nslots, 128)
    assert ws["acc"].shape == (2, 8, nslots, 128)
    acc_ptr = ws["acc"].data_ptr()
    assert_close(out, oracle_attention(q, kq, vq, sm_scale=0.05))
    fused_decode_attention(q, kq, vq, sm_scale=0.05, out=out, _workspace=ws, num_splits=8)
    assert ws["acc"].data_ptr() == acc_ptr  # no reallocation
    # the call is capturable and replayable once out and workspace exist
    g = torch.cuda.CUDAGraph()
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        fused_decode_attention(q, kq, vq, sm_scale=0.05, out=out, _workspace=ws, num_splits=8)
    torch.cuda.current_stream().wait_stream(s)
    with torch.cuda.graph(g):
        fused_decode_attention(q, kq, vq, sm_scale=0.05, out=out, _workspace=ws, num_splits=8)
    out.zero_()
    g.replay()
    torch.cuda.synchronize()
    assert_close(out, oracle_attention(q, kq, vq, sm_scale=0.05))


def test_argument_errors_match_reference():
    q, k, v = make_random_kv(1, 12, 2, 64, 128, device=DEV, seed=42)
    kq, vq = Q.quantize_kv(k, v, 4, 32)
    kq2, _ = Q.quantize_kv(k, v, 2, 32)
    with pytest.raises(ValueError, match="same nbits/group_size"):
        fused_decode_attention(q, kq2, vq)
    with pytest.raises(ValueError, match="incompatible with cache"):
        fused_decode_attention(q[:, :, :64].contiguous(), kq, vq)
    with pytest.raises(ValueError, match="multiple of HKV"):
        fused_decode_attention(q[:, :11].contiguous(), kq, vq)
    kq8 = Q.quantize_groupwise(k, 4, 8)
    with pytest.raises(ValueError, match="fold_zp needs group_size >= 16"):
        fused_decode_attention(q, kq8, kq8, fold_zp=True)
    with pytest.raises(ValueError, match="unsupported"):
        fused_decode_attention(q, kq8, kq8)
    with pytest.raises(RuntimeError, match="no CPU path"):
        fused_decode_attention(q.cpu(), kq, vq)
    # cache tensors the kernels would reinterpret silently: refused by dtype and by device
    f32meta = Q.QuantizedTensor(kq.packed, kq.scale.float(), kq.zero.float(), 4, 32, 128)
    with pytest.raises(TypeError, match="scale must be float16"):
        fused_decode_attention(q, f32meta, vq)
    with pytest.raises(TypeError, match="scale must be float16"):
        Q.dequantize_groupwise(f32meta)
    badcodes = Q.QuantizedTensor(kq.packed.to(torch.int8), kq.scale, kq.zero, 4, 32, 128)
    with pytest.raises(TypeError, match="packed must be uint8"):
        fused_decode_attention(q, kq, badcodes)
    cpu_meta = Q.QuantizedTensor(vq.packed, vq.scale.cpu(), vq.zero, 4, 32, 128)
    with pytest.raises(ValueError, match="is on cpu"):
        fused_decode_attention(q, kq, cpu_meta)


# ------------------------------------------------------------------ fp16 control


@pytest.mark.parametrize("S", [1, 17, 128, 2048, 16384])
@pytest.mark.parametrize("shape", SHAPES)
def test_fp16_control_matches_reference(S, shape):
    B, HQ, HKV, D = shape
    q, k, v = make_random_kv(B, HQ, HKV, S, D, device=DEV, seed=50)
    got = fp16_decode_attention(q, k, v)
    ref = O.reference_decode_attention(q.float().cpu().numpy(), k.float().cpu().numpy(),
                                       v.float().cpu().numpy())
    assert_close(got, ref, f"fp16 S={S} {shape}")


@pytest.mark.parametrize("num_splits", [1, 3, 17])
def test_fp16_control_splits(num_splits):
    q, k, v = make_random_kv(1, 12, 2, 3000, 128, device=DEV, seed=51)
    got = fp16_decode_attention(q, k, v, num_splits=num_splits, block_n=32)
    ref = O.reference_decode_attention(q.float().cpu().numpy(), k.float().cpu().numpy(),
                                       v.float().cpu().numpy())
    assert_close(got, ref, f"fp16 splits={num_splits}")


# ------------------------------------------------------------------ combine


@pytest.mark.parametrize("NS", [1, 2, 7, 33, 300])
@pytest.mark.parametrize("D", [64, 128])
def test_combine_matches_oracle(NS, D):
    g = torch.Generator().manual_seed(NS * 10 + D)
    acc = torch.randn(2, 5, NS, D, generator=g)
    m = torch.randn(2, 5, NS, generator=g) * 8
    l = torch.rand(2, 5, NS, generator=g) * 50 + 0.1
    if NS > 2:  # empty splits contribute nothing
        m[:, :, 1] = float("-inf")
        l[:, :, 1] = 0
        acc[:, :, 1] = 0
    ref = O.combine_splits(acc.numpy(), m.numpy(), l.numpy())
    got = combine_splits(acc.to(DEV), m.to(DEV), l.to(DEV))
    assert np.allclose(got.cpu().numpy(), ref, rtol=2e-5, atol=2e-6)
    om = torch.empty(2, 5, device=DEV)
    ol = torch.empty(2, 5, device=DEV)
    raw = combine_splits(acc.to(DEV), m.to(DEV), l.to(DEV), out_m=om, out_l=ol)
    assert np.allclose((raw / ol[..., None]).cpu().numpy(), ref, rtol=2e-5, atol=2e-6)
    assert torch.equal(om.cpu(), m.max(dim=-1).values)


def test_partials_match_oracle_format():
    """(acc, m, l) of the split kernel in the exp2 domain against the oracle's
    restatement of the reference's partial format.  The kernel may cut a split into
    several CTA segments (slots); merged per split they are the split's partial."""
    q, k, v = make_random_kv(1, 12, 2, 1024, 128, device=DEV, seed=60)
    kq, vq = Q.quantize_kv(k, v, 4, 32)
    ws = {}
    fused_decode_attention(q, kq, vq, num_splits=4, block_n=64, _workspace=ws)
    B, HQ, nslots, D = ws["key"]
    SEG = nslots // 4
    kd = O.dequantize_groupwise(to_oracle(kq))
    vd = O.dequantize_groupwise(to_oracle(vq))
    acc, m, l = O.split_partials(q.float().cpu().numpy(), kd, vd, 256, 4)
    ka = ws["acc"].cpu().numpy().reshape(B, HQ, 4, SEG, D)
    km = ws["maxs"].cpu().numpy().reshape(B, HQ, 4, SEG)
    kl = ws["sums"].cpu().numpy().reshape(B, HQ, 4, SEG)
    gm = km.max(axis=-1)
    with np.errstate(invalid="ignore"):
        w = np.where(np.isneginf(km), 0.0, np.exp2(km - gm[..., None]))
    ga = (np.where(w[..., None] > 0, ka, 0.0) * w[..., None]).sum(axis=3)
    gl = (np.where(w > 0, kl, 0.0) * w).sum(axis=-1)
    assert np.allclose(gm, m, atol=2e-3)  # m is the true maximum of the split
    got = ga * np.exp2(gm - m)[..., None]
    assert np.linalg.norm(got - acc) / np.linalg.norm(acc) < 5e-3
    assert np.allclose(gl * np.exp2(gm - m), l, rtol=5e-3)


# ------------------------------------------------------------------ ragged batches


@pytest.mark.parametrize("nbits,D,gs,HQ,HKV", [(4, 128, 32, 32, 8), (2, 64, 64, 8, 1),
                                               (4, 64, 32, 8, 1), (2, 128, 128, 32, 8)])
def test_ragged_seq_lens(nbits, D, gs, HQ, HKV):
    B, S = 6, 2500
    lens = ragged_seq_lens(B, 1, S, seed=7)
    lens[0] = S
    lens[1] = 1
    q, k, v = make_random_kv(B, HQ, HKV, S, D, device=DEV, seed=70)
    kq, vq = Q.quantize_kv(k, v, nbits, gs)
    sl = lens.to(DEV)
    got = fused_decode_attention(q, kq, vq, seq_lens=sl)
    assert_close(got, oracle_attention(q, kq, vq, seq_lens=lens), "ragged fused")
    got16 = fp16_decode_attention(q, k, v, seq_lens=sl)
    ref16 = O.reference_decode_attention(q.float().cpu().numpy(), k.float().cpu().numpy(),
                                         v.float().cpu().numpy(), seq_lens=lens.numpy())
    assert_close(got16, ref16, "ragged fp16")


def test_full_size_properties_llama8b_batch():
    """Llama-3-8B shape, batch 8 of ctx 4096, at full per-sequence size: output is
    a convex combination of dequantised V rows (bounded by their min/max per dim),
    invariant to the split count, and equal to the oracle on one sampled sequence."""
    B, HQ, HKV, S, D = 8, 32, 8, 4096, 128
    q, k, v = make_random_kv(B, HQ, HKV, S, D, device=DEV, seed=80, outlier_frac=0.0)
    kq, vq = Q.quantize_kv(k, v, 4, 32)
    out = fused_decode_attention(q, kq, vq)
    vd = Q.dequantize_groupwise(vq, torch.float32)
    lo = vd.amin(dim=2).repeat_interleave(HQ // HKV, dim=1)
    hi = vd.amax(dim=2).repeat_interleave(HQ // HKV, dim=1)
    assert torch.all(out >= lo - 1e-3) and torch.all(out <= hi + 1e-3)
    out2 = fused_decode_attention(q, kq, vq, num_splits=7)
    assert (out - out2).abs().max().item() < 2e-3
    b = 5
    sub = lambda t: Q.QuantizedTensor(t.packed[b:b + 1], t.scale[b:b + 1], t.zero[b:b + 1], 4, 32, D)
    assert_close(out[b:b + 1], oracle_attention(q[b:b + 1], sub(kq), sub(vq)), "sampled sequence")


def test_no_bounded_wait_gave_up():
    """Every copy barrier inside the decode kernels completed: the device status word
    that a timed-out wait would set is still clear after the cases above."""
    from tritonkv_b200 import _cabi

    q, k, v = make_random_kv(1, 12, 2, 4096, 128, device=DEV, seed=90)
    kq, vq = Q.quantize_kv(k, v, 4, 32)
    fused_decode_attention(q, kq, vq)
    torch.cuda.synchronize()
    assert _cabi.device_status() == 0


# ------------------------------------------------------------------ history split over ranks


@pytest.mark.parametrize("world", [2, 4, 8])
def test_history_split_merge_emulated_on_one_gpu(world):
    """The cross-GPU history split with all ranks' work done in turn on one GPU: every
    "rank" reduces its token range to one unnormalised partial in the wire layout, the
    gathered buffer is merged by the strided combine kernel, and the result equals the
    oracle on the whole history (Llama-3-70B head layout, 2-bit, shortened context)."""
    from tritonkv_b200 import parallel as P
    from tritonkv_b200.kernels import combine_splits as combine

    B, HQ, HKV, S, D = 1, 64, 8, 5000, 128
    q, k, v = make_random_kv(B, HQ, HKV, S, D, device=DEV, seed=95)
    kq, vq = Q.quantize_kv(k, v, 2, 32)
    n = P.wire_floats(B, HQ, D)
    gathered = torch.empty(world, n, device=DEV)
    for r in range(world):
        lo, hi = P.history_shard(S, world, r)
        if hi <= lo:
            P.empty_partial_(gathered[r], B, HQ, D)
            continue
        sl = lambda t: Q.QuantizedTensor(t.packed[:, :, lo:hi].contiguous(),
                                         t.scale[:, :, lo:hi].contiguous(),
                                         t.zero[:, :, lo:hi].contiguous(), 2, 32, D)
        ws = {}
        fused_decode_attention(q, sl(kq), sl(vq), _workspace=ws, _partials_only=True)
        acc, m, l = P.wire_views(gathered[r], B, HQ, D)
        combine(ws["acc"], ws["maxs"], ws["sums"], out=acc, out_m=m, out_l=l)
    got = P.merge_gathered(gathered, B, HQ, D)
    assert_close(got, oracle_attention(q, kq, vq), f"history split over {world} ranks")


# ------------------------------------------------------------------ benchmark configurations


def _ragged_grid():
    for D in (64, 128):
        for HQ, HKV in ((8, 1), (32, 8)):
            for nbits in (2, 4):
                for gs in (32, 64, 128):
                    if gs <= D:  # gs=128 with D=64 is invalid in the reference too (quantize.py:200)
                        yield D, HQ, HKV, nbits, gs


@pytest.mark.parametrize("D,HQ,HKV,nbits,gs", list(_ragged_grid()))
def test_ragged_sweep_grid(D, HQ, HKV, nbits, gs):
    """The ragged batched sweep (batch 16, per-sequence lengths from a seed, 1 % of the K
    entries x20) over its whole (D, heads, nbits, group) grid, at lengths the oracle does
    in a second (the full lengths are covered by the property test below)."""
    from oracle.workloads import make_entry_outlier_k

    B, S = 16, 1536
    lens = ragged_seq_lens(B, 48, S, seed=D + HQ + nbits + gs)
    q, k, v = make_entry_outlier_k(B, HQ, HKV, S, D, device=DEV, seed=7, frac=0.01, factor=20.0)
    kq, vq = Q.quantize_kv(k, v, nbits, gs)
    got = fused_decode_attention(q, kq, vq, seq_lens=lens.to(DEV))
    assert_close(got, oracle_attention(q, kq, vq, seq_lens=lens), f"ragged D={D} {HQ}/{HKV} {nbits}b gs={gs}")


def test_ragged_full_lengths_properties():
    """Ragged batch at the sweep's full lengths (1024..32768): each sequence's output
    equals a dense call on that sequence alone cut to its length (bit-for-bit geometry
    differs, so within the kernel tolerance), and padding beyond seq_lens is never read
    (poisoning it with NaN scale/zero changes nothing)."""
    B, HQ, HKV, D = 4, 32, 8, 128
    lens = torch.tensor([32768, 1024, 20011, 7], dtype=torch.int32)
    S = 32768
    g = torch.Generator(device=DEV).manual_seed(5)
    q = torch.randn(B, HQ, D, generator=g, device=DEV).half()
    k = torch.randn(B, HKV, S, D, generator=g, device=DEV).half()
    v = torch.randn(B, HKV, S, D, generator=g, device=DEV).half()
    kq, vq = Q.quantize_kv(k, v, 4, 32)
    out = fused_decode_attention(q, kq, vq, seq_lens=lens.to(DEV))
    for b in range(B):
        n = int(lens[b])
        cut = lambda t: Q.QuantizedTensor(t.packed[b:b + 1, :, :n].contiguous(),
                                          t.scale[b:b + 1, :, :n].contiguous(),
                                          t.zero[b:b + 1, :, :n].contiguous(), 4, 32, D)
        alone = fused_decode_attention(q[b:b + 1], cut(kq), cut(vq))
        assert (out[b:b + 1] - alone).abs().max().item() < 2e-3
    for b in range(B):  # poison everything past each sequence's end
        n = int(lens[b])
        for t in (kq, vq):
            t.scale[b, :, n:] = float("nan")
            t.zero[b, :, n:] = float("inf")
            t.packed[b, :, n:] = 255
    out2 = fused_decode_attention(q, kq, vq, seq_lens=lens.to(DEV))
    assert torch.equal(out, out2)


def test_llama70b_long_context_full_size():
    """Llama-3-70B-shaped long-context decode at full size (HQ 64, HKV 8, ctx 131072,
    2-bit, 100 MB of cache) against the C twin of the oracle."""
    from oracle import c_oracle

    B, HQ, HKV, S, D = 1, 64, 8, 131072, 128
    g = torch.Generator(device=DEV).manual_seed(11)
    q = torch.randn(B, HQ, D, generator=g, device=DEV).half()
    k = torch.randn(B, HKV, S, D, generator=g, device=DEV).half()
    v = torch.randn(B, HKV, S, D, generator=g, device=DEV).half()
    kq, vq = Q.quantize_kv(k, v, 2, 32)
    del k, v
    got = fused_decode_attention(q, kq, vq)
    c_oracle.use_all_cores()
    h = lambda t: (t.cpu().numpy() if t.dtype == torch.uint8 else t.cpu().numpy().view(np.uint16))
    ref = c_oracle.decode_step(q.float().cpu().numpy(), h(kq.packed), h(kq.scale), h(kq.zero),
                               h(vq.packed), h(vq.scale), h(vq.zero), 2, 32)
    assert_close(got, ref, "llama-70b ctx 131072 2-bit")


def test_long_context_sweep_top_context_against_oracle():
    """The longest context of the reference's long-context sweep (ctx 393216, Qwen2.5-1.5B
    head layout, 4-bit; docs/preregistration_l2.md:36-38 of the reference), fused kernel and
    fp16 control, against the C twin of the memory-frugal grouped oracle
    (l2_sweep.py:196-236)."""
    from oracle import c_oracle

    B, HQ, HKV, S, D = 1, 12, 2, 393216, 128
    g = torch.Generator(device=DEV).manual_seed(31)
    q = torch.randn(B, HQ, D, generator=g, device=DEV).half()
    k = torch.randn(B, HKV, S, D, generator=g, device=DEV).half()
    v = torch.randn(B, HKV, S, D, generator=g, device=DEV).half()
    kq, vq = Q.quantize_kv(k, v, 4, 32)
    c_oracle.use_all_cores()
    assert_close(fused_decode_attention(q, kq, vq), c_oracle_attention(q, kq, vq), "ctx 393216 4-bit")
    got16 = fp16_decode_attention(q, k, v)
    ref16 = O.reference_decode_attention(q.float().cpu().numpy(), k.float().cpu().numpy(),
                                         v.float().cpu().numpy())
    assert_close(got16, ref16, "ctx 393216 fp16 control")


@pytest.mark.parametrize("nbits", [4, 2])
def test_llama8b_batch64_full_size_against_oracle(nbits):
    """Llama-3-8B-shaped decode at its full size (batch 64, HQ 32 / HKV 8, ctx 4096): the
    balanced dense schedule whose CTAs straddle unit boundaries and mark unused slots empty.
    Eight sampled sequences -- first, last and six between -- against the C twin of the
    oracle; every other sequence through the split-count invariance below."""
    B, HQ, HKV, S, D = 64, 32, 8, 4096, 128
    g = torch.Generator(device=DEV).manual_seed(21 + nbits)
    q = torch.randn(B, HQ, D, generator=g, device=DEV).half()
    k = torch.randn(B, HKV, S, D, generator=g, device=DEV).half()
    v = torch.randn(B, HKV, S, D, generator=g, device=DEV).half()
    kq, vq = Q.quantize_kv(k, v, nbits, 32)
    del k, v
    got = fused_decode_attention(q, kq, vq)
    rows = [0, 9, 18, 27, 36, 45, 54, 63]
    ref = c_oracle_attention(q, kq, vq, rows=rows)
    assert_close(got[rows], ref, f"batch 64 x ctx 4096, {nbits}-bit, sampled sequences")
    # a different cut of the same work (explicit splits: static units) agrees everywhere
    other = fused_decode_attention(q, kq, vq, num_splits=3)
    assert (got - other).abs().max().item() < 2e-3


@pytest.mark.parametrize("D,HQ,HKV,nbits,gs", [(128, 32, 8, 4, 32), (128, 8, 1, 2, 64),
                                               (64, 32, 8, 2, 32), (64, 8, 1, 4, 64)])
def test_ragged_sweep_full_lengths_against_oracle(D, HQ, HKV, nbits, gs):
    """One cell per (head_dim, heads) of the ragged batched sweep at its real lengths (batch
    16, lengths uniform in [1024, 32768] from the seed, 1 % of the K entries x20): the
    longest, the shortest and two more sequences against the C twin of the oracle."""
    B, S_max = 16, 32768
    lens = ragged_seq_lens(B, 1024, S_max, seed=D + HQ)
    S = int(lens.max())
    g = torch.Generator(device=DEV).manual_seed(17)  # drawn on the device: 0.5 G values at HKV 8
    q = torch.randn(B, HQ, D, generator=g, device=DEV).half()
    k = torch.randn(B, HKV, S, D, generator=g, device=DEV)
    k = torch.where(torch.rand(B, HKV, S, D, generator=g, device=DEV) < 0.01, k * 20.0, k).half()
    v = torch.randn(B, HKV, S, D, generator=g, device=DEV).half()
    kq, vq = Q.quantize_kv(k, v, nbits, gs)
    del k, v
    got = fused_decode_attention(q, kq, vq, seq_lens=lens.to(DEV))
    rows = sorted({int(lens.argmax()), int(lens.argmin()), 3, 11})
    ref = c_oracle_attention(q, kq, vq, seq_lens=lens, rows=rows)
    assert_close(got[rows], ref, f"ragged full lengths D={D} {HQ}/{HKV} {nbits}b gs={gs}")


# ------------------------------------------------------------------ metadata alignment
@pytest.mark.parametrize("nbits,D,gs", [(4, 128, 128), (2, 64, 64), (4, 128, 64), (2, 128, 32),
                                        (4, 64, 16)])
@pytest.mark.parametrize("S", [33, 1001, 2050, 4099])
def test_scale_zero_rows_at_every_alignment(nbits, D, gs, S):
    """History lengths that leave the per-sequence scale/zero rows on 2-, 4-, 8- and 16-byte
    boundaries (one to eight groups per token), dense and ragged, and the same cache seen
    through a view that starts one sequence in: all copy paths give the oracle's answer."""
    B, HQ, HKV = 3, 8, 2
    q, k, v = make_random_kv(B, HQ, HKV, S, D, device=DEV, seed=S + gs)
    kq, vq = Q.quantize_kv(k, v, nbits, gs)
    ref = oracle_attention(q, kq, vq)
    assert_close(fused_decode_attention(q, kq, vq), ref, "dense")
    lens = torch.tensor([S, max(1, S // 3), S - 7], dtype=torch.int32)
    assert_close(fused_decode_attention(q, kq, vq, seq_lens=lens.to(DEV)),
                 oracle_attention(q, kq, vq, seq_lens=lens), "ragged")
    # sequences 1.. of the same storage: the pointers now sit HKV*S rows into the allocation
    cut = lambda t: Q.QuantizedTensor(t.packed[1:], t.scale[1:], t.zero[1:], nbits, gs, D)
    if (HKV * S * D * nbits // 8) % 16 == 0:  # the packed codes themselves need 16-byte alignment
        got = fused_decode_attention(q[1:].contiguous(), cut(kq), cut(vq))
        assert_close(got, ref[1:], "offset view")


# ------------------------------------------------------------------ graphed serving step
def test_graphed_decode_step_equals_direct_calls_and_follows_the_cache():
    """GraphedDecodeStep replays H2D(q) + decode + D2H(out) as one graph: same bits as the
    direct call, and a cache that grows in place (append + seq_lens on the device) is seen
    by later replays without re-capturing."""
    from tritonkv_b200 import GraphedDecodeStep

    torch.manual_seed(11)
    B, HQ, HKV, D, cap, nbits, gs = 2, 8, 2, 128, 300, 4, 32
    k = torch.randn(B, HKV, cap, D, device=DEV, dtype=torch.float16)
    v = torch.randn(B, HKV, cap, D, device=DEV, dtype=torch.float16)
    kq = Q.empty_cache(B, HKV, cap, D, nbits, gs, DEV)
    vq = Q.empty_cache(B, HKV, cap, D, nbits, gs, DEV)
    n0 = 200
    Q.append_kv(kq, vq, k[:, :, :n0], v[:, :, :n0], 0)
    lens = torch.full((B,), n0, dtype=torch.int32, device=DEV)
    step = GraphedDecodeStep(kq, vq, HQ, seq_lens=lens)
    for t in range(n0, n0 + 40):
        q = torch.randn(B, HQ, D, dtype=torch.float16)
        step.run(q)
        got = step.result().clone()
        ref = fused_decode_attention(q.to(DEV), kq, vq, seq_lens=lens)
        assert torch.equal(got, ref.cpu()), t
        # the loop's write side: one more token, lengths bumped on the device
        Q.append_kv(kq, vq, k[:, :, t:t + 1], v[:, :, t:t + 1], lens)
        lens += 1
    dense = Q.quantize_kv(k[:, :, :n0 + 40].contiguous(), v[:, :, :n0 + 40].contiguous(), nbits, gs)
    q = torch.randn(B, HQ, D, dtype=torch.float16)
    step.run(q)
    assert_close(step.result(), oracle_attention(q.to(DEV), dense[0], dense[1]), "after 40 appends")


@pytest.mark.parametrize("B,HQ,HKV,S", [(1, 12, 2, 8192), (4, 32, 8, 1000), (1, 12, 2, 17)])
def test_zero_copy_graphed_step_equals_the_copying_one(B, HQ, HKV, S):
    """GraphedDecodeStep(zero_copy=True): the last kernel of the step writes the result into
    pinned host memory itself (no device-to-host copy node in the graph); same bits as the
    copying form and as the direct call, step after step."""
    from tritonkv_b200 import GraphedDecodeStep

    q0, k, v = make_random_kv(B, HQ, HKV, S, 128, device=DEV, seed=41)
    kq, vq = Q.quantize_kv(k, v, 4, 32)
    zc = GraphedDecodeStep(kq, vq, HQ, zero_copy=True)
    cp = GraphedDecodeStep(kq, vq, HQ)
    g = torch.Generator().manual_seed(5)
    for _ in range(4):
        q = torch.randn(B, HQ, 128, generator=g).half()
        zc.run(q)
        a = zc.result().clone()
        cp.run(q)
        b = cp.result().clone()
        assert torch.equal(a, b)
        assert torch.equal(a, fused_decode_attention(q.to(DEV), kq, vq).cpu())


def test_combine_flag_equals_two_calls_through_the_c_abi():
    """TKV_FLAG_COMBINE (split kernel + combine enqueued by one call) gives the bits of
    tkv_fused_decode followed by tkv_combine."""
    from tritonkv_b200 import _cabi
    from tritonkv_b200.kernels._launch import split_geometry

    B, HQ, HKV, D, S, nbits, gs = 2, 8, 2, 128, 3000, 4, 32
    q, k, v = make_random_kv(B, HQ, HKV, S, D, device=DEV, seed=31)
    kq, vq = Q.quantize_kv(k, v, nbits, gs)
    lib = _cabi.load()
    _, ns, ss = split_geometry(S, 64, 4, B, HKV, None)  # explicit splits: several partial slots per head
    nslots, _ = _cabi.decode_plan(_cabi.KERNEL_FUSED_SPLIT, nbits, D, gs, B, HQ, HKV, S, ns, ss, False)
    assert nslots > 1
    stream = _cabi.stream_ptr(q.device)
    outs = []
    for flags in (0, _cabi.FLAG_COMBINE):
        acc = torch.empty(B, HQ, nslots, D, device=DEV)
        m = torch.empty(B, HQ, nslots, device=DEV)
        l = torch.empty(B, HQ, nslots, device=DEV)
        out = torch.full((B, HQ, D), float("nan"), device=DEV)
        _cabi.check(lib.tkv_fused_decode(
            q.data_ptr(), _cabi.dtype_code(q), kq.packed.data_ptr(), kq.scale.data_ptr(),
            kq.zero.data_ptr(), vq.packed.data_ptr(), vq.scale.data_ptr(), vq.zero.data_ptr(),
            acc.data_ptr(), m.data_ptr(), l.data_ptr(), out.data_ptr(), B, HQ, HKV, S, D, nbits, gs,
            1.0 / D ** 0.5, ns, ss, nslots, None, flags, stream))
        if flags == 0:
            assert torch.isnan(out).all()  # partials only: out untouched
            _cabi.check(lib.tkv_combine(acc.data_ptr(), m.data_ptr(), l.data_ptr(), out.data_ptr(),
                                        None, None, B, HQ, nslots, D, stream))
        outs.append(out)
    torch.cuda.synchronize()
    assert torch.equal(outs[0], outs[1])
    assert_close(outs[1], oracle_attention(q, kq, vq), "combine flag")
