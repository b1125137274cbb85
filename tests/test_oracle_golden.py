"""The numpy oracle against the fixtures produced by the reference itself.

These pin the checker: if the oracle drifts from the reference's quantize.py /
reference.py / Triton kernels (run under Triton's CPU interpreter), these fail
before any CUDA parity claim is made.  Fixture provenance: tests/golden/make_golden.py.
"""

import os

import numpy as np
import pytest

from oracle import tkv_oracle as O


def _load(golden_dir, name):
    return np.load(os.path.join(golden_dir, name))


def test_pack_known_answers(golden_dir):
    g = _load(golden_dir, "pack.npz")
    # split-P: byte j = code[j] | code[j+DP] << nbits ...  (quantize.py:42-46)
    assert bytes(g["pack4_known_packed"]) == bytes([0x51, 0x62, 0x73, 0x84])
    assert bytes(g["pack2_known_packed"]) == bytes([0x88, 0xDD])
    assert np.array_equal(O.pack_codes(g["pack4_known_codes"], 4), g["pack4_known_packed"])
    assert np.array_equal(O.pack_codes(g["pack2_known_codes"], 2), g["pack2_known_packed"])


def f16_equal(a, b):
    """Bit patterns of two fp16 arrays agree; NaNs agree with NaNs whatever their payload."""
    a, b = np.asarray(a).view(np.float16), np.asarray(b).view(np.float16)
    nan = np.isnan(a)
    return bool(np.array_equal(nan, np.isnan(b)) and
                np.array_equal(a.view(np.uint16)[~nan], b.view(np.uint16)[~nan]))


@pytest.mark.parametrize("nbits", [2, 4])
@pytest.mark.parametrize("gs", [32, 128])
def test_quantize_edges_bit_exact(golden_dir, nbits, gs):
    """Edges the reference's own tests leave open, pinned on what its quantiser returns:
    group ranges that underflow fp16 (scale becomes a subnormal or 0 and the codes collapse
    to {0, qmax}), a constant group, and +inf / -inf / NaN inside a group (scale inf or 1,
    zero -inf or NaN, codes 0)."""
    g = _load(golden_dir, "quantize_edges.npz")
    qt = O.quantize_groupwise(g["x_edges"], nbits, gs)
    key = f"edges_n{nbits}_g{gs}"
    assert f16_equal(qt.scale, g[f"scale_{key}"])
    assert f16_equal(qt.zero, g[f"zero_{key}"])
    assert np.array_equal(qt.packed, g[f"packed_{key}"])


@pytest.mark.parametrize("nbits", [2, 4])
@pytest.mark.parametrize("D", [64, 128])
def test_pack_unpack_bit_exact(golden_dir, nbits, D):
    g = _load(golden_dir, "pack.npz")
    codes, packed = g[f"pack_codes_n{nbits}_d{D}"], g[f"pack_packed_n{nbits}_d{D}"]
    assert np.array_equal(O.pack_codes(codes, nbits), packed)
    assert np.array_equal(O.unpack_codes(packed, nbits, D), codes)


def _bf16_to_f32(raw):
    return (raw.astype(np.uint16).astype(np.uint32) << 16).view(np.float32)


@pytest.mark.parametrize("name", ["f32", "f16", "bf16"])
@pytest.mark.parametrize("nbits", [2, 4])
@pytest.mark.parametrize("gs", [16, 32, 64, 128])
def test_quantize_bit_exact(golden_dir, name, nbits, gs):
    g = _load(golden_dir, "quantize.npz")
    x = g[f"x_{name}"]
    if name == "bf16":
        x = _bf16_to_f32(x.view(np.uint16))
    qt = O.quantize_groupwise(x, nbits, gs)
    key = f"{name}_n{nbits}_g{gs}"
    assert np.array_equal(qt.scale.view(np.uint16), g[f"scale_{key}"].view(np.uint16))
    assert np.array_equal(qt.zero.view(np.uint16), g[f"zero_{key}"].view(np.uint16))
    assert np.array_equal(qt.packed, g[f"packed_{key}"])
    if name == "f16":
        deq = O.dequantize_groupwise(qt)
        assert np.array_equal(deq.view(np.uint32), g[f"deq_{key}"].view(np.uint32))


@pytest.mark.parametrize("nbits", [2, 4])
@pytest.mark.parametrize("gs", [16, 32, 64])
def test_quantize_d64_bit_exact(golden_dir, nbits, gs):
    g = _load(golden_dir, "quantize.npz")
    qt = O.quantize_groupwise(g["x64_f16"], nbits, gs)
    key = f"d64_n{nbits}_g{gs}"
    assert np.array_equal(qt.packed, g[f"packed_{key}"])
    assert np.array_equal(qt.scale.view(np.uint16), g[f"scale_{key}"].view(np.uint16))
    assert np.array_equal(qt.zero.view(np.uint16), g[f"zero_{key}"].view(np.uint16))


ATT = ["cfg1", "qwen_s17_2b", "mha_d64", "llama_b2_d64_g64", "gqa8_g128_2b", "gqa4_g16"]


def _case(g, name):
    B, HQ, HKV, S, D, nbits, gs, seed = [int(v) for v in g[f"{name}_meta"]]
    kq = O.OracleQuantized(g[f"{name}_kpacked"], g[f"{name}_kscale"], g[f"{name}_kzero"], nbits, gs, D)
    vq = O.OracleQuantized(g[f"{name}_vpacked"], g[f"{name}_vscale"], g[f"{name}_vzero"], nbits, gs, D)
    return g[f"{name}_q"], kq, vq


@pytest.mark.parametrize("name", ATT)
def test_attention_matches_reference(golden_dir, name):
    """fp32 attention: summation order differs from torch's, hence a tolerance
    (1e-5 abs + 1e-5 rel), the bound the reference uses for its own twin
    (test_l2_sweep.py:74-94)."""
    g = _load(golden_dir, "attention.npz")
    q, kq, vq = _case(g, name)
    got = O.reference_on_quantized(q, kq, vq)
    ref = g[f"{name}_out"]
    assert np.allclose(got, ref, atol=1e-5, rtol=1e-5), np.abs(got - ref).max()


@pytest.mark.parametrize("name", ["qwen_s17_2b", "mha_d64"])
def test_attention_fp16_cache_matches_reference(golden_dir, name):
    g = _load(golden_dir, "attention.npz")
    got = O.reference_decode_attention(g[f"{name}_q"], g[f"{name}_k16"], g[f"{name}_v16"])
    assert np.allclose(got, g[f"{name}_out_fp16cache"], atol=1e-5, rtol=1e-5)


@pytest.mark.parametrize("name", ATT)
def test_split_then_combine_equals_attention(golden_dir, name):
    g = _load(golden_dir, "attention.npz")
    q, kq, vq = _case(g, name)
    k, v = O.dequantize_groupwise(kq), O.dequantize_groupwise(vq)
    S = k.shape[2]
    for want in (1, 2, 5):
        _, ns, ss = O.split_geometry(S, 16, want)
        acc, m, l = O.split_partials(q, k, v, ss, ns)
        got = O.combine_splits(acc, m, l)
        assert np.allclose(got, g[f"{name}_out"], atol=2e-5, rtol=2e-5)


@pytest.mark.parametrize("name", ["tk_qwen", "tk_2b_d64"])
def test_partial_format_matches_reference_kernels(golden_dir, name):
    """(acc, m, l) produced by the reference's Triton split kernel (CPU
    interpreter) against the oracle's restatement.  The kernel rounds the
    dequantised K/V and p to fp16 before its dots, so partials agree to fp16
    accuracy (rel 5e-3), while m -- a plain max of fp32 dots -- agrees to 1e-2 abs
    in log2 units, and the combined output to the reference's own thresholds."""
    g = _load(golden_dir, "triton_partials.npz")
    assert int(g["triton_interpreter"][0]) == 1
    B, HQ, HKV, S, D, nbits, gs, seed, ns, ss = [int(v) for v in g[f"{name}_meta"]]
    kq = O.OracleQuantized(g[f"{name}_kpacked"], g[f"{name}_kscale"], g[f"{name}_kzero"], nbits, gs, D)
    vq = O.OracleQuantized(g[f"{name}_vpacked"], g[f"{name}_vscale"], g[f"{name}_vzero"], nbits, gs, D)
    q = g[f"{name}_q"]
    k, v = O.dequantize_groupwise(kq), O.dequantize_groupwise(vq)
    acc, m, l = O.split_partials(q, k, v, ss, ns)
    assert acc.shape == g[f"{name}_acc"].shape
    assert np.allclose(m, g[f"{name}_maxs"], atol=1e-2)
    # compare partials after removing the (slightly different) max
    w_o = np.exp2(m - m.max(axis=-1, keepdims=True))
    w_r = np.exp2(g[f"{name}_maxs"] - g[f"{name}_maxs"].max(axis=-1, keepdims=True))
    assert np.allclose(l * w_o, g[f"{name}_sums"] * w_r, rtol=1e-2, atol=1e-3)
    a_o, a_r = acc * w_o[..., None], g[f"{name}_acc"] * w_r[..., None]
    assert np.linalg.norm(a_o - a_r) / np.linalg.norm(a_r) < 5e-3
    # the oracle's combine applied to the reference kernel's partials gives the
    # reference kernel's own output (same sequential loop)
    got = O.combine_splits(g[f"{name}_acc"], g[f"{name}_maxs"], g[f"{name}_sums"])
    assert np.allclose(got, g[f"{name}_out"], atol=1e-5, rtol=1e-5)
    rep = O.allclose_report(g[f"{name}_out"], O.reference_decode_attention(q, k, v))
    assert rep["ok"] and rep["cosine"] >= 0.99999 and rep["rel_l2"] <= 5e-3, rep


def test_split_geometry_matches_reference_launcher():
    # kernels/fused_decode_attn.py:487-499 worked by hand
    assert O.split_geometry(4096, 64, 17) == (64, 16, 256)
    assert O.split_geometry(3000, 128, 5) == (128, 5, 640)
    assert O.split_geometry(1, 64, 8) == (16, 1, 16)
    assert O.split_geometry(17, 64, 64) == (32, 1, 32)
    assert O.pick_num_splits(1, 2, 128, 592) == 128
    assert O.pick_num_splits(64, 8, 64, 592) == 1


@pytest.mark.parametrize("order", ["sorted", "shuffled", "finite_shuffled"])
@pytest.mark.parametrize("nbits", [2, 4])
@pytest.mark.parametrize("gs", [8, 32])
def test_quantize_every_f16_bit_pattern_pinned_on_the_reference(golden_dir, order, nbits, gs):
    """All 65536 fp16 bit patterns (exact ties, fp16-underflowing ranges, infinities and NaNs in
    every position) through the oracle's quantiser against what the reference's own
    ``quantize_groupwise`` returned for them."""
    g = np.load(os.path.join(golden_dir, "quantize_allbits.npz"))
    x = g[f"x_{order}"].view(np.float16)
    ref = O.quantize_groupwise(x, nbits, gs)
    key = f"{order}_n{nbits}_g{gs}"
    assert np.array_equal(ref.packed, g[f"packed_{key}"])
    assert f16_equal(ref.scale, g[f"scale_{key}"].view(np.float16))
    assert f16_equal(ref.zero, g[f"zero_{key}"].view(np.float16))
