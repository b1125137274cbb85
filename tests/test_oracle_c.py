"""The C restatement of the reference's CPU path against the numpy oracle (itself
pinned to reference-generated fixtures): bit-exact for quantiser and packing,
1e-5 for fp32 attention."""

import ctypes
import os
import subprocess

import numpy as np
import pytest

from oracle import tkv_oracle as O
from oracle import c_oracle


@pytest.fixture(scope="module")
def C():
    return c_oracle.load()


def _x(rows, D, seed):
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((rows, D)).astype(np.float32)
    x[rng.random((rows, D)) < 0.02] *= 8
    x[1, :32] = 3.5
    return x.astype(np.float16).astype(np.float32)


@pytest.mark.parametrize("nbits", [2, 4])
@pytest.mark.parametrize("D,gs", [(128, 16), (128, 32), (128, 128), (64, 32), (64, 64)])
def test_quantize_pack_dequantize_bit_exact(C, nbits, D, gs):
    x = _x(50, D, nbits + D + gs)
    ref = O.quantize_groupwise(x, nbits, gs)
    packed, scale, zero = c_oracle.quantize_groupwise(x, nbits, gs)
    assert np.array_equal(packed, ref.packed)
    assert np.array_equal(scale, ref.scale.view(np.uint16))
    assert np.array_equal(zero, ref.zero.view(np.uint16))
    codes = O.unpack_codes(ref.packed, nbits, D)
    assert np.array_equal(c_oracle.unpack_codes(packed, nbits, D), codes)
    assert np.array_equal(c_oracle.pack_codes(codes, nbits), ref.packed)
    deq = c_oracle.dequantize_groupwise(packed, scale, zero, nbits, gs, D)
    assert np.array_equal(deq.view(np.uint32), O.dequantize_groupwise(ref).view(np.uint32))


@pytest.mark.parametrize("nbits", [2, 4])
@pytest.mark.parametrize("gs", [32, 128])
def test_quantize_edges_match_the_reference_fixture(C, golden_dir, nbits, gs):
    from test_oracle_golden import f16_equal

    g = np.load(os.path.join(golden_dir, "quantize_edges.npz"))
    packed, scale, zero = c_oracle.quantize_groupwise(g["x_edges"], nbits, gs)
    key = f"edges_n{nbits}_g{gs}"
    assert f16_equal(scale, g[f"scale_{key}"])
    assert f16_equal(zero, g[f"zero_{key}"])
    assert np.array_equal(packed, g[f"packed_{key}"])


@pytest.mark.parametrize("name", ["cfg1", "qwen_s17_2b", "mha_d64", "llama_b2_d64_g64",
                                  "gqa8_g128_2b", "gqa4_g16"])
def test_decode_step_matches_golden(C, golden_dir, name):
    g = np.load(os.path.join(golden_dir, "attention.npz"))
    B, HQ, HKV, S, D, nbits, gs, seed = [int(v) for v in g[f"{name}_meta"]]
    out = c_oracle.decode_step(g[f"{name}_q"].astype(np.float32),
                               g[f"{name}_kpacked"], g[f"{name}_kscale"], g[f"{name}_kzero"],
                               g[f"{name}_vpacked"], g[f"{name}_vscale"], g[f"{name}_vzero"],
                               nbits, gs)
    assert np.allclose(out, g[f"{name}_out"], atol=1e-5, rtol=1e-5)


def test_decode_step_ragged(C):
    rng = np.random.default_rng(5)
    B, HQ, HKV, S, D = 3, 8, 2, 70, 64
    q = rng.standard_normal((B, HQ, D)).astype(np.float32)
    k = rng.standard_normal((B, HKV, S, D)).astype(np.float32)
    v = rng.standard_normal((B, HKV, S, D)).astype(np.float32)
    kq, vq = O.quantize_kv(k, v, 4, 32)
    lens = np.array([70, 1, 33], np.int32)
    out = c_oracle.decode_step(q, kq.packed, kq.scale, kq.zero, vq.packed, vq.scale, vq.zero, 4, 32,
                               seq_lens=lens)
    ref = O.reference_on_quantized(q, kq, vq, seq_lens=lens)
    assert np.allclose(out, ref, atol=1e-5, rtol=1e-5)
