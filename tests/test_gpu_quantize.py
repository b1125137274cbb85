"""GPU parity of the pack / quantise kernels: bit-exact against the oracle and the
reference-generated golden fixtures, all through the C ABI.  Cases follow the
reference's quantiser tests (test_correctness.py:78-134)."""

import math
import os

import numpy as np
import pytest
import torch

from oracle import tkv_oracle as O
from tritonkv_b200 import quantize as Q

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _np(t):
    return t.cpu().numpy()


@pytest.mark.parametrize("nbits", Q.SUPPORTED_BITS)
@pytest.mark.parametrize("head_dim", [64, 128])
def test_pack_unpack_roundtrip(nbits, head_dim):
    torch.manual_seed(0)
    qmax = (1 << nbits) - 1
    codes = torch.randint(0, qmax + 1, (3, 5, head_dim), dtype=torch.uint8)
    packed = Q.pack_codes(codes.to(DEV), nbits)
    assert packed.shape == (3, 5, head_dim // (8 // nbits))
    assert np.array_equal(_np(packed), O.pack_codes(codes.numpy(), nbits))
    back = Q.unpack_codes(packed, nbits, head_dim)
    assert torch.equal(back.cpu(), codes)


def test_pack_known_answers_and_golden(golden_dir):
    g = np.load(os.path.join(golden_dir, "pack.npz"))
    p4 = Q.pack_codes(torch.arange(1, 9, dtype=torch.uint8, device=DEV), 4)
    assert bytes(_np(p4)) == bytes([0x51, 0x62, 0x73, 0x84])
    p2 = Q.pack_codes(torch.tensor([0, 1, 2, 3, 0, 1, 2, 3], dtype=torch.uint8, device=DEV), 2)
    assert bytes(_np(p2)) == bytes([0x88, 0xDD])
    for nbits in (2, 4):
        for D in (64, 128):
            codes = torch.from_numpy(g[f"pack_codes_n{nbits}_d{D}"]).to(DEV)
            assert np.array_equal(_np(Q.pack_codes(codes, nbits)), g[f"pack_packed_n{nbits}_d{D}"])


def _bf16(raw):
    return torch.from_numpy(raw.copy()).view(torch.bfloat16)


@pytest.mark.parametrize("name", ["f32", "f16", "bf16"])
@pytest.mark.parametrize("nbits", [2, 4])
@pytest.mark.parametrize("gs", [16, 32, 64, 128])
def test_quantize_golden_bit_exact(golden_dir, name, nbits, gs):
    g = np.load(os.path.join(golden_dir, "quantize.npz"))
    x = _bf16(g["x_bf16"]) if name == "bf16" else torch.from_numpy(g[f"x_{name}"])
    qt = Q.quantize_groupwise(x.to(DEV), nbits, gs)
    key = f"{name}_n{nbits}_g{gs}"
    assert np.array_equal(_np(qt.scale).view(np.uint16), g[f"scale_{key}"].view(np.uint16))
    assert np.array_equal(_np(qt.zero).view(np.uint16), g[f"zero_{key}"].view(np.uint16))
    assert np.array_equal(_np(qt.packed), g[f"packed_{key}"])
    if name == "f16":
        deq = Q.dequantize_groupwise(qt, torch.float32)
        assert np.array_equal(_np(deq).view(np.uint32), g[f"deq_{key}"].view(np.uint32))


@pytest.mark.parametrize("nbits", [2, 4])
@pytest.mark.parametrize("gs", [16, 32, 64])
def test_quantize_golden_d64(golden_dir, nbits, gs):
    g = np.load(os.path.join(golden_dir, "quantize.npz"))
    qt = Q.quantize_groupwise(torch.from_numpy(g["x64_f16"]).to(DEV), nbits, gs)
    key = f"d64_n{nbits}_g{gs}"
    assert np.array_equal(_np(qt.packed), g[f"packed_{key}"])
    assert np.array_equal(_np(qt.scale).view(np.uint16), g[f"scale_{key}"].view(np.uint16))
    assert np.array_equal(_np(qt.zero).view(np.uint16), g[f"zero_{key}"].view(np.uint16))


@pytest.mark.parametrize("nbits", [2, 4])
@pytest.mark.parametrize("D,gs", [(128, 32), (128, 128), (64, 16), (64, 64), (256, 32)])
@pytest.mark.parametrize("dtype", [torch.float16, torch.float32])
def test_quantize_matches_oracle_on_a_cache_shaped_tensor(nbits, D, gs, dtype):
    """A (B, HKV, S, D) tensor with outliers, ragged row count (not a multiple of
    the warp's row tiling), against the oracle bit for bit."""
    g = torch.Generator().manual_seed(nbits * 1000 + D + gs)
    x = torch.randn(2, 3, 37, D, generator=g)
    x = torch.where(torch.rand(x.shape, generator=g) < 0.01, x * 20, x).to(dtype)
    qt = Q.quantize_groupwise(x.to(DEV), nbits, gs)
    ref = O.quantize_groupwise(x.numpy(), nbits, gs)
    assert np.array_equal(_np(qt.packed), ref.packed)
    assert np.array_equal(_np(qt.scale).view(np.uint16), ref.scale.view(np.uint16))
    assert np.array_equal(_np(qt.zero).view(np.uint16), ref.zero.view(np.uint16))
    for dt, npdt in ((torch.float32, np.float32), (torch.float16, np.float16)):
        deq = Q.dequantize_groupwise(qt, dt)
        assert np.array_equal(_np(deq), O.dequantize_groupwise(ref, npdt))


@pytest.mark.parametrize("nbits", Q.SUPPORTED_BITS)
@pytest.mark.parametrize("group_size", [16, 32, 64])
def test_quant_error_within_half_step(nbits, group_size):
    torch.manual_seed(1)
    x = torch.randn(4, 7, 128, device=DEV)
    qt = Q.quantize_groupwise(x, nbits, group_size)
    xh = Q.dequantize_groupwise(qt)
    step = qt.scale.float().repeat_interleave(group_size, dim=-1)
    err = (xh - x).abs()
    assert torch.all(err <= step / 2 + 1e-2 * step + 1e-6)


@pytest.mark.parametrize("nbits", Q.SUPPORTED_BITS)
def test_constant_group_is_exact(nbits):
    x = torch.full((2, 64), 3.5, device=DEV)
    qt = Q.quantize_groupwise(x, nbits, 32)
    xh = Q.dequantize_groupwise(qt)
    assert torch.allclose(xh, x, atol=1e-3)
    assert torch.isfinite(xh).all()
    assert torch.all(qt.scale == 1.0) and torch.all(qt.packed == 0)


def test_higher_bits_are_more_accurate_and_effective_bits():
    torch.manual_seed(2)
    x = torch.randn(8, 256, device=DEV)
    e2 = (Q.dequantize_groupwise(Q.quantize_groupwise(x, 2, 32)) - x).norm().item()
    e4 = (Q.dequantize_groupwise(Q.quantize_groupwise(x, 4, 32)) - x).norm().item()
    assert e4 < e2
    qt = Q.quantize_groupwise(x[:, :128].contiguous(), 4, 32)
    assert math.isclose(qt.effective_bits_per_element(), 5.0)
    assert qt.nbytes() * 8 / (8 * 128) == pytest.approx(5.0)
    r = Q.roundtrip_error(x, 4, 32)
    assert r["effective_bits"] == 5.0 and 0 < r["rel_l2"] < 0.2


def test_quantize_kv_full_size_round_trip_property():
    """Size-independent property at a full benchmark size (batch 4 of the
    Llama-3-8B shape, ctx 4096): pack(unpack(packed)) == packed, and
    re-quantising the dequantised cache reproduces codes, scale and zero."""
    torch.manual_seed(3)
    k = torch.randn(4, 8, 4096, 128, device=DEV, dtype=torch.float16)
    qt = Q.quantize_groupwise(k, 4, 32)
    codes = Q.unpack_codes(qt.packed, 4, 128)
    assert torch.equal(Q.pack_codes(codes, 4), qt.packed)
    assert int(codes.max()) <= 15
    # every group attains code 0 (its minimum) unless constant
    cg = codes.view(4, 8, 4096, 4, 32)
    assert torch.all(cg.amin(dim=-1) == 0)
    deq = Q.dequantize_groupwise(qt, torch.float32)
    step = qt.scale.float().repeat_interleave(32, dim=-1)
    assert torch.all((deq - k.float()).abs() <= step / 2 + 1e-2 * step + 1e-6)


# ---- appending tokens to a preallocated cache (no reference counterpart: the property
# ---- is that a cache filled step by step equals quantising the whole tensor at once)
@pytest.mark.parametrize("nbits", Q.SUPPORTED_BITS)
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
def test_append_equals_whole_tensor_quantisation(nbits, dtype):
    torch.manual_seed(5)
    B, HKV, S, D, gs = 3, 2, 37, 128, 32
    x = (torch.randn(B, HKV, S, D, device=DEV) * 1.7).to(dtype)
    whole = Q.quantize_groupwise(x, nbits, gs)
    cache = Q.empty_cache(B, HKV, S + 5, D, nbits, gs, DEV)
    # a prefill chunk, then single tokens, then a ragged tail through per-sequence positions
    Q.append_groupwise(cache, x[:, :, :16], 0)
    for t in range(16, 30):
        Q.append_groupwise(cache, x[:, :, t:t + 1], t)
    pos = torch.full((B,), 30, dtype=torch.int32, device=DEV)
    Q.append_groupwise(cache, x[:, :, 30:], pos)
    assert torch.equal(cache.packed[:, :, :S], whole.packed)
    assert torch.equal(cache.scale[:, :, :S].view(torch.int16), whole.scale.view(torch.int16))
    assert torch.equal(cache.zero[:, :, :S].view(torch.int16), whole.zero.view(torch.int16))
    assert int(cache.packed[:, :, S:].max()) == 0 and float(cache.scale[:, :, S:].abs().max()) == 0.0


def test_append_per_sequence_positions_and_decode():
    """Sequences of different lengths grow in one cache; decoding it with seq_lens equals
    decoding each sequence's own dense cache."""
    from tritonkv_b200.kernels import fused_decode_attention

    torch.manual_seed(6)
    B, HQ, HKV, D, gs, nbits, cap = 3, 8, 2, 128, 32, 4, 96
    lens = [17, 64, 41]
    k = torch.randn(B, HKV, cap, D, device=DEV, dtype=torch.float16)
    v = torch.randn(B, HKV, cap, D, device=DEV, dtype=torch.float16)
    q = torch.randn(B, HQ, D, device=DEV, dtype=torch.float16)
    kq = Q.empty_cache(B, HKV, cap, D, nbits, gs, DEV)
    vq = Q.empty_cache(B, HKV, cap, D, nbits, gs, DEV)
    pos = torch.zeros(B, dtype=torch.int32, device=DEV)
    for t in range(max(lens)):
        # every sequence appends its token t; finished sequences send theirs out of range
        p = torch.tensor([t if t < n else cap for n in lens], dtype=torch.int32, device=DEV)
        Q.append_kv(kq, vq, k[:, :, t:t + 1], v[:, :, t:t + 1], p)
    seq = torch.tensor(lens, dtype=torch.int32, device=DEV)
    got = fused_decode_attention(q, kq, vq, seq_lens=seq)
    for b, n in enumerate(lens):
        kb, vb = Q.quantize_kv(k[b:b + 1, :, :n].contiguous(), v[b:b + 1, :, :n].contiguous(), nbits, gs)
        assert torch.equal(kq.packed[b, :, :n], kb.packed[0])
        ref = fused_decode_attention(q[b:b + 1], kb, vb)
        assert torch.allclose(got[b], ref[0], atol=2e-5, rtol=1e-4)
        assert int(kq.packed[b, :, n:].max()) == 0  # dropped tokens wrote nothing


def test_append_argument_errors():
    cache = Q.empty_cache(2, 2, 8, 128, 4, 32, DEV)
    x = torch.randn(2, 2, 4, 128, device=DEV, dtype=torch.float16)
    with pytest.raises(ValueError):
        Q.append_groupwise(cache, x, 6)  # 6 + 4 > 8
    with pytest.raises(ValueError):
        Q.append_groupwise(cache, x[:, :1], 0)  # head mismatch
    with pytest.raises(ValueError):
        Q.append_groupwise(cache, x, torch.zeros(2, dtype=torch.int64, device=DEV))
    with pytest.raises(RuntimeError):
        Q.append_groupwise(cache, x.cpu(), 0)
