"""Per-channel key quantisation with an fp16 residual window on the GPU, against
``oracle/kivi_oracle.py``.  PARITY UNPINNED for this format: the reference describes it as
future work (docs/future_work.md:229-293) and ships no implementation, so the oracle is a
specification written here; what IS pinned is its per-element arithmetic (the reference
quantiser's, see tests/test_oracle_kivi.py).  Bit-exact for the quantiser,
|got-ref| <= 2e-3 + 1e-2*|ref| plus the reference's cosine / rel-L2 thresholds for attention."""

import numpy as np
import pytest
import torch

from oracle import kivi_oracle as KO
from oracle import tkv_oracle as O
from tritonkv_b200 import quantize as Q
from tritonkv_b200.kernels import (KiviCache, fused_decode_attention, kivi_decode_attention,
                                   quantize_kv_kivi)

from util import assert_close, to_oracle

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _kv(B, HQ, HKV, S, D, seed, channel_outliers=True):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(B, HQ, D, generator=g)
    k = torch.randn(B, HKV, S, D, generator=g)
    v = torch.randn(B, HKV, S, D, generator=g)
    if channel_outliers:  # dimensions that are large for every token (what real keys look like)
        idx = torch.randperm(D, generator=g)[:max(2, D // 32)]
        k[..., idx] *= 10.0
    return q.half().to(DEV), k.half().to(DEV), v.half().to(DEV)


def _oracle(q, cache: KiviCache):
    kc = KO.ChannelKeys(cache.k.packed.cpu().numpy(), cache.k.scale.cpu().numpy(),
                        cache.k.zero.cpu().numpy(), cache.k.nbits, 32, cache.k.head_dim)
    return KO.reference_attention(q.float().cpu().numpy(), kc, to_oracle(cache.v),
                                  cache.k_res.float().cpu().numpy(), cache.v_res.float().cpu().numpy())


@pytest.mark.parametrize("dtype", [torch.float16, torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nbits", [2, 4])
@pytest.mark.parametrize("D,S", [(128, 100), (64, 64), (128, 31), (256, 40)])
def test_quantiser_bit_exact_against_the_oracle(dtype, nbits, D, S):
    g = torch.Generator().manual_seed(D + S + nbits)
    k = torch.randn(2, 3, S, D, generator=g)
    k[..., 5] *= 30.0
    k[0, 0, :32, 7] = 1.25      # a constant group
    k = k.to(dtype)
    kc, res = Q.quantize_keys_per_channel(k.to(DEV), nbits)
    ref, ref_res = KO.quantize_keys_per_channel(k.float().numpy(), nbits, 32)
    assert kc.packed.shape == ref.packed.shape and res.shape == ref_res.shape
    assert np.array_equal(kc.packed.cpu().numpy(), ref.packed)
    assert np.array_equal(kc.scale.cpu().numpy().view(np.uint16), ref.scale.view(np.uint16))
    assert np.array_equal(kc.zero.cpu().numpy().view(np.uint16), ref.zero.view(np.uint16))
    assert np.array_equal(res.cpu().numpy().view(np.uint16), ref_res.view(np.uint16))
    if S >= 32:
        deq = Q.dequantize_keys_per_channel(kc).cpu().numpy()
        assert np.array_equal(deq, KO.dequantize_keys_per_channel(ref))


@pytest.mark.parametrize("B,HQ,HKV,S,D,nbits", [
    (1, 12, 2, 2048 + 17, 128, 4),   # long units, fp16 tail of 17 tokens
    (1, 12, 2, 4096, 128, 2),        # no tail
    (2, 32, 8, 1000, 128, 2),
    (64, 32, 8, 160, 128, 4),        # balanced dense schedule across many units
    (3, 8, 8, 333, 64, 4),           # head_dim 64, no GQA sharing
    (2, 24, 2, 96 + 5, 64, 2),       # GQA 12: two head chunks
    (1, 12, 2, 20, 128, 4),          # shorter than one group: the fp16 tail only
    (1, 64, 8, 32, 128, 2),          # exactly one group
])
def test_decode_matches_the_oracle(B, HQ, HKV, S, D, nbits):
    q, k, v = _kv(B, HQ, HKV, S, D, seed=S + D + nbits)
    cache = quantize_kv_kivi(k, v, nbits)
    assert cache.tokens == S and cache.k_res.shape[2] == S % 32
    got = kivi_decode_attention(q, cache)
    assert_close(got, _oracle(q, cache), f"{(B, HQ, HKV, S, D, nbits)}")
    ws: dict = {}
    out = torch.empty_like(got)
    again = kivi_decode_attention(q, cache, out=out, _workspace=ws)
    assert again is out and torch.equal(out, got)
    assert torch.equal(kivi_decode_attention(q, cache, out=out, _workspace=ws), got)  # buffers reused


def test_two_bit_keys_become_usable_on_outlier_channels():
    """What the format is for: with channels that are large for every token, 2-bit per-token
    keys wreck the attention output and 2-bit per-channel keys do not."""
    B, HQ, HKV, S, D = 1, 12, 2, 4096, 128
    q, k, v = _kv(B, HQ, HKV, S, D, seed=77)
    ref = O.reference_decode_attention(q.float().cpu().numpy(), k.float().cpu().numpy(),
                                       v.float().cpu().numpy())
    got_c = kivi_decode_attention(q, quantize_kv_kivi(k, v, 2)).cpu().numpy()
    kq, vq = Q.quantize_kv(k, v, 2, 32)
    got_t = fused_decode_attention(q, kq, vq).cpu().numpy()
    err = lambda a: float(np.linalg.norm(a - ref) / np.linalg.norm(ref))
    assert err(got_c) < 0.7 * err(got_t), (err(got_c), err(got_t))


def test_argument_errors():
    q, k, v = _kv(1, 12, 2, 64, 128, seed=1)
    cache = quantize_kv_kivi(k, v, 4)
    with pytest.raises(ValueError):
        kivi_decode_attention(q[:, :11], cache)            # HQ not a multiple of HKV
    bad = KiviCache(cache.k, Q.quantize_groupwise(v, 4, 64), cache.k_res, cache.v_res)
    with pytest.raises(ValueError, match="group_size 32"):
        kivi_decode_attention(q, bad)
    with pytest.raises(ValueError):
        Q.quantize_keys_per_channel(k[0], 4)               # not (B, HKV, S, D)
    with pytest.raises(ValueError, match="shorter than 16"):
        Q.quantize_keys_per_channel(k[..., :32].contiguous(), 2)   # packed rows of 8 bytes
    kc, _ = Q.quantize_keys_per_channel(k[..., :32].contiguous(), 4)  # 16-byte rows: the smallest
    assert kc.packed.shape == (1, 2, 64, 16)
