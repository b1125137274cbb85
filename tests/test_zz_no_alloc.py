"""The allocation-free decode entry point against the regular one.

``tkv_fused_decode_static`` serves callers that have no way to allocate the split
partials (a frozen memory pool, a capture region, a host that owns all device memory):
it keeps them in a fixed array inside the library.  Here it is called through the C ABI
twice in a row -- the array is shared and keeps the previous call's contents, so the
second call on a different problem shape must not be disturbed by the first.  Both entry
points plan the same split (one split over the whole history) and run the same kernels,
so the results must be identical bit for bit, which is stricter than the tolerance of the
other decode tests; one case is also compared with the CPU oracle within that tolerance.
This file sorts last on purpose: a run that stops at the first failure has then already
run everything else.
"""

import math

import pytest
import torch

from tritonkv_b200 import _cabi
from tritonkv_b200 import quantize as Q
from tritonkv_b200.kernels import fused_decode_attention
from oracle.workloads import make_random_kv

from util import assert_close, oracle_attention

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _static_decode(q, kq, vq):
    B, HQ, D = q.shape
    _, HKV, S, _ = kq.packed.shape
    out = torch.empty(B, HQ, D, device=q.device, dtype=torch.float32)
    lib = _cabi.load()
    with torch.cuda.device(q.device):
        _cabi.check(lib.tkv_fused_decode_static(
            q.data_ptr(), _cabi.dtype_code(q), kq.packed.data_ptr(), kq.scale.data_ptr(),
            kq.zero.data_ptr(), vq.packed.data_ptr(), vq.scale.data_ptr(), vq.zero.data_ptr(),
            out.data_ptr(), B, HQ, HKV, S, D, kq.nbits, kq.group_size, 1.0 / math.sqrt(D),
            _cabi.stream_ptr(q.device)))
    return out


def test_static_entry_matches_regular_entry_twice_in_a_row():
    cases = [(2, 32, 8, 3000, 128, 4, 32, 100), (1, 12, 2, 8192, 128, 2, 32, 101)]
    for B, HQ, HKV, S, D, nbits, gs, seed in cases:
        q, k, v = make_random_kv(B, HQ, HKV, S, D, device=DEV, seed=seed)
        kq, vq = Q.quantize_kv(k, v, nbits, gs)
        want = fused_decode_attention(q, kq, vq)
        got = _static_decode(q, kq, vq)
        assert torch.equal(got, want), f"static entry differs from the regular entry, seed={seed}"
        if seed == 100:
            assert_close(got, oracle_attention(q, kq, vq), "static entry against the oracle")
    # same shape again after a different one used the array in between
    B, HQ, HKV, S, D, nbits, gs, seed = cases[0]
    q, k, v = make_random_kv(B, HQ, HKV, S, D, device=DEV, seed=seed)
    kq, vq = Q.quantize_kv(k, v, nbits, gs)
    assert torch.equal(_static_decode(q, kq, vq), fused_decode_attention(q, kq, vq)), "repeated"


def test_static_entry_single_slot_plan():
    """A history of one tile plans a single partial slot: the scratch array is not touched,
    the output comes straight from the split kernel, and the call still succeeds as a
    first (set-up) call on the device."""
    q, k, v = make_random_kv(1, 12, 2, 17, 128, device=DEV, seed=103)
    kq, vq = Q.quantize_kv(k, v, 4, 32)
    got = _static_decode(q, kq, vq)
    assert torch.equal(got, fused_decode_attention(q, kq, vq))
    assert_close(got, oracle_attention(q, kq, vq), "static entry, one slot")


def test_static_entry_rejects_oversized_problems():
    q, k, v = make_random_kv(128, 64, 8, 64, 128, device=DEV, seed=102)
    kq, vq = Q.quantize_kv(k, v, 4, 32)
    # 128 x 64 heads x 2 slots x 130 floats = 2.13 M floats > 8 MiB of partials
    with pytest.raises(ValueError, match="built-in scratch"):
        _static_decode(q, kq, vq)
