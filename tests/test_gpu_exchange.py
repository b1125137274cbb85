"""The cross-GPU exchange kernels on ONE GPU, through the C ABI: a rank that talks to
itself must reproduce the plain combine, and a peer that never sends must run the bounded
wait out, leave a status bit and a usable context (no fault, no hang: the wait counts
its polls).  The multi-GPU path proper is in test_gpu_multi.py."""

import ctypes

import pytest
import torch

from tritonkv_b200 import _cabi
from tritonkv_b200 import parallel as P
from tritonkv_b200.kernels._launch import combine_splits

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _partials(rows_b, HQ, NS, D, seed):
    g = torch.Generator(device=DEV).manual_seed(seed)
    acc = torch.randn(rows_b, HQ, NS, D, device=DEV, generator=g)
    m = torch.randn(rows_b, HQ, NS, device=DEV, generator=g) * 3
    l = torch.rand(rows_b, HQ, NS, device=DEV, generator=g) + 0.5
    m[:, :, NS // 2] = float("-inf")  # an empty slot
    return acc, m, l


def _buffers(world, wire):
    state_off, total = P.exchange_layout(world, wire)
    bufs = [torch.zeros(total // 4, device=DEV, dtype=torch.float32) for _ in range(world)]
    table = (ctypes.c_void_p * world)(*[b.data_ptr() for b in bufs])
    return bufs, table, state_off


def test_exchange_with_itself_equals_plain_combine():
    B, HQ, NS, D = 2, 8, 37, 128
    wire = P.wire_floats(B, HQ, D)
    bufs, table, state_off = _buffers(1, wire)
    lib = _cabi.load()
    stream = _cabi.stream_ptr(torch.device("cuda", torch.cuda.current_device()))
    out = torch.empty(B, HQ, D, device=DEV)
    for step in range(5):  # both parities, counter carried on the device
        acc, m, l = _partials(B, HQ, NS, D, seed=step)
        _cabi.check(lib.tkv_combine_push(acc.data_ptr(), m.data_ptr(), l.data_ptr(), B * HQ, NS, D,
                                         NS * D, D, NS, 1, table, bufs[0].data_ptr() + state_off,
                                         1, 0, wire, stream))
        _cabi.check(lib.tkv_merge_wait(out.data_ptr(), B * HQ, D, table,
                                       bufs[0].data_ptr() + state_off, 1, 0, wire, stream))
        ref = combine_splits(acc, m, l)
        torch.cuda.synchronize()
        assert torch.allclose(out, ref, rtol=1e-5, atol=1e-6), step
    assert _cabi.device_status() == 0


def test_missing_peer_runs_the_wait_out_and_sets_the_status_bit():
    B, HQ, NS, D = 1, 8, 4, 64
    wire = P.wire_floats(B, HQ, D)
    bufs, table, state_off = _buffers(2, wire)  # "rank 1" exists as a buffer but never pushes
    lib = _cabi.load()
    stream = _cabi.stream_ptr(torch.device("cuda", torch.cuda.current_device()))
    acc, m, l = _partials(B, HQ, NS, D, seed=9)
    out = torch.empty(B, HQ, D, device=DEV)
    assert _cabi.device_status() == 0
    _cabi.check(lib.tkv_combine_push(acc.data_ptr(), m.data_ptr(), l.data_ptr(), B * HQ, NS, D,
                                     NS * D, D, NS, 1, table, bufs[0].data_ptr() + state_off,
                                     2, 0, wire, stream))
    _cabi.check(lib.tkv_merge_wait(out.data_ptr(), B * HQ, D, table, bufs[0].data_ptr() + state_off,
                                   2, 0, wire, stream))
    torch.cuda.synchronize()  # returns: the wait is bounded
    assert _cabi.device_status() & 2
    _cabi.device_status_clear()
    assert _cabi.device_status() == 0
    # the context is intact: an ordinary call still works
    ref = combine_splits(acc, m, l)
    assert torch.isfinite(ref).all()


def _fused(lib, acc, m, l, out, table, state, world, rank, wire, stream):
    B, HQ, NS, D = acc.shape
    _cabi.check(lib.tkv_combine_exchange(acc.data_ptr(), m.data_ptr(), l.data_ptr(), out.data_ptr(),
                                         B * HQ, NS, D, NS * D, D, NS, 1, table, state, world, rank,
                                         wire, stream))


def test_single_kernel_exchange_with_itself_equals_plain_combine():
    """The one-kernel form (merge, push, wait, merge) over several steps, alternating with the
    two-kernel form on the same buffers: the step counter and both parities carry over."""
    B, HQ, NS, D = 2, 8, 37, 128
    wire = P.wire_floats(B, HQ, D)
    bufs, table, state_off = _buffers(1, wire)
    lib = _cabi.load()
    stream = _cabi.stream_ptr(torch.device("cuda", torch.cuda.current_device()))
    state = bufs[0].data_ptr() + state_off
    out = torch.empty(B, HQ, D, device=DEV)
    for step in range(6):
        acc, m, l = _partials(B, HQ, NS, D, seed=20 + step)
        if step % 3 == 2:
            _cabi.check(lib.tkv_combine_push(acc.data_ptr(), m.data_ptr(), l.data_ptr(), B * HQ, NS, D,
                                             NS * D, D, NS, 1, table, state, 1, 0, wire, stream))
            _cabi.check(lib.tkv_merge_wait(out.data_ptr(), B * HQ, D, table, state, 1, 0, wire, stream))
        else:
            _fused(lib, acc, m, l, out, table, state, 1, 0, wire, stream)
        ref = combine_splits(acc, m, l)
        torch.cuda.synchronize()
        assert torch.allclose(out, ref, rtol=1e-5, atol=1e-6), step
    assert _cabi.device_status() == 0


def test_single_kernel_exchange_two_ranks_emulated_in_turn():
    """Two "ranks" on one GPU, run one after the other: rank 0's kernel finds rank 1's block
    empty and would wait, so rank 1 pushes first with the two-kernel form's push, then rank 0
    runs the one-kernel form and must merge both contributions."""
    B, HQ, NS, D = 1, 8, 5, 128
    wire = P.wire_floats(B, HQ, D)
    bufs, table, state_off = _buffers(2, wire)
    lib = _cabi.load()
    stream = _cabi.stream_ptr(torch.device("cuda", torch.cuda.current_device()))
    a0, m0, l0 = _partials(B, HQ, NS, D, seed=31)
    a1, m1, l1 = _partials(B, HQ, NS, D, seed=32)
    out = torch.empty(B, HQ, D, device=DEV)
    _cabi.check(lib.tkv_combine_push(a1.data_ptr(), m1.data_ptr(), l1.data_ptr(), B * HQ, NS, D,
                                     NS * D, D, NS, 1, table, bufs[1].data_ptr() + state_off, 2, 1,
                                     wire, stream))
    _fused(lib, a0, m0, l0, out, table, bufs[0].data_ptr() + state_off, 2, 0, wire, stream)
    ref = combine_splits(torch.cat([a0, a1], dim=2), torch.cat([m0, m1], dim=2),
                         torch.cat([l0, l1], dim=2))
    torch.cuda.synchronize()
    assert torch.allclose(out, ref, rtol=1e-5, atol=1e-6)
    assert _cabi.device_status() == 0


def test_single_kernel_exchange_missing_peer_runs_the_wait_out():
    B, HQ, NS, D = 1, 8, 4, 64
    wire = P.wire_floats(B, HQ, D)
    bufs, table, state_off = _buffers(2, wire)  # "rank 1" never pushes
    lib = _cabi.load()
    stream = _cabi.stream_ptr(torch.device("cuda", torch.cuda.current_device()))
    acc, m, l = _partials(B, HQ, NS, D, seed=33)
    out = torch.empty(B, HQ, D, device=DEV)
    assert _cabi.device_status() == 0
    _fused(lib, acc, m, l, out, table, bufs[0].data_ptr() + state_off, 2, 0, wire, stream)
    torch.cuda.synchronize()  # returns: the wait is bounded
    assert _cabi.device_status() & 2
    _cabi.device_status_clear()
    assert _cabi.device_status() == 0
    assert torch.isfinite(combine_splits(acc, m, l)).all()  # the context is intact


def test_exchange_argument_errors():
    lib = _cabi.load()
    t = torch.zeros(64, device=DEV)
    table = (ctypes.c_void_p * 1)(t.data_ptr())
    with pytest.raises(ValueError):  # more ranks than the kernels serve
        _cabi.check(lib.tkv_merge_wait(t.data_ptr(), 1, 32, table, t.data_ptr(), 9, 0, 64, None))
    with pytest.raises(ValueError):  # a block too small for the rows
        _cabi.check(lib.tkv_merge_wait(t.data_ptr(), 8, 32, table, t.data_ptr(), 1, 0, 16, None))
