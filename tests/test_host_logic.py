"""Host-side mirror of the reference interface: geometry, containers, error behaviour.
No GPU needed."""

import math

import pytest
import torch

from oracle import tkv_oracle as O
from tritonkv_b200 import quantize as Q
from tritonkv_b200.kernels import _launch
from tritonkv_b200.kernels import fused_decode_attention, fp16_decode_attention, triton_available


@pytest.mark.parametrize("S,block_n,ns", [(4096, 64, 17), (3000, 128, 5), (1, 64, 8), (17, 64, 64),
                                          (16384, 32, 64), (2048, 64, 1), (8192, 16, 1000)])
def test_split_geometry_equals_oracle(S, block_n, ns):
    assert _launch.split_geometry(S, block_n, ns, 1, 2, None) == O.split_geometry(S, block_n, ns)


def test_split_geometry_properties():
    for S in (1, 16, 17, 100, 1000, 4097, 65536):
        for want in (1, 2, 3, 7, 64, 500):
            bn, ns, ss = _launch.split_geometry(S, 64, want, 1, 1, None)
            assert ss % 16 == 0 and ss % bn == 0
            assert ns * ss >= S > (ns - 1) * ss  # covers S, last split not empty


def test_pick_num_splits_rule():
    assert _launch.pick_num_splits(1, 2, 128, 592) == O.pick_num_splits(1, 2, 128, 592) == 128
    assert _launch.pick_num_splits(1, 2, 1024, 592) == 296
    assert _launch.pick_num_splits(64, 8, 64, 592) == 1
    assert _launch.pick_num_splits(1, 1, 5, 592) == 5


def test_quantized_tensor_container():
    qt = Q.QuantizedTensor(torch.zeros(2, 3, 64, dtype=torch.uint8),
                           torch.zeros(2, 3, 4, dtype=torch.float16),
                           torch.zeros(2, 3, 4, dtype=torch.float16), 4, 32, 128)
    assert qt.codes_per_byte == 2 and qt.n_groups == 4
    assert qt.batch_shape == (2, 3) and qt.shape == (2, 3, 128)
    assert math.isclose(qt.effective_bits_per_element(), 5.0)
    assert qt.nbytes() * 8 / (2 * 3 * 128) == pytest.approx(5.0)
    assert qt.contiguous().packed.is_contiguous()
    q2 = Q.QuantizedTensor(qt.packed[..., :32], qt.scale, qt.zero, 2, 32, 128)
    assert math.isclose(q2.effective_bits_per_element(), 3.0)


def test_quantizer_argument_errors_match_reference():
    x = torch.zeros(4, 128)
    with pytest.raises(ValueError, match="nbits must be one of"):
        Q.quantize_groupwise(x, 3, 32)
    with pytest.raises(ValueError, match="must divide head_dim"):
        Q.quantize_groupwise(x, 4, 48)
    with pytest.raises(ValueError, match="must divide head_dim"):
        Q.quantize_groupwise(torch.zeros(4, 64), 4, 128)
    with pytest.raises(TypeError, match="codes must be uint8"):
        Q.pack_codes(torch.zeros(4, 128, dtype=torch.int32), 4)
    with pytest.raises(ValueError, match="packed last dim"):
        Q.unpack_codes(torch.zeros(4, 60, dtype=torch.uint8), 4, 128)


def test_no_cpu_path():
    """CPU tensors are rejected loudly; nothing silently computes on the host."""
    if torch.cuda.is_available():
        pytest.skip("checks the behaviour of a box without a GPU")
    ok, why = triton_available()
    assert not ok and "cuda" in why.lower()
    with pytest.raises(RuntimeError, match="no CPU path"):
        Q.quantize_groupwise(torch.zeros(4, 128), 4, 32)
    with pytest.raises(RuntimeError, match="no CPU path"):
        Q.pack_codes(torch.zeros(4, 128, dtype=torch.uint8), 4)
    qt = Q.QuantizedTensor(torch.zeros(1, 2, 16, 64, dtype=torch.uint8),
                           torch.zeros(1, 2, 16, 4, dtype=torch.float16),
                           torch.zeros(1, 2, 16, 4, dtype=torch.float16), 4, 32, 128)
    with pytest.raises(RuntimeError, match="requires the CUDA library"):
        fused_decode_attention(torch.zeros(1, 12, 128), qt, qt)
    with pytest.raises(RuntimeError, match="requires the CUDA library"):
        fp16_decode_attention(torch.zeros(1, 12, 128), torch.zeros(1, 2, 16, 128),
                              torch.zeros(1, 2, 16, 128))


def test_product_never_imports_the_oracle():
    """The checker must not be reachable from the shipped package."""
    import os
    import re

    root = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "tritonkv_b200")
    for dirpath, _, files in os.walk(root):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh")):
                text = open(os.path.join(dirpath, f)).read()
                assert not re.search(r"^\s*(from|import)\s+oracle\b", text, flags=re.M), f
                assert "tkv_oracle" not in text, f


def test_ragged_batches_ask_for_one_split_up_to_the_device_schedule_limit():
    """Ragged batches are balanced by the kernel from seq_lens (one split requested) up to
    MAX_BALANCED_RAGGED_BATCH sequences; above it the static schedule gets a split count
    from the cost model."""
    lim = _launch.MAX_BALANCED_RAGGED_BATCH
    assert _launch.split_geometry(20000, 64, None, 16, 8, 444, ragged=True)[1] == 1
    assert _launch.split_geometry(20000, 64, None, lim, 8, 444, ragged=True)[1] == 1
    assert _launch.split_geometry(20000, 64, None, lim + 1, 1, 444, ragged=True)[1] >= 1
    # an explicit split count is always honoured
    assert _launch.split_geometry(20000, 64, 5, 16, 8, 444, ragged=True)[1] == 5


def test_peer_exchange_layout():
    from tritonkv_b200 import parallel as P

    wire = P.wire_floats(1, 64, 128)
    state_off, total = P.exchange_layout(8, wire)
    assert state_off == 2 * 8 * wire * 8          # two parities x world blocks of 8-byte pairs
    assert total >= state_off + 4 * (wire // 130) * (128 // 32)  # a step counter per (row, 32-dim slice)
    assert total % 16 == 0 and state_off % 16 == 0
    assert wire % 4 == 0 and wire >= 64 * (128 + 2)
