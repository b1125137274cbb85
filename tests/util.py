"""Helpers shared by the GPU parity tests: torch <-> numpy glue for the oracle."""

import numpy as np
import torch

from oracle import tkv_oracle as O

# Fused/fp16 kernel vs fp32 dequantise-then-attend on identical values
# (test_correctness.py:51-52 of the reference) ...
KERNEL_COSINE_MIN = 0.99999
KERNEL_REL_L2_MAX = 5e-3
# ... and the elementwise bound the target states: |got-ref| <= 2e-3 + 1e-2*|ref|.
ATOL, RTOL = 2e-3, 1e-2


def to_oracle(qt) -> O.OracleQuantized:
    return O.OracleQuantized(qt.packed.cpu().numpy(), qt.scale.cpu().numpy(), qt.zero.cpu().numpy(),
                             qt.nbits, qt.group_size, qt.head_dim)


def oracle_attention(q, kq, vq, sm_scale=None, seq_lens=None) -> np.ndarray:
    sl = None if seq_lens is None else seq_lens.cpu().numpy()
    return O.reference_on_quantized(q.float().cpu().numpy(), to_oracle(kq), to_oracle(vq),
                                    sm_scale, sl)


def assert_close(got: torch.Tensor, ref: np.ndarray, what=""):
    rep = O.allclose_report(got.float().cpu().numpy(), ref, ATOL, RTOL)
    assert rep["ok"], f"{what}: {rep}"
    assert rep["cosine"] >= KERNEL_COSINE_MIN, f"{what}: {rep}"
    assert rep["rel_l2"] <= KERNEL_REL_L2_MAX, f"{what}: {rep}"
    return rep


def c_oracle_attention(q, kq, vq, seq_lens=None, rows=None) -> np.ndarray:
    """The oracle's C twin (same arithmetic, OpenMP) for cases too large for numpy; ``rows``
    selects the sequences to compute (all if None)."""
    from oracle import c_oracle

    idx = torch.arange(q.shape[0]) if rows is None else torch.as_tensor(list(rows))
    it = idx.to(q.device)
    h = lambda t: t.index_select(0, it).cpu().numpy()
    hm = lambda t: h(t).view(np.uint16)
    sl = None if seq_lens is None else seq_lens.cpu().index_select(0, idx).numpy()
    return c_oracle.decode_step(h(q.float()), h(kq.packed), hm(kq.scale), hm(kq.zero), h(vq.packed),
                                hm(vq.scale), hm(vq.zero), kq.nbits, kq.group_size, seq_lens=sl)
