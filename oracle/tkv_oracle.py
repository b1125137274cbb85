"""CPU oracle for the packed-KV decode-attention path (TEST INFRASTRUCTURE ONLY).

This module is a numpy restatement of the reference project's CPU arithmetic for
the one path this library replaces.  It is the *checker*: tests, the smoke entry
and the benchmark's CPU-baseline leg import it; the product package never does.

Parity status: PINNED.  Every function here is checked against outputs of the
reference's own Python implementation (quantize.py / reference.py /
kernels/fused_decode_attn.py run on CPU) stored as fixtures under
``tests/golden/`` together with the script that produced them, and against the
two hand-derivable byte vectors of the split-P packing.

Reference citations (paths inside the reference project):

* ``pack_codes``            quantize.py:149-169
* ``unpack_codes``          quantize.py:172-183
* ``quantize_groupwise``    quantize.py:186-236
* ``dequantize_groupwise``  quantize.py:239-246
* ``reference_decode_attention``  reference.py:61-88
* ``reference_grouped``     l2_sweep.py:196-236 (memory-frugal twin of the above)
* ``split_partials``        kernels/fused_decode_attn.py:209-353 (the (acc, m, l)
  partial format in the exp2 domain) and ``split_geometry`` :487-499
* ``combine_splits``        kernels/fused_decode_attn.py:355-395
* ``pick_num_splits``       kernels/fused_decode_attn.py:402-416

Bit-exactness notes.  All quantiser arithmetic is IEEE float32 with one rounding
per operation, exactly as torch's CPU elementwise kernels do it; ``np.rint`` and
``torch.round`` both round half to even; ``astype(np.float16)`` and
``Tensor.half()`` both round to nearest even.  Attention is float32 with
whatever summation order numpy picks, so it is compared with a tolerance
(1e-5 relative to the output scale), not bit for bit.
"""

from __future__ import annotations

import math
from dataclasses import dataclass

import numpy as np

SUPPORTED_BITS = (2, 4)
LOG2E = 1.4426950408889634


def _check_bits(nbits: int) -> None:
    if nbits not in SUPPORTED_BITS:
        raise ValueError(f"nbits must be one of {SUPPORTED_BITS}, got {nbits}")


@dataclass
class OracleQuantized:
    """numpy twin of the reference's QuantizedTensor (quantize.py:73-146)."""

    packed: np.ndarray  # uint8  (*batch, D // P)
    scale: np.ndarray   # float16 (*batch, D // group_size)
    zero: np.ndarray    # float16 (*batch, D // group_size)
    nbits: int
    group_size: int
    head_dim: int

    def nbytes(self) -> int:
        return self.packed.nbytes + self.scale.nbytes + self.zero.nbytes

    def effective_bits_per_element(self) -> float:
        return self.nbits + 32.0 / self.group_size


# --------------------------------------------------------------------------
# split-P packing (quantize.py:149-183)
# --------------------------------------------------------------------------


def pack_codes(codes: np.ndarray, nbits: int) -> np.ndarray:
    """``packed[..., j] = OR_p codes[..., j + p*DP] << (p*nbits)``."""
    _check_bits(nbits)
    if codes.dtype != np.uint8:
        raise TypeError(f"codes must be uint8, got {codes.dtype}")
    P = 8 // nbits
    D = codes.shape[-1]
    if D % P != 0:
        raise ValueError(f"head_dim {D} must be divisible by {P} for {nbits}-bit packing")
    chunks = codes.reshape(*codes.shape[:-1], P, D // P)
    packed = np.zeros(chunks.shape[:-2] + chunks.shape[-1:], dtype=np.uint8)
    for p in range(P):
        # uint8 shift wraps modulo 256 exactly like torch's uint8 ``<<``.
        packed |= (chunks[..., p, :].astype(np.uint16) << (p * nbits)).astype(np.uint8)
    return packed


def unpack_codes(packed: np.ndarray, nbits: int, head_dim: int) -> np.ndarray:
    _check_bits(nbits)
    P = 8 // nbits
    DP = head_dim // P
    if packed.shape[-1] != DP:
        raise ValueError(f"packed last dim {packed.shape[-1]} != head_dim//P = {DP}")
    mask = (1 << nbits) - 1
    parts = [((packed >> (p * nbits)) & mask).astype(np.uint8) for p in range(P)]
    return np.ascontiguousarray(np.concatenate(parts, axis=-1))


# --------------------------------------------------------------------------
# group-wise quantiser (quantize.py:186-246)
# --------------------------------------------------------------------------


def quantize_groupwise(x: np.ndarray, nbits: int, group_size: int) -> OracleQuantized:
    _check_bits(nbits)
    D = x.shape[-1]
    if group_size <= 0 or D % group_size != 0:
        raise ValueError(f"group_size {group_size} must divide head_dim {D}")
    P = 8 // nbits
    if D % P != 0:
        raise ValueError(f"head_dim {D} must be divisible by {P} for {nbits}-bit packing")
    qmax = np.float32((1 << nbits) - 1)
    ng = D // group_size

    xg = x.reshape(*x.shape[:-1], ng, group_size).astype(np.float32)
    gmin = xg.min(axis=-1)
    gmax = xg.max(axis=-1)
    with np.errstate(all="ignore"):
        scale = ((gmax - gmin) / qmax).astype(np.float32)
        scale = np.where(scale > 0, scale, np.float32(1.0)).astype(np.float32)
        scale16 = scale.astype(np.float16)
        zero16 = gmin.astype(np.float16)
        scale_f = scale16.astype(np.float32)
        zero_f = zero16.astype(np.float32)
        t = ((xg - zero_f[..., None]).astype(np.float32) / scale_f[..., None]).astype(np.float32)
        codes = np.clip(np.rint(t), 0.0, float(qmax))
        codes = np.nan_to_num(codes, nan=0.0).astype(np.uint8)
    codes = codes.reshape(*x.shape[:-1], D)
    return OracleQuantized(pack_codes(codes, nbits), scale16, zero16, nbits, group_size, D)


def dequantize_groupwise(qt: OracleQuantized, dtype=np.float32) -> np.ndarray:
    codes = unpack_codes(qt.packed, qt.nbits, qt.head_dim)
    ng = qt.head_dim // qt.group_size
    cg = codes.reshape(*codes.shape[:-1], ng, qt.group_size).astype(np.float32)
    out = cg * qt.scale.astype(np.float32)[..., None] + qt.zero.astype(np.float32)[..., None]
    return out.reshape(*codes.shape[:-1], qt.head_dim).astype(dtype)


def quantize_kv(k, v, nbits, group_size):
    return quantize_groupwise(k, nbits, group_size), quantize_groupwise(v, nbits, group_size)


# --------------------------------------------------------------------------
# ground-truth attention (reference.py:61-88, l2_sweep.py:196-236)
# --------------------------------------------------------------------------


def reference_decode_attention(q, k, v, sm_scale=None, seq_lens=None) -> np.ndarray:
    """fp32 softmax(q K^T * sm_scale) V for one query row per head.

    q (B, HQ, D); k, v (B, HKV, S, D); returns (B, HQ, D) float32.  The query is
    grouped as (B, HKV, G, D) so K/V are never expanded -- the arithmetic is the
    reference's, the layout is its memory-frugal twin's.  ``seq_lens`` (B,) limits
    each sequence's history to its first ``seq_lens[b]`` tokens; it has no
    reference counterpart and equals slicing the cache per sequence.
    """
    B, HQ, D = q.shape
    _, HKV, S, _ = k.shape
    assert HQ % HKV == 0
    G = HQ // HKV
    sm_scale = 1.0 / math.sqrt(D) if sm_scale is None else sm_scale
    qg = q.astype(np.float32).reshape(B, HKV, G, D)
    out = np.zeros((B, HKV, G, D), dtype=np.float32)
    for b in range(B):
        n = S if seq_lens is None else int(seq_lens[b])
        if n == 0:
            continue
        kf = k[b, :, :n].astype(np.float32)
        vf = v[b, :, :n].astype(np.float32)
        scores = np.einsum("hgd,hsd->hgs", qg[b], kf, optimize=True) * np.float32(sm_scale)
        scores = scores - scores.max(axis=-1, keepdims=True)
        e = np.exp(scores, dtype=np.float32)
        probs = e / e.sum(axis=-1, keepdims=True, dtype=np.float32)
        out[b] = np.einsum("hgs,hsd->hgd", probs, vf, optimize=True)
    return out.reshape(B, HQ, D)


def reference_on_quantized(q, kq: OracleQuantized, vq: OracleQuantized, sm_scale=None,
                           seq_lens=None) -> np.ndarray:
    """Dequantise in fp32, then attend: the comparison every kernel test makes."""
    return reference_decode_attention(
        q, dequantize_groupwise(kq), dequantize_groupwise(vq), sm_scale, seq_lens
    )


# --------------------------------------------------------------------------
# flash-decoding split geometry and partial format
# --------------------------------------------------------------------------


def next_pow2(x: int) -> int:
    return 1 << (x - 1).bit_length()


def pick_num_splits(B: int, HKV: int, n_blocks: int, target_programs: int) -> int:
    want = max(1, target_programs // max(1, B * HKV))
    return max(1, min(n_blocks, want))


def split_geometry(S: int, block_n: int, num_splits: int):
    """(block_n, num_splits, split_size) after the reference's clamping
    (kernels/fused_decode_attn.py:487-499): no empty splits."""
    block_n = min(block_n, max(16, next_pow2(S)))
    n_blocks = -(-S // block_n)
    num_splits = max(1, min(num_splits, n_blocks))
    bps = -(-n_blocks // num_splits)
    num_splits = -(-n_blocks // bps)
    return block_n, num_splits, bps * block_n


def split_partials(q, k, v, split_size: int, num_splits: int, sm_scale=None):
    """Per-split unnormalised partials in the exp2 domain.

    acc (B, HQ, NS, D) = sum_n 2^(s_n - m) v_n,  m (B, HQ, NS) = max_n s_n with
    s_n = (q.k_n) * sm_scale * log2(e),  l (B, HQ, NS) = sum_n 2^(s_n - m).
    """
    B, HQ, D = q.shape
    _, HKV, S, _ = k.shape
    G = HQ // HKV
    sm_scale = 1.0 / math.sqrt(D) if sm_scale is None else sm_scale
    c = np.float32(sm_scale * LOG2E)
    qg = q.astype(np.float32).reshape(B, HKV, G, D)
    acc = np.zeros((B, HQ, num_splits, D), np.float32)
    m = np.full((B, HQ, num_splits), -np.inf, np.float32)
    l = np.zeros((B, HQ, num_splits), np.float32)
    for s in range(num_splits):
        lo, hi = s * split_size, min(S, (s + 1) * split_size)
        if lo >= hi:
            continue
        kf = k[:, :, lo:hi].astype(np.float32)
        vf = v[:, :, lo:hi].astype(np.float32)
        sc = np.einsum("bhgd,bhsd->bhgs", qg, kf, optimize=True) * c
        ms = sc.max(axis=-1)
        p = np.exp2(sc - ms[..., None]).astype(np.float32)
        acc[:, :, s] = np.einsum("bhgs,bhsd->bhgd", p, vf, optimize=True).reshape(B, HQ, D)
        m[:, :, s] = ms.reshape(B, HQ)
        l[:, :, s] = p.sum(axis=-1, dtype=np.float32).reshape(B, HQ)
    return acc, m, l


def combine_splits(acc, m, l) -> np.ndarray:
    """Sequential log-sum-exp merge over the split axis, exactly the loop of
    kernels/fused_decode_attn.py:380-395 (exp2 domain), extended with the
    empty-split guard (m = -inf, l = 0 contributes nothing)."""
    B, HQ, NS, D = acc.shape
    a = np.zeros((B, HQ, D), np.float32)
    mg = np.full((B, HQ), -np.inf, np.float32)
    lg = np.zeros((B, HQ), np.float32)
    with np.errstate(invalid="ignore"):
        for s in range(NS):
            ms, ls = m[:, :, s], l[:, :, s]
            mn = np.maximum(mg, ms)
            alpha = np.where(np.isneginf(mn), np.float32(0), np.exp2(mg - mn)).astype(np.float32)
            beta = np.where(np.isneginf(mn), np.float32(0), np.exp2(ms - mn)).astype(np.float32)
            a = a * alpha[..., None] + acc[:, :, s] * beta[..., None]
            lg = lg * alpha + ls * beta
            mg = mn
        out = a / lg[..., None]
    return np.where(lg[..., None] > 0, out, np.float32(0)).astype(np.float32)


# --------------------------------------------------------------------------
# seeded inputs (reference.py:361-392 and the benchmark configurations)
# --------------------------------------------------------------------------


def allclose_report(got, ref, atol=2e-3, rtol=1e-2) -> dict:
    """|got - ref| <= atol + rtol*|ref| plus the reference suite's own metrics
    (test_correctness.py:59-67)."""
    g = np.asarray(got, np.float64).ravel()
    r = np.asarray(ref, np.float64).ravel()
    err = np.abs(g - r)
    denom = max(np.linalg.norm(r), 1e-12)
    cos = float(g @ r / max(np.linalg.norm(g) * np.linalg.norm(r), 1e-30))
    return {
        "ok": bool(np.all(err <= atol + rtol * np.abs(r))),
        "max_abs_err": float(err.max()) if err.size else 0.0,
        "rel_l2": float(np.linalg.norm(g - r) / denom),
        "cosine": cos,
        "worst_excess": float((err - (atol + rtol * np.abs(r))).max()) if err.size else 0.0,
    }
