"""The arithmetic the CUDA quantiser uses in place of the reference's per-element IEEE
division, restated in numpy and checked against the oracle's formula on the CPU
(``tritonkv_b200/csrc/tkv_quant.cu``; reference ``quantize.py:217-226``).

1. codes: ``u = sat((x - zero) * r)``, ``r = rcp(scale) / qmax``; ``m = fma(u, qmax, 1.5*2^23)``
   carries ``rint(u*qmax)`` in its low mantissa bits; elements whose ``u*qmax`` lies within 1e-4
   of a half-integer are redone with the division.  Must equal ``clip(rint((x-zero)/scale))``.
2. scale: ``d / qmax`` as ``q0 = d*R; q1 = fma(fma(-q0, qmax, d), R, q0)`` with ``R = fl(1/qmax)``.
   Must equal the IEEE quotient for every finite ``d``.
float64 holds every product and sum below exactly before the one rounding to float32, so the
numpy expressions are the fused operations of the kernel."""

import numpy as np
import pytest

f32 = np.float32
MAGIC = 12582912.0  # 1.5 * 2^23


def _kernel_codes(x16, zef, scf, nbits):
    qmax = float((1 << nbits) - 1)
    a = (x16.astype(f32) - zef).astype(f32)
    with np.errstate(all="ignore"):
        ref = np.clip(np.rint((a / scf).astype(f32)), 0, qmax)
        ref = np.where(np.isnan(ref), 0, ref)
        rs = ((f32(1) / scf).astype(f32) * f32(1.0 / qmax)).astype(f32)
        u = (a * rs).astype(f32)
        u = np.where(np.isnan(u), 0, np.clip(u, 0, 1)).astype(f32)
        m = (u.astype(np.float64) * qmax + MAGIC).astype(f32)
        t = (m - f32(MAGIC)).astype(f32)
        d = (u.astype(np.float64) * qmax - t.astype(np.float64)).astype(f32)
    tie = np.abs(d) > f32(0.4999)
    fast = (m.view(np.uint32) & 0xFF).astype(f32)
    return ref, np.where(tie, ref, fast), tie


def _groups(x16, nbits):
    xf = x16.astype(f32)
    qmax = f32((1 << nbits) - 1)
    with np.errstate(all="ignore"):
        mn, mx = xf.min(axis=1, keepdims=True), xf.max(axis=1, keepdims=True)
        sc = ((mx - mn) / qmax).astype(f32)
        sc = np.where(sc > 0, sc, f32(1))
    return mn.astype(np.float16).astype(f32), sc.astype(np.float16).astype(f32)


@pytest.mark.parametrize("nbits", [2, 4])
@pytest.mark.parametrize("kind", ["normal", "scaled", "bit_patterns", "offset"])
def test_codes_from_the_reciprocal_equal_the_division(nbits, kind):
    rng = np.random.default_rng(nbits * 7 + len(kind))
    n = 1 << 18
    if kind == "normal":
        x = rng.standard_normal(n).astype(np.float16)
    elif kind == "scaled":
        x = (rng.standard_normal(n) * 10.0 ** rng.uniform(-6, 4)).astype(np.float16)
    elif kind == "bit_patterns":
        x = rng.integers(0, 65536, n).astype(np.uint16).view(np.float16)
    else:
        x = (rng.standard_normal(n) * 0.01 + 100).astype(np.float16)
    x = x.reshape(-1, 32)
    zef, scf = _groups(x, nbits)
    ref, got, tie = _kernel_codes(x, zef, scf, nbits)
    assert np.array_equal(ref, got)
    assert tie.mean() < 0.05  # the redo stays rare (exact ties of fp16 data: about 7 in 10 000)


def test_exact_ties_are_caught():
    """x = zero + (k + 1/2) * scale exactly: the reciprocal path alone could round either way."""
    k = np.arange(0, 15, dtype=np.float32)
    x = ((k + 0.5) * f32(0.25)).astype(np.float16).reshape(1, -1)   # scale 0.25, zero 0
    ref, got, tie = _kernel_codes(x, f32(0.0), f32(0.25), 4)
    assert tie.all() and np.array_equal(ref, got)
    assert np.array_equal(ref[0], np.rint(k + 0.5))                 # ties to even, as torch.round


@pytest.mark.parametrize("qmax", [3.0, 15.0])
def test_division_by_qmax_through_two_fmas_is_the_ieee_quotient(qmax):
    rng = np.random.default_rng(int(qmax))
    R = f32(1.0 / qmax)
    f16 = np.arange(0x7C00, dtype=np.uint16).view(np.float16).astype(f32)       # every finite fp16 >= 0
    a = rng.integers(0, 0x7C00, 1 << 20).astype(np.uint16).view(np.float16).astype(f32)
    b = rng.integers(0, 0x7C00, 1 << 20).astype(np.uint16).view(np.float16).astype(f32)
    any32 = (np.abs(rng.standard_normal(1 << 20)) * 10.0 ** rng.uniform(-7, 5, 1 << 20)).astype(f32)
    for d in (f16, np.abs(a - b).astype(f32), (a + b).astype(f32), any32):
        q0 = (d * R).astype(f32)
        rem = (d.astype(np.float64) - q0.astype(np.float64) * qmax).astype(f32)
        q1 = (rem.astype(np.float64) * np.float64(R) + q0.astype(np.float64)).astype(f32)
        assert np.array_equal(q1.view(np.uint32), (d / f32(qmax)).astype(f32).view(np.uint32))
