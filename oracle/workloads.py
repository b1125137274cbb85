"""Seeded synthetic inputs for the parity tests and the smoke check (test infrastructure,
like the rest of this directory: the shipped package never imports it).

The reference measures and tests on seeded synthetic tensors only (no dataset):
``make_random_kv`` restates its generator (reference.py:361-392: CPU ``torch.Generator``, fp32
``randn``, a fraction of entries multiplied by an outlier factor, draw order q, k, v, cast to
fp16), so that the CPU checker and the GPU kernels see the same bits.
"""

from __future__ import annotations

import torch

def make_random_kv(B: int, HQ: int, HKV: int, S: int, D: int, device="cuda",
                   dtype: torch.dtype = torch.float16, seed: int = 0,
                   outlier_frac: float = 0.01, outlier_scale: float = 8.0):
    """q (B, HQ, D), k and v (B, HKV, S, D): N(0,1) with ``outlier_frac`` of the
    entries scaled by ``outlier_scale``."""
    g = torch.Generator(device="cpu").manual_seed(seed)

    def _rand(*shape):
        x = torch.randn(*shape, generator=g, dtype=torch.float32)
        if outlier_frac > 0:
            m = torch.rand(*shape, generator=g) < outlier_frac
            x = torch.where(m, x * outlier_scale, x)
        return x.to(device=device, dtype=dtype)

    q = _rand(B, HQ, D)
    k = _rand(B, HKV, S, D)
    v = _rand(B, HKV, S, D)
    return q, k, v


def make_entry_outlier_k(B: int, HQ: int, HKV: int, S: int, D: int, device="cuda",
                         dtype: torch.dtype = torch.float16, seed: int = 0,
                         frac: float = 0.01, factor: float = 20.0):
    """N(0,1) q/k/v with ``frac`` of the K entries (only K) multiplied by ``factor``."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    q = torch.randn(B, HQ, D, generator=g, dtype=torch.float32)
    k = torch.randn(B, HKV, S, D, generator=g, dtype=torch.float32)
    v = torch.randn(B, HKV, S, D, generator=g, dtype=torch.float32)
    m = torch.rand(B, HKV, S, D, generator=g) < frac
    k = torch.where(m, k * factor, k)
    return tuple(t.to(device=device, dtype=dtype) for t in (q, k, v))


def ragged_seq_lens(B: int, lo: int, hi: int, seed: int = 0) -> torch.Tensor:
    """int32 (B,) lengths uniform in [lo, hi] from the seeded host generator."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    return torch.randint(lo, hi + 1, (B,), generator=g, dtype=torch.int64).to(torch.int32)
