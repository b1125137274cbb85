"""Seeded synthetic inputs for the decode-attention path.

The reference measures and tests on seeded synthetic tensors only (no dataset):
``make_random_kv`` below restates its generator (reference.py:361-392: CPU
``torch.Generator``, fp32 ``randn``, a fraction of entries multiplied by an
outlier factor, draw order q, k, v, cast to fp16), and the ``config*`` helpers
produce the value distributions of the benchmark configurations.  Everything is
generated on the host generator so that CPU checker and GPU kernels see the same
bits, then moved to ``device``.
"""

from __future__ import annotations

from dataclasses import dataclass

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


def make_channel_outlier_kv(B: int, HQ: int, HKV: int, S: int, D: int, device="cuda",
                            dtype: torch.dtype = torch.float16, seed: int = 0, sigma: float = 0.5):
    """N(0,1) q/k/v with K channels multiplied by per-channel lognormal(0, sigma)
    factors (outlier channels), the single-sequence sweep's distribution."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    q = torch.randn(B, HQ, D, generator=g, dtype=torch.float32)
    k = torch.randn(B, HKV, S, D, generator=g, dtype=torch.float32)
    v = torch.randn(B, HKV, S, D, generator=g, dtype=torch.float32)
    chan = torch.exp(sigma * torch.randn(HKV, D, generator=g, dtype=torch.float32))
    k = k * chan[None, :, None, :]
    return tuple(t.to(device=device, dtype=dtype) for t in (q, k, v))


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


@dataclass(frozen=True)
class Shape:
    name: str
    B: int
    HQ: int
    HKV: int
    D: int


QWEN25_1P5B = Shape("qwen2.5-1.5b", 1, 12, 2, 128)       # GQA 6
LLAMA3_8B_B64 = Shape("llama-3-8b", 64, 32, 8, 128)      # GQA 4, batch 64
LLAMA3_70B = Shape("llama-3-70b", 1, 64, 8, 128)         # GQA 8, long context


def cache_bytes_fused(B: int, HKV: int, tokens_total: int, D: int, nbits: int, gs: int) -> int:
    """Algorithmic bytes of one decode step on a packed cache: K+V codes and
    scale/zero of every cached token (``tokens_total`` = sum over the batch)."""
    return HKV * tokens_total * (2 * D * nbits // 8 + 8 * (D // gs))


def cache_bytes_fp16(B: int, HKV: int, tokens_total: int, D: int) -> int:
    return HKV * tokens_total * 4 * D
