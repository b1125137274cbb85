"""CPU oracle for per-channel key quantisation with an fp16 residual window (TEST
INFRASTRUCTURE ONLY).

PARITY UNPINNED.  The reference project describes this format as future work
(docs/future_work.md:229-293: "make 2-bit usable: per-channel keys, the KIVI idea") and
ships no implementation, no test and no golden vector of it.  This module is therefore a
specification written here, not a restatement of reference code:

* the per-element arithmetic is the reference quantiser's (quantize.py:186-236: fp32 min/max
  of a group, ``scale = (max - min) / qmax`` (1 where not > 0), scale and zero rounded to fp16
  BEFORE coding, ``code = clamp(rint((x - zero16) / scale16), 0, qmax)``), which IS pinned by
  ``tests/golden`` through ``tkv_oracle.quantize_groupwise``;
* only the grouping axis differs: a key group is ``group_tokens`` consecutive tokens of ONE
  head dimension (future_work.md:252-256: "key metadata becomes one row per tile"), so scale
  and zero have shape ``(B, HKV, S_q / group_tokens, D)``;
* the byte layout of the codes stays split-P along the head dimension (future_work.md:263-266
  leaves the choice open; keeping it lets the decode kernel reuse its code path);
* the last ``S mod group_tokens`` tokens -- a group that is not full yet -- stay in fp16
  (the "residual window", future_work.md:246-248), keys and values alike; values of the
  quantised part stay per-token as today (future_work.md:257).

What anchors it: the round trip bound of the pinned quantiser (half a step per element)
holds per channel group, and attention on the dequantised cache is the pinned
``tkv_oracle.reference_decode_attention``.
"""

from __future__ import annotations

from dataclasses import dataclass

import numpy as np

from . import tkv_oracle as O


@dataclass
class ChannelKeys:
    """Keys quantised per channel over groups of ``group_tokens`` tokens."""

    packed: np.ndarray   # uint8   (B, HKV, S_q, D // P), split-P along D
    scale: np.ndarray    # float16 (B, HKV, S_q // group_tokens, D)
    zero: np.ndarray     # float16 (B, HKV, S_q // group_tokens, D)
    nbits: int
    group_tokens: int
    head_dim: int


def quantize_keys_per_channel(k: np.ndarray, nbits: int, group_tokens: int = 32):
    """k (B, HKV, S, D) -> (ChannelKeys over the first S_q = S - S % group_tokens tokens,
    residual keys (B, HKV, S - S_q, D) float16)."""
    O._check_bits(nbits)
    B, HKV, S, D = k.shape
    G = group_tokens
    S_q = S - S % G
    qmax = np.float32((1 << nbits) - 1)
    xq = k[:, :, :S_q].astype(np.float32).reshape(B, HKV, S_q // G, G, D)
    gmin = xq.min(axis=3)
    gmax = xq.max(axis=3)
    with np.errstate(all="ignore"):
        scale = ((gmax - gmin) / qmax).astype(np.float32)
        scale = np.where(scale > 0, scale, np.float32(1.0)).astype(np.float32)
        scale16 = scale.astype(np.float16)
        zero16 = gmin.astype(np.float16)
        t = ((xq - zero16.astype(np.float32)[:, :, :, None]).astype(np.float32)
             / scale16.astype(np.float32)[:, :, :, None]).astype(np.float32)
        codes = np.nan_to_num(np.clip(np.rint(t), 0.0, float(qmax)), nan=0.0).astype(np.uint8)
    codes = codes.reshape(B, HKV, S_q, D)
    keys = ChannelKeys(O.pack_codes(codes, nbits), scale16, zero16, nbits, G, D)
    return keys, k[:, :, S_q:].astype(np.float16)


def dequantize_keys_per_channel(kc: ChannelKeys, dtype=np.float32) -> np.ndarray:
    codes = O.unpack_codes(kc.packed, kc.nbits, kc.head_dim).astype(np.float32)
    B, HKV, S_q, D = codes.shape
    G = kc.group_tokens
    cg = codes.reshape(B, HKV, S_q // G, G, D)
    out = cg * kc.scale.astype(np.float32)[:, :, :, None] + kc.zero.astype(np.float32)[:, :, :, None]
    return out.reshape(B, HKV, S_q, D).astype(dtype)


def reference_attention(q, kc: ChannelKeys, vq: O.OracleQuantized, k_res, v_res, sm_scale=None):
    """fp32 attention over [dequantised per-channel keys | residual keys] and
    [dequantised per-token values | residual values]: the ground truth of the decode path."""
    kd = dequantize_keys_per_channel(kc)
    vd = O.dequantize_groupwise(vq)
    k = np.concatenate([kd, np.asarray(k_res, np.float32)], axis=2)
    v = np.concatenate([vd, np.asarray(v_res, np.float32)], axis=2)
    return O.reference_decode_attention(np.asarray(q, np.float32), k, v, sm_scale)
