"""Decode attention on a cache whose keys are quantised per channel, with an fp16 residual
window -- the format the reference describes as future work (docs/future_work.md:229-293,
"make 2-bit usable: per-channel keys, the KIVI idea") and does not implement.  No reference
counterpart; the ground truth is ``oracle/kivi_oracle.py``.

The cache has two parts (future_work.md:246-262):

* the first ``S_q`` tokens (a multiple of 32): keys quantised per channel over groups of 32
  tokens (``quantize.quantize_keys_per_channel``), values per token in groups of 32 as today;
  the fused split kernel reads them with the key scale folded into the query once per tile
  (``TKV_FLAG_K_PER_CHANNEL``);
* the last ``S - S_q < 32`` tokens -- a key group that is not full yet -- in fp16, through the
  fp16 control kernel "as one more split".

Each part is merged to one unnormalised partial ``(acc, m, l)`` per head and the two are
combined by the same log-sum-exp merge that combines history splits.
"""

from __future__ import annotations

import math
from dataclasses import dataclass

import torch

from .. import _cabi
from ..quantize import (CHANNEL_GROUP_TOKENS, ChannelKeys, QuantizedTensor, quantize_groupwise,
                        quantize_keys_per_channel)
from ._launch import check_out, combine_splits, get_workspace, q_for_kernel, split_geometry
from .fp16_decode_attn import fp16_decode_attention

VALUE_GROUP = 32  # per-token value groups the per-channel kernels are built for


@dataclass
class KiviCache:
    """Per-channel keys + per-token values for the first ``S_q`` tokens, fp16 for the rest."""

    k: ChannelKeys
    v: QuantizedTensor
    k_res: torch.Tensor  # (B, HKV, S - S_q, D) float16
    v_res: torch.Tensor

    @property
    def tokens(self) -> int:
        return self.k.tokens + self.k_res.shape[2]

    def nbytes(self) -> int:
        return (self.k.nbytes() + self.v.nbytes()
                + sum(t.numel() * t.element_size() for t in (self.k_res, self.v_res)))


def quantize_kv_kivi(k: torch.Tensor, v: torch.Tensor, nbits: int) -> KiviCache:
    """k, v ``(B, HKV, S, D)`` -> :class:`KiviCache`."""
    if k.shape != v.shape:
        raise ValueError("K and V must have the same shape")
    kc, k_res = quantize_keys_per_channel(k, nbits)
    S_q = kc.tokens
    vq = quantize_groupwise(v[:, :, :S_q].contiguous(), nbits, VALUE_GROUP).contiguous()
    return KiviCache(kc, vq, k_res, v[:, :, S_q:].to(torch.float16).contiguous())


def kivi_decode_attention(q: torch.Tensor, cache: KiviCache, sm_scale: float | None = None,
                          out: torch.Tensor | None = None, _workspace: dict | None = None) -> torch.Tensor:
    """Single decode step on a :class:`KiviCache`.  q ``(B, HQ, D)``; returns ``(B, HQ, D)``
    float32.  With ``out`` and ``_workspace`` supplied the call allocates nothing after its
    first use."""
    ok, why = _cabi.available()
    if not ok:
        raise RuntimeError(f"kivi_decode_attention requires the CUDA library on a GPU: {why}")
    kc, vq = cache.k, cache.v
    B, HQ, D = q.shape
    Bk, HKV, S_q, _ = kc.packed.shape
    R = cache.k_res.shape[2]
    if (B, D) != (Bk, kc.head_dim) or vq.packed.shape != kc.packed.shape:
        raise ValueError(f"q shape {tuple(q.shape)} incompatible with cache {tuple(kc.packed.shape)}")
    if HQ % HKV != 0:
        raise ValueError(f"HQ={HQ} must be a multiple of HKV={HKV}")
    if vq.nbits != kc.nbits or vq.group_size != VALUE_GROUP:
        raise ValueError(f"values must be {kc.nbits}-bit with group_size {VALUE_GROUP}")
    if S_q % CHANNEL_GROUP_TOKENS != 0 or S_q + R == 0:
        raise ValueError("the quantised part must be whole 32-token groups and the cache not empty")
    _cabi.require_cuda(q, "q")
    device = q.device
    sm_scale = 1.0 / math.sqrt(D) if sm_scale is None else sm_scale
    q = q_for_kernel(q)
    out = check_out(out, B, HQ, D, device)
    ws = _workspace if _workspace is not None else {}
    rows = B * HQ
    pair = ws.get("kivi_pair")
    if pair is None or pair[0].shape != (2, rows, D) or pair[0].device != device:
        pair = (torch.empty((2, rows, D), device=device, dtype=torch.float32),
                torch.empty((2, rows), device=device, dtype=torch.float32),
                torch.empty((2, rows), device=device, dtype=torch.float32))
        ws["kivi_pair"] = pair
    pacc, pm, pl = pair
    lib = _cabi.load()
    parts = 0
    with _cabi.on_device(device):
        stream = _cabi.stream_ptr(device)
        if S_q > 0:
            _, num_splits, split_size = split_geometry(S_q, 64, 1, B, HKV, None)
            nslots, _ = _cabi.decode_plan(_cabi.KERNEL_FUSED_SPLIT_KCHAN, kc.nbits, D, VALUE_GROUP, B, HQ,
                                          HKV, S_q, num_splits, split_size, False)
            wq = ws.setdefault("kivi_q", {})
            acc, maxs, sums = get_workspace(wq, B, HQ, nslots, D, device, True)
            _cabi.check(lib.tkv_fused_decode(
                q.data_ptr(), _cabi.dtype_code(q), kc.packed.data_ptr(), kc.scale.data_ptr(),
                kc.zero.data_ptr(), vq.packed.data_ptr(), vq.scale.data_ptr(), vq.zero.data_ptr(),
                acc.data_ptr(), maxs.data_ptr(), sums.data_ptr(), out.data_ptr(), B, HQ, HKV, S_q, D,
                kc.nbits, VALUE_GROUP, float(sm_scale), num_splits, split_size, nslots, None,
                _cabi.FLAG_PARTIALS_ONLY | _cabi.FLAG_K_PER_CHANNEL, stream))
            if R == 0:  # no fp16 tail: the merge of the split partials is the result
                return combine_splits(acc, maxs, sums, out=out)
            combine_splits(acc, maxs, sums, out=pacc[parts].view(B, HQ, D), out_m=pm[parts].view(B, HQ),
                           out_l=pl[parts].view(B, HQ))
            parts += 1
        if R > 0:
            w16 = ws.setdefault("kivi_res", {})
            if S_q == 0:  # shorter than one key group: the fp16 kernel alone
                return fp16_decode_attention(q, cache.k_res, cache.v_res, sm_scale=sm_scale, out=out,
                                             _workspace=w16)
            fp16_decode_attention(q, cache.k_res, cache.v_res, sm_scale=sm_scale, out=out,
                                  _workspace=w16, _partials_only=True)
            combine_splits(w16["acc"], w16["maxs"], w16["sums"], out=pacc[parts].view(B, HQ, D),
                           out_m=pm[parts].view(B, HQ), out_l=pl[parts].view(B, HQ))
            parts += 1
        _cabi.check(lib.tkv_combine_strided(pacc.data_ptr(), pm.data_ptr(), pl.data_ptr(), out.data_ptr(),
                                            None, None, rows, parts, D, D, rows * D, 1, rows, stream))
    return out
