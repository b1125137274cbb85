"""fp16 flash-decoding attention -- the *control* for the fused kernel.

Drop-in for the reference's ``kernels/fp16_decode_attn.py`` (launcher :142-241).
Same split over the history, same online softmax, same GQA amortisation, same
combine kernel as ``fused_decode_attention``, with K/V read as plain fp16, so the
two differ only in how the cache is read:

    this kernel -> fused 4-bit  =  the quantisation/fusion effect alone
"""

from __future__ import annotations

import math

import torch

from .. import _cabi
from ._launch import (check_out, check_seq_lens, get_workspace, q_for_kernel, split_geometry)


def fp16_decode_attention(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    sm_scale: float | None = None,
    block_n: int = 64,
    num_warps: int = 4,
    num_stages: int = 2,
    num_splits: int | None = None,
    out: torch.Tensor | None = None,
    _workspace: dict | None = None,
    seq_lens: torch.Tensor | None = None,
    _partials_only: bool = False,
) -> torch.Tensor:
    """Decode attention on an unquantised fp16 cache, same shape as the fused kernel.

    q: (B, HQ, D); k, v: (B, HKV, S, D) (cast to fp16 if they are not). Returns
    (B, HQ, D) float32.  ``num_warps`` / ``num_stages`` are accepted and ignored.
    """
    ok, why = _cabi.available()
    if not ok:
        raise RuntimeError(f"fp16_decode_attention requires the CUDA library on a GPU: {why}")

    B, HQ, D = q.shape
    Bk, HKV, S, Dk = k.shape
    if HQ % HKV != 0:
        raise ValueError(f"HQ={HQ} must be a multiple of HKV={HKV}")
    if (B, D) != (Bk, Dk) or v.shape != k.shape:
        raise ValueError(f"q {tuple(q.shape)}, k {tuple(k.shape)}, v {tuple(v.shape)} are incompatible")
    _cabi.require_cuda(q, "q")
    _cabi.require_cuda(k, "k")

    device = q.device
    sm_scale = 1.0 / math.sqrt(D) if sm_scale is None else sm_scale
    q = q_for_kernel(q)
    k = k.to(torch.float16).contiguous()
    v = v.to(torch.float16).contiguous()
    seq_lens = check_seq_lens(seq_lens, B, device)

    lib = _cabi.load()
    with _cabi.on_device(device):
        ragged = seq_lens is not None
        target = None
        if num_splits is None and ragged:
            target = _cabi.wave_programs(_cabi.KERNEL_FP16_SPLIT, 0, D, 0)
        block_n, num_splits, split_size = split_geometry(S, block_n, num_splits, B, HKV, target,
                                                         ragged)
        nslots, _ = _cabi.decode_plan(_cabi.KERNEL_FP16_SPLIT, 0, D, 0, B, HQ, HKV, S, num_splits,
                                      split_size, ragged)

        out = check_out(out, B, HQ, D, device)
        ws = _workspace if _workspace is not None else {}
        acc, maxs, sums = get_workspace(ws, B, HQ, nslots, D, device, _partials_only)

        stream = _cabi.stream_ptr(device)
        # one call enqueues the split kernel and, when there are partials to merge, the combine
        flags = _cabi.FLAG_PARTIALS_ONLY if _partials_only else _cabi.FLAG_COMBINE
        _cabi.check(lib.tkv_fp16_decode(
            q.data_ptr(), _cabi.dtype_code(q), k.data_ptr(), v.data_ptr(),
            _cabi.ptr(acc), _cabi.ptr(maxs), _cabi.ptr(sums), out.data_ptr(),
            B, HQ, HKV, S, D, float(sm_scale), num_splits, split_size, nslots,
            _cabi.ptr(seq_lens), flags, stream))
    return out
