"""Host logic shared by the two decode launchers: split geometry, workspace reuse
and the combine launch.  Mirrors kernels/fused_decode_attn.py:486-521 and :558-568."""

from __future__ import annotations

import torch

from .. import _cabi


def next_pow2(x: int) -> int:
    return 1 << (x - 1).bit_length()


def cdiv(a: int, b: int) -> int:
    return -(-a // b)


def pick_num_splits(B: int, HKV: int, n_blocks: int, target_programs: int | None = None) -> int:
    """Choose how many history splits to use so the GPU is filled.

    Same rule as the reference (kernels/fused_decode_attn.py:402-416):
    ``clamp(target_programs // (B*HKV), 1, n_blocks)``.  The reference's default
    target is 4 programs per SM; the launchers here pass the number of CTAs of
    their own kernel that are resident at once (one full wave), which is what the
    occupancy query of the compiled kernel reports.
    """
    if target_programs is None:
        try:
            target_programs = _cabi.device_info()["sm_count"] * 4
        except Exception:
            target_programs = 128
    want = max(1, target_programs // max(1, B * HKV))
    return max(1, min(n_blocks, want))


def balanced_num_splits(B: int, HKV: int, n_blocks: int, block_n: int, wave: int,
                        max_splits: int = 64) -> int:
    """Number of history splits that minimises the modelled step time on a device
    that holds ``wave`` CTAs at once.

    The reference fills the device with ``target // (B*HKV)`` splits
    (kernels/fused_decode_attn.py:402-416), which is right while ``B*HKV`` is far
    below one wave.  Near or above one wave that rule leaves a ragged last wave
    (512 CTAs on 444 slots run as two waves, the second 15 % full), so here the
    split count is chosen by a cost model: waves x (tokens per CTA + a fixed
    per-CTA cost) plus a per-split cost of the combine pass.
    """
    units = max(1, B * HKV)
    if units * 2 <= wave:  # far below one wave: the reference's rule
        return pick_num_splits(B, HKV, n_blocks, wave)
    best, best_cost = 1, None
    for s in range(1, max(1, min(n_blocks, max_splits)) + 1):
        bps = cdiv(n_blocks, s)
        s_eff = cdiv(n_blocks, bps)
        tokens = bps * block_n
        waves = cdiv(units * s_eff, wave)
        cost = waves * (tokens + 160) + 24 * (s_eff if s_eff > 1 else 0)
        if best_cost is None or cost < best_cost:
            best, best_cost = s_eff, cost
    return best


MAX_BALANCED_RAGGED_BATCH = 512  # kMaxRaggedB of the kernels: sequences per device-built schedule


def split_geometry(S: int, block_n: int, num_splits: int | None, B: int, HKV: int,
                   target_programs: int | None, ragged: bool = False):
    """(block_n, num_splits, split_size) with the reference's clamping
    (kernels/fused_decode_attn.py:487-499): block_n is limited to ``max(16, pow2(S))``,
    splits are whole multiples of block_n and none is empty.

    ``num_splits=None``: the kernels balance the work themselves (every CTA gets an
    equal contiguous range of tiles, see ``tkv_decode_plan``; for ragged batches the
    tile sequence is built on the device from ``seq_lens``), so one split covering the
    whole history is requested -- except for ragged batches of more than
    ``MAX_BALANCED_RAGGED_BATCH`` sequences, which are scheduled one CTA per (sequence,
    KV head, split) and get a split count from the cost model, given ``target_programs``
    CTAs resident at once.
    """
    block_n = min(block_n, max(16, next_pow2(S)))
    if block_n < 16 or block_n % 16:
        raise ValueError(f"block_n must be a multiple of 16, got {block_n}")
    n_blocks = cdiv(S, block_n)
    if num_splits is None:
        if not ragged or B <= MAX_BALANCED_RAGGED_BATCH:
            num_splits = 1
        elif target_programs is None:
            num_splits = pick_num_splits(B, HKV, n_blocks, None)
        else:
            num_splits = balanced_num_splits(B, HKV, n_blocks, block_n, target_programs)
    num_splits = max(1, min(num_splits, n_blocks))
    blocks_per_split = cdiv(n_blocks, num_splits)
    num_splits = cdiv(n_blocks, blocks_per_split)  # tighten: no empty splits
    return block_n, num_splits, blocks_per_split * block_n


def get_workspace(ws: dict, B: int, HQ: int, nslots: int, D: int, device, force_partials: bool):
    """Split-partial buffers, reused through the caller's dict exactly as the
    reference does (keys ``key``, ``acc``, ``maxs``, ``sums``, ``dummy_acc``), so a
    call with ``out`` and ``_workspace`` supplied allocates nothing.  ``nslots`` is the
    number of partials per (batch, head) the split kernel writes; it takes the place
    of the reference's ``num_splits`` in the key and the buffer shapes."""
    single = nslots == 1 and not force_partials
    key = (B, HQ, nslots, D)
    if single:
        acc = ws.get("dummy_acc")
        if acc is None or acc.device != device:
            acc = torch.empty((1, 1, 1, 1), device=device, dtype=torch.float32)
            ws["dummy_acc"] = acc
        return None, None, None
    if ws.get("key") == key and ws["acc"].device == device:
        return ws["acc"], ws["maxs"], ws["sums"]
    acc = torch.empty((B, HQ, nslots, D), device=device, dtype=torch.float32)
    maxs = torch.empty((B, HQ, nslots), device=device, dtype=torch.float32)
    sums = torch.empty((B, HQ, nslots), device=device, dtype=torch.float32)
    ws.update(key=key, acc=acc, maxs=maxs, sums=sums)
    return acc, maxs, sums


def check_out(out, B: int, HQ: int, D: int, device):
    if out is None:
        return torch.empty((B, HQ, D), device=device, dtype=torch.float32)
    if out.shape != (B, HQ, D) or out.dtype != torch.float32 or out.device != device:
        raise ValueError(f"out must be a float32 tensor of shape {(B, HQ, D)} on {device}")
    if not out.is_contiguous():
        raise ValueError("out must be contiguous")
    return out


def check_seq_lens(seq_lens, B: int, device):
    if seq_lens is None:
        return None
    if seq_lens.shape != (B,) or seq_lens.dtype != torch.int32 or seq_lens.device != device:
        raise ValueError(f"seq_lens must be an int32 tensor of shape ({B},) on {device}")
    return seq_lens.contiguous()


def q_for_kernel(q: torch.Tensor) -> torch.Tensor:
    if q.dtype not in (torch.float16, torch.bfloat16, torch.float32):
        q = q.float()
    return q.contiguous()


def combine_splits(acc: torch.Tensor, maxs: torch.Tensor, sums: torch.Tensor,
                   out: torch.Tensor | None = None, out_m: torch.Tensor | None = None,
                   out_l: torch.Tensor | None = None) -> torch.Tensor:
    """Log-sum-exp merge of split partials (kernels/fused_decode_attn.py:355-395).

    acc ``(B, HQ, NS, D)``, maxs/sums ``(B, HQ, NS)`` float32 in the exp2 domain.
    Returns ``out (B, HQ, D)``: normalised, or -- when ``out_m`` and ``out_l``
    ``(B, HQ)`` are given -- the merged partial left unnormalised with its (m, l).
    """
    _cabi.require_cuda(acc, "acc")
    lib = _cabi.load()
    B, HQ, NS, D = acc.shape
    if maxs.shape != (B, HQ, NS) or sums.shape != (B, HQ, NS):
        raise ValueError("maxs and sums must have shape (B, HQ, NS)")
    for t in (acc, maxs, sums):
        if t.dtype != torch.float32 or not t.is_contiguous():
            raise ValueError("partials must be contiguous float32 tensors")
    out = check_out(out, B, HQ, D, acc.device)
    if (out_m is None) != (out_l is None):
        raise ValueError("out_m and out_l must be given together")
    with _cabi.on_device(acc.device):
        _cabi.check(lib.tkv_combine(acc.data_ptr(), maxs.data_ptr(), sums.data_ptr(),
                                    out.data_ptr(), _cabi.ptr(out_m), _cabi.ptr(out_l), B, HQ, NS,
                                    D, _cabi.stream_ptr(acc.device)))
    return out
