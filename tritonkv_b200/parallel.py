"""Decode attention across the GPUs of one node (one process per GPU, torch.distributed).

The reference is single-GPU; both partitions below are additions that keep its partial
format ``(acc, m, l)`` in the exp2 domain (kernels/fused_decode_attn.py:340-353) as the
only thing that ever crosses a link.

* **batch x KV-head sharding** (``batch_shard``): every rank owns whole sequences, runs
  ``fused_decode_attention`` on its shard and nothing is exchanged.
* **history split** (``history_shard`` / ``history_split_decode``): one long sequence,
  rank ``r`` holds the contiguous token range ``history_shard(S, world, r)``.  Each rank
  produces ONE locally merged, unnormalised partial per head, the ranks all-gather these
  ``B*HQ*(D+2)`` floats in a single collective, and every rank finishes with the same
  log-sum-exp merge kernel that combines intra-GPU splits (``NS = world``).

The plan functions are pure Python and backend-agnostic so the multi-rank logic is
testable with the ``gloo`` backend on CPU tensors; only the compute calls need CUDA.
"""

from __future__ import annotations

import torch

from . import _cabi
from .kernels._launch import combine_splits


def batch_shard(B: int, world: int, rank: int) -> tuple[int, int]:
    """[lo, hi) of the sequences rank ``rank`` owns: contiguous, sizes differ by <= 1."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError(f"bad rank {rank} of {world}")
    base, extra = divmod(B, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def history_shard(S: int, world: int, rank: int, align: int = 32) -> tuple[int, int]:
    """[lo, hi) of the tokens rank ``rank`` holds.  Boundaries fall on multiples of
    ``align`` tokens (one kernel tile) so no tile straddles two GPUs; the last rank
    takes the remainder and trailing ranks may be empty for short histories."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError(f"bad rank {rank} of {world}")
    per = -(-S // world)
    per = -(-per // align) * align
    lo = min(S, rank * per)
    return lo, min(S, lo + per)


def wire_floats(B: int, HQ: int, D: int) -> int:
    """Floats one rank contributes to the all-gather: acc (B,HQ,D) | m (B,HQ) | l (B,HQ),
    padded to a multiple of 4 so every rank's block starts on a 16-byte boundary."""
    return -(-(B * HQ * (D + 2)) // 4) * 4


def wire_views(buf: torch.Tensor, B: int, HQ: int, D: int):
    """(acc, m, l) views into one rank's flat wire buffer."""
    n = B * HQ
    return (buf[: n * D].view(B, HQ, D), buf[n * D: n * D + n].view(B, HQ),
            buf[n * D + n: n * D + 2 * n].view(B, HQ))


def empty_partial_(buf: torch.Tensor, B: int, HQ: int, D: int) -> torch.Tensor:
    """Fill a wire buffer with the neutral partial (m = -inf, l = 0, acc = 0): what a rank
    that holds no tokens contributes."""
    acc, m, l = wire_views(buf, B, HQ, D)
    acc.zero_()
    m.fill_(float("-inf"))
    l.zero_()
    return buf


def gather_partials(local: torch.Tensor, group=None, out: torch.Tensor | None = None) -> torch.Tensor:
    """One all-gather of every rank's flat wire buffer -> (world, wire_floats)."""
    import torch.distributed as dist

    world = dist.get_world_size(group)
    if out is None:
        out = torch.empty((world, local.numel()), dtype=local.dtype, device=local.device)
    dist.all_gather_into_tensor(out.view(-1), local.contiguous().view(-1), group=group)
    return out


def merge_gathered(gathered: torch.Tensor, B: int, HQ: int, D: int,
                   out: torch.Tensor | None = None) -> torch.Tensor:
    """Log-sum-exp merge of the ranks' partials straight from the gathered buffer
    (world, [acc | m | l]) with the strided combine kernel; returns (B, HQ, D) float32."""
    _cabi.require_cuda(gathered, "gathered")
    world, n = gathered.shape
    rows = B * HQ
    if n != wire_floats(B, HQ, D) or gathered.dtype != torch.float32 or not gathered.is_contiguous():
        raise ValueError("gathered must be a contiguous float32 (world, wire_floats(B, HQ, D)) tensor")
    if out is None:
        out = torch.empty((B, HQ, D), device=gathered.device, dtype=torch.float32)
    base = gathered.data_ptr()
    with torch.cuda.device(gathered.device):
        _cabi.check(_cabi.load().tkv_combine_strided(
            base, base + 4 * rows * D, base + 4 * (rows * D + rows), out.data_ptr(), None, None,
            rows, world, D, D, n, 1, n, _cabi.stream_ptr(gathered.device)))
    return out


class HistorySplitDecoder:
    """Single-sequence long-context decode with the history split over the ranks of
    ``group``.  Buffers are allocated once; ``step`` enqueues: local split kernel ->
    local merge into the wire buffer -> one all-gather -> cross-rank merge."""

    def __init__(self, B: int, HQ: int, D: int, device, group=None):
        import torch.distributed as dist

        self.B, self.HQ, self.D, self.group = B, HQ, D, group
        self.world = dist.get_world_size(group)
        n = wire_floats(B, HQ, D)
        self.local = torch.empty(n, device=device, dtype=torch.float32)
        self.gathered = torch.empty((self.world, n), device=device, dtype=torch.float32)
        self.out = torch.empty((B, HQ, D), device=device, dtype=torch.float32)
        self.ws: dict = {}

    def local_partial(self, q, kq, vq, sm_scale=None):
        """Rank-local unnormalised partial written into the wire buffer."""
        from .kernels import fused_decode_attention

        acc, m, l = wire_views(self.local, self.B, self.HQ, self.D)
        if kq is None or kq.packed.shape[2] == 0:
            empty_partial_(self.local, self.B, self.HQ, self.D)
            return self.local
        fused_decode_attention(q, kq, vq, sm_scale=sm_scale, _workspace=self.ws,
                               _partials_only=True, out=self.out)
        combine_splits(self.ws["acc"], self.ws["maxs"], self.ws["sums"], out=acc, out_m=m, out_l=l)
        return self.local

    def step(self, q, kq, vq, sm_scale=None) -> torch.Tensor:
        self.local_partial(q, kq, vq, sm_scale)
        gather_partials(self.local, self.group, out=self.gathered)
        return merge_gathered(self.gathered, self.B, self.HQ, self.D, out=self.out)


def history_split_decode(q, kq, vq, group=None, sm_scale=None) -> torch.Tensor:
    """One-shot form of :class:`HistorySplitDecoder` (allocates its buffers per call).
    ``kq``/``vq`` are this rank's slice of the cache (``history_shard`` of the tokens)."""
    B, HQ, D = q.shape
    return HistorySplitDecoder(B, HQ, D, q.device, group).step(q, kq, vq, sm_scale)
