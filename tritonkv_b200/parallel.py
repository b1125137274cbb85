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

  The exchange has two forms: one NCCL all-gather (``exchange="nccl"``), or stores into
  every peer's receive buffer through symmetric memory with a flag per rank
  (``exchange="peer"``, :class:`PeerExchange`): the local merge kernel writes its result
  straight into the peers' buffers as {value, step} pairs and the cross-rank merge kernel
  waits, bounded, until the pairs of this step have arrived -- no collective launch, no
  fence, one NVLink latency.

The plan functions are pure Python and backend-agnostic so the multi-rank logic is
testable with the ``gloo`` backend on CPU tensors; only the compute calls need CUDA.
"""

from __future__ import annotations

import ctypes

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


def exchange_layout(world: int, wire: int) -> tuple[int, int]:
    """Byte offset of the step counters and total bytes of one rank's symmetric buffer:
    ``2 * world`` blocks of ``wire`` 8-byte pairs {value, step}, then one 32-bit step counter per
    (row, 32-dim slice) of the output -- ``wire // 32`` words hold them (wire = rows * (D + 2))."""
    state_off = 2 * world * wire * 8
    return state_off, state_off + (4 * (wire // 32) + 15) // 16 * 16


class PeerExchange:
    """Receive buffers of all ranks mapped on every rank (torch symmetric memory) and the
    two kernels that use them: ``push`` (local merge stored into every rank's buffer as
    {value, step} pairs) and ``wait_merge`` (bounded wait until every pair of this step has
    arrived, then the cross-rank merge).  Ranks call the pair in lockstep, once per decode step."""

    def __init__(self, B: int, HQ: int, D: int, device, group=None):
        import os

        import torch.distributed as dist

        # The kernels use plain peer stores only.  Without this switch the rendezvous also
        # binds the buffer to an NVLink multicast object on NVLS-capable machines, which
        # nothing here uses and which turns a rank that exits early into link faults on its
        # peers.  It has to be set before the first symmetric-memory call of the process.
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        group = group if group is not None else dist.group.WORLD
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        if self.world > 8:
            raise ValueError("the peer exchange serves at most 8 ranks")
        self.rows, self.D, self.wire = B * HQ, D, wire_floats(B, HQ, D)
        state_off, total = exchange_layout(self.world, self.wire)
        # Allocation can fail on one rank only (no symmetric-memory support, no memory); the
        # rendezvous is a collective, so the ranks first agree that everyone has a buffer.
        err = None
        self.buf = self.handle = None
        try:
            import torch.distributed._symmetric_memory as symm_mem

            self.buf = symm_mem.empty(total // 4, dtype=torch.float32, device=device)
            self.buf.zero_()
            torch.cuda.synchronize(device)
        except Exception as exc:
            err = exc
        flag = torch.tensor([0 if err is not None else 1], device=device)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=group)
        if not bool(flag.item()):
            self.buf = None
            raise RuntimeError(f"symmetric memory is not available on every rank (this rank: {err!r})")
        self.handle = symm_mem.rendezvous(self.buf, group.group_name)
        dist.barrier(group)  # every rank has zeroed its buffer before anyone pushes
        ptrs = [int(p) for p in self.handle.buffer_ptrs]
        table = ctypes.c_void_p * self.world
        self.data_ptrs = table(*ptrs)
        self.state_ptr = ptrs[self.rank] + state_off

    def close(self) -> None:
        """Drop the mapping of the peers' buffers and this rank's own buffer.  Call on every
        rank, with no step in flight, before the process group is destroyed."""
        if self.buf is not None:
            torch.cuda.synchronize(self.buf.device)
        self.data_ptrs = None
        self.state_ptr = 0
        self.handle = None
        self.buf = None

    def push(self, acc: torch.Tensor, m: torch.Tensor, l: torch.Tensor) -> None:
        """``acc (B, HQ, NS, D)``, ``m, l (B, HQ, NS)``: this rank's split partials."""
        NS = acc.shape[2]
        with torch.cuda.device(acc.device):
            _cabi.check(_cabi.load().tkv_combine_push(
                acc.data_ptr(), m.data_ptr(), l.data_ptr(), self.rows, NS, self.D, NS * self.D, self.D,
                NS, 1, self.data_ptrs, self.state_ptr, self.world, self.rank, self.wire,
                _cabi.stream_ptr(acc.device)))

    def push_empty(self, scratch: dict, device) -> None:
        """A rank without tokens contributes the neutral partial (m = -inf, l = 0)."""
        if "acc" not in scratch:
            scratch["acc"] = torch.zeros(self.rows, 1, self.D, device=device, dtype=torch.float32)
            scratch["m"] = torch.full((self.rows, 1), float("-inf"), device=device, dtype=torch.float32)
            scratch["l"] = torch.zeros(self.rows, 1, device=device, dtype=torch.float32)
        a = scratch["acc"]
        self.push(a.view(1, self.rows, 1, self.D) if a.dim() == 3 else a, scratch["m"], scratch["l"])

    def exchange(self, acc: torch.Tensor, m: torch.Tensor, l: torch.Tensor,
                 out: torch.Tensor) -> torch.Tensor:
        """:meth:`push` and :meth:`wait_merge` as one kernel launch."""
        NS = acc.shape[2]
        with torch.cuda.device(acc.device):
            _cabi.check(_cabi.load().tkv_combine_exchange(
                acc.data_ptr(), m.data_ptr(), l.data_ptr(), out.data_ptr(), self.rows, NS, self.D,
                NS * self.D, self.D, NS, 1, self.data_ptrs, self.state_ptr, self.world, self.rank,
                self.wire, _cabi.stream_ptr(acc.device)))
        return out

    def wait_merge(self, out: torch.Tensor) -> torch.Tensor:
        with torch.cuda.device(out.device):
            _cabi.check(_cabi.load().tkv_merge_wait(
                out.data_ptr(), self.rows, self.D, self.data_ptrs, self.state_ptr, self.world,
                self.rank, self.wire, _cabi.stream_ptr(out.device)))
        return out


class HistorySplitDecoder:
    """Single-sequence long-context decode with the history split over the ranks of
    ``group``.  Buffers are allocated once; ``step`` enqueues: local split kernel ->
    local merge -> exchange -> cross-rank merge.  ``exchange``: ``"nccl"`` (one
    all-gather), ``"peer"`` (stores into peer memory, see :class:`PeerExchange`) or
    ``"auto"`` (peer when symmetric memory can be set up on every rank, else NCCL)."""

    def __init__(self, B: int, HQ: int, D: int, device, group=None, exchange: str = "auto"):
        import torch.distributed as dist

        if exchange not in ("auto", "peer", "nccl"):
            raise ValueError(f"exchange must be 'auto', 'peer' or 'nccl', got {exchange!r}")
        self.B, self.HQ, self.D, self.group = B, HQ, D, group
        self.world = dist.get_world_size(group)
        n = wire_floats(B, HQ, D)
        self.local = torch.empty(n, device=device, dtype=torch.float32)
        self.gathered = torch.empty((self.world, n), device=device, dtype=torch.float32)
        self.out = torch.empty((B, HQ, D), device=device, dtype=torch.float32)
        self.ws: dict = {}
        self.peer = None
        self._empty: dict = {}
        if exchange != "nccl" and self.world <= 8:
            # PeerExchange agrees across the ranks before its collective set-up, so either
            # every rank gets one or every rank raises.
            try:
                self.peer = PeerExchange(B, HQ, D, device, group)
            except RuntimeError:
                if exchange == "peer":
                    raise
                self.peer = None
        self.exchange = "peer" if self.peer is not None else "nccl"

    def close(self) -> None:
        """Release the peer mappings (see :meth:`PeerExchange.close`); the decoder cannot
        step afterwards."""
        if self.peer is not None:
            self.peer.close()
            self.peer = None

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
        if self.peer is not None:
            from .kernels import fused_decode_attention

            if kq is None or kq.packed.shape[2] == 0:
                self.peer.push_empty(self._empty, self.out.device)
                return self.peer.wait_merge(self.out)
            fused_decode_attention(q, kq, vq, sm_scale=sm_scale, _workspace=self.ws,
                                   _partials_only=True, out=self.out)
            return self.peer.exchange(self.ws["acc"], self.ws["maxs"], self.ws["sums"], self.out)
        self.local_partial(q, kq, vq, sm_scale)
        gather_partials(self.local, self.group, out=self.gathered)
        return merge_gathered(self.gathered, self.B, self.HQ, self.D, out=self.out)


def history_split_decode(q, kq, vq, group=None, sm_scale=None) -> torch.Tensor:
    """One-shot form of :class:`HistorySplitDecoder` (allocates its buffers per call, NCCL
    exchange).  ``kq``/``vq`` are this rank's slice of the cache (``history_shard`` of the
    tokens)."""
    B, HQ, D = q.shape
    return HistorySplitDecoder(B, HQ, D, q.device, group, exchange="nccl").step(q, kq, vq, sm_scale)
