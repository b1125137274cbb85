"""The multi-rank logic of tritonkv_b200.parallel on CPU: two `gloo` ranks shard a
decode step by history (one all-gather of (acc, m, l) + log-sum-exp merge) and by batch
(no exchange), with the oracle standing in for the CUDA kernels.  What is tested here is
the host side: shard boundaries, the wire layout, gather order and the merge convention."""

import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import tkv_oracle as O
from tritonkv_b200 import parallel as P


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _inputs(B, HQ, HKV, S, D, seed):
    rng = np.random.default_rng(seed)
    q = rng.standard_normal((B, HQ, D)).astype(np.float16).astype(np.float32)
    k = rng.standard_normal((B, HKV, S, D)).astype(np.float16).astype(np.float32)
    v = rng.standard_normal((B, HKV, S, D)).astype(np.float16).astype(np.float32)
    return q, k, v


def _worker(rank, world, port, S, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        B, HQ, HKV, D = 2, 8, 2, 64
        q, k, v = _inputs(B, HQ, HKV, S, D, seed=7)
        # ---- history split: this rank's token range -> one unnormalised partial ----
        lo, hi = P.history_shard(S, world, rank)
        buf = torch.empty(P.wire_floats(B, HQ, D))
        acc, m, l = P.wire_views(buf, B, HQ, D)
        if hi > lo:
            a, mm, ll = O.split_partials(q, k[:, :, lo:hi], v[:, :, lo:hi], hi - lo, 1)
            acc.copy_(torch.from_numpy(a[:, :, 0]))
            m.copy_(torch.from_numpy(mm[:, :, 0]))
            l.copy_(torch.from_numpy(ll[:, :, 0]))
        else:
            P.empty_partial_(buf, B, HQ, D)
        gathered = P.gather_partials(buf)
        assert gathered.shape == (world, P.wire_floats(B, HQ, D))
        parts = [P.wire_views(gathered[r], B, HQ, D) for r in range(world)]
        A = np.stack([p[0].numpy() for p in parts], axis=2)
        M = np.stack([p[1].numpy() for p in parts], axis=2)
        L = np.stack([p[2].numpy() for p in parts], axis=2)
        merged = O.combine_splits(A, M, L)
        full = O.reference_decode_attention(q, k, v)
        ok_hist = np.allclose(merged, full, atol=2e-5, rtol=2e-5)
        # ---- batch sharding: whole sequences per rank, nothing exchanged but the check ----
        blo, bhi = P.batch_shard(B, world, rank)
        mine = O.reference_decode_attention(q[blo:bhi], k[blo:bhi], v[blo:bhi])
        outs = [None] * world
        dist.all_gather_object(outs, (blo, bhi, mine))
        cat = np.concatenate([o[2] for o in sorted(outs, key=lambda t: t[0])], axis=0)
        ok_batch = np.allclose(cat, full, atol=2e-5, rtol=2e-5)
        if rank == 0:
            ret["hist"], ret["batch"] = bool(ok_hist), bool(ok_batch)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("S", [200, 40])  # 40 tokens: the second rank's shard is short/empty
def test_two_ranks_history_split_and_batch_shard(S):
    world = 2
    with mp.Manager() as mgr:
        ret = mgr.dict()
        mp.spawn(_worker, args=(world, _free_port(), S, ret), nprocs=world, join=True)
        assert ret["hist"] and ret["batch"]


def test_shard_plans():
    for B in (1, 7, 64):
        for world in (1, 2, 4, 8):
            spans = [P.batch_shard(B, world, r) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == B
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            sizes = [hi - lo for lo, hi in spans]
            assert max(sizes) - min(sizes) <= 1
    for S in (1, 31, 32, 1000, 131072):
        for world in (1, 2, 4, 8):
            spans = [P.history_shard(S, world, r) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == S
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            assert all(lo % 32 == 0 for lo, _ in spans if lo < S)
    assert P.history_shard(131072, 8, 3) == (49152, 65536)
    assert P.wire_floats(1, 64, 128) == 64 * 130 and P.wire_floats(1, 3, 128) % 4 == 0
    with pytest.raises(ValueError):
        P.batch_shard(4, 2, 2)
