"""History split and batch sharding on real GPUs over NCCL (needs >= 2 GPUs; skipped on a
single-GPU box).  Each rank quantises the same seeded cache, keeps its own token range
(or its own sequences), and the merged result is checked against the CPU oracle."""

import os
import socket

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, ret):
    import torch.distributed as dist

    from oracle import tkv_oracle as O
    from tritonkv_b200 import parallel as P
    from tritonkv_b200 import quantize as Q
    from tritonkv_b200.kernels import fused_decode_attention
    from oracle.workloads import make_random_kv

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        # ---- history split: Llama-3-70B head layout, 2-bit, shortened context ----
        B, HQ, HKV, S, D = 1, 64, 8, 6000, 128
        q, k, v = make_random_kv(B, HQ, HKV, S, D, device=dev, seed=123)
        kq, vq = Q.quantize_kv(k, v, 2, 32)
        lo, hi = P.history_shard(S, world, rank)
        cut = lambda t: Q.QuantizedTensor(t.packed[:, :, lo:hi].contiguous(),
                                          t.scale[:, :, lo:hi].contiguous(),
                                          t.zero[:, :, lo:hi].contiguous(), 2, 32, D)
        to_o = lambda t: O.OracleQuantized(t.packed.cpu().numpy(), t.scale.cpu().numpy(),
                                           t.zero.cpu().numpy(), 2, 32, D)
        ref = O.reference_on_quantized(q.float().cpu().numpy(), to_o(kq), to_o(vq))
        ok_hist, exchanges = True, []
        for exchange in ("nccl", "auto"):  # auto: stores into peer memory where it can be set up
            dec = P.HistorySplitDecoder(B, HQ, D, dev, exchange=exchange)
            exchanges.append(dec.exchange)
            outs = [dec.step(q, cut(kq), cut(vq)).clone() for _ in range(5)]  # buffers are reused
            torch.cuda.synchronize()
            rep = O.allclose_report(outs[0].cpu().numpy(), ref)
            ok_hist = (ok_hist and rep["ok"] and rep["cosine"] >= 0.99999
                       and all(torch.equal(outs[0], o) for o in outs[1:]))
        from tritonkv_b200 import _cabi
        ok_hist = ok_hist and _cabi.device_status() == 0
        # ---- batch sharding: nothing is exchanged, every rank checks its own shard ----
        B2 = 6
        q2, k2, v2 = make_random_kv(B2, 32, 8, 700, D, device=dev, seed=124)
        blo, bhi = P.batch_shard(B2, world, rank)
        kq2, vq2 = Q.quantize_kv(k2[blo:bhi].contiguous(), v2[blo:bhi].contiguous(), 4, 32)
        mine = fused_decode_attention(q2[blo:bhi].contiguous(), kq2, vq2)
        to_o4 = lambda t: O.OracleQuantized(t.packed.cpu().numpy(), t.scale.cpu().numpy(),
                                            t.zero.cpu().numpy(), 4, 32, D)
        ref2 = O.reference_on_quantized(q2[blo:bhi].float().cpu().numpy(), to_o4(kq2), to_o4(vq2))
        ok_batch = O.allclose_report(mine.cpu().numpy(), ref2)["ok"]
        flags = torch.tensor([int(ok_hist), int(ok_batch)], device=dev)
        dist.all_reduce(flags, op=dist.ReduceOp.MIN)
        if rank == 0:
            ret["hist"], ret["batch"] = bool(flags[0].item()), bool(flags[1].item())
            ret["rep"] = str(rep) + " exchanges=" + str(exchanges)
    finally:
        dist.destroy_process_group()


def test_history_split_and_batch_shard_over_nccl():
    world = min(torch.cuda.device_count(), 4)
    if world < 2:
        pytest.skip("needs at least 2 GPUs")
    import torch.multiprocessing as mp

    with mp.Manager() as mgr:
        ret = mgr.dict()
        mp.spawn(_worker, args=(world, _free_port(), ret), nprocs=world, join=True)
        assert ret["hist"], ret.get("rep")
        assert ret["batch"]
