"""Host side of bench.py that needs no GPU: the seeded input generator shared by the GPU
arm and the CPU (reference) arm, the config object both arms print, the context placement
of the L2 sweep, and the reference arm itself on a small case."""

import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
import bench  # noqa: E402


def test_any_token_range_of_a_sequence_is_reproducible():
    """A rank that owns tokens [lo, hi) of a sequence draws exactly the values the whole
    sequence holds there, whatever the chunk boundaries."""
    k, v = bench.host_sequence("llama70b-128k", 0, 0, 3 * bench.CHUNK, seed=3)
    for lo, hi in [(0, 100), (bench.CHUNK - 5, bench.CHUNK + 7), (2 * bench.CHUNK, 3 * bench.CHUNK),
                   (1234, 9000)]:
        k2, v2 = bench.host_sequence("llama70b-128k", 0, lo, hi, seed=3)
        assert torch.equal(k2, k[:, lo:hi]) and torch.equal(v2, v[:, lo:hi])
    k3, _ = bench.host_sequence("llama70b-128k", 1, 0, 100, seed=3)
    assert not torch.equal(k3, k[:, :100])  # another sequence, other values


def test_value_distributions():
    k, v = bench.host_sequence("llama8b-b64", 0, 0, 4096, seed=0)
    assert k.dtype == torch.float16 and k.shape == (8, 4096, 128)
    assert abs(float(k.float().std()) - 1.0) < 0.02 and abs(float(v.float().mean())) < 0.01
    kc, _ = bench.host_sequence("qwen-b1", 0, 0, 4096, seed=0)
    per_channel = kc.float().std(dim=1)  # (HKV, D): lognormal(0, 0.5) factors -> wide spread
    assert float(per_channel.max() / per_channel.min()) > 3.0
    ke, _ = bench.host_sequence("ragged-b16", 0, 0, 4096, seed=0)
    frac = float((ke.float().abs() > 6.0).float().mean())
    assert 0.004 < frac < 0.012  # 1 % of the K entries x20: most of them leave N(0,1)'s range


def test_both_arms_print_the_same_config():
    a = bench.workload_config("llama8b-b64", 64, 32, 8, 128, 4096, 4, 4)
    b = bench.workload_config("llama8b-b64", 64, 32, 8, 128, 4096, 4, 4)
    assert a == b and "ctx=4096" in a["workload"] and "batch sharded" in a["partition"]
    assert bench.workload_config("llama8b-b64", 64, 32, 8, 128, 4096, 4, 1)["partition"] == "single GPU"


def test_l2_sweep_contexts_follow_the_footprint_rule():
    l2 = 126 * 1024 * 1024
    ctxs = bench.l2_sweep_contexts(l2, HKV=2, D=128)
    assert len(ctxs) == len(bench.L2_SWEEP_FACTORS) and ctxs == sorted(ctxs)
    for f, c in zip(bench.L2_SWEEP_FACTORS, ctxs):
        assert c % 256 == 0
        assert abs(bench.fp16_bytes(1, 2, c, 128) / l2 - f) / f < 0.01
    assert ctxs[-1] > 393216 * 3  # B200's L2 is far larger than the laptop's: 12 x L2 is 1.5 M tokens


def test_byte_accounting():
    # per (token, KV head): K+V codes + scale/zero -- 160 B at 4-bit, 96 B at 2-bit, 512 B fp16
    assert bench.fused_bytes(1, 1, 1, 128, 4) == 160
    assert bench.fused_bytes(1, 1, 1, 128, 2) == 96
    assert bench.fp16_bytes(1, 1, 1, 128) == 512
    assert bench.fused_bytes(64, 8, 4096, 128, 4) == 335_544_320


def test_reference_arm_runs_the_cpu_path_and_prints_one_line():
    """``--impl reference`` on a small case: one JSON line with the contract's keys, the CPU
    port timed on the whole (small) configuration."""
    env = dict(os.environ, PYTHONPATH=ROOT)
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference",
                        "--workload", "qwen-b1", "--ctx", "2048", "--steps", "3", "--warmup", "1"],
                       capture_output=True, text=True, env=env, timeout=300)
    assert r.returncode == 0, r.stderr[-2000:]
    line = json.loads(r.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and line["unit"] == "GB/s" and line["value"] > 0
    assert line["cpu_baseline"]["kind"] == "port" and line["cpu_baseline"]["cores"] >= 1
    assert "the whole configuration" in line["cpu_baseline"]["sample"]
    assert line["e2e"]["h2d_bytes_per_step"] == 0 and line["gpu_launches"] == 0
    assert line["config"] == bench.workload_config("qwen-b1", 1, 12, 2, 128, 2048, 4, 1)


def test_host_quantized_matches_the_oracle_quantiser():
    from oracle import tkv_oracle as O

    q, kq, vq = bench.host_quantized("qwen-b1", 1, 512, 4, seed=1)
    _, k, v = bench.host_batch("qwen-b1", 0, 1, 0, 512, seed=1)
    ref = O.quantize_groupwise(k.float().numpy(), 4, 32)
    assert np.array_equal(kq[0], ref.packed)
    assert np.array_equal(kq[1], ref.scale.view(np.uint16))
    assert q.shape == (1, 12, 128) and q.dtype == np.float32
