"""Host-side pieces of bench.py: the synthetic draws and the CPU leg, at toy sizes (no GPU)."""
import json
import subprocess
import sys
import os

import torch

import bench

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_topk_draw_is_causal_without_repeats():
    T, S, K = 300, 300, 64
    idx = bench.draw_topk_positions(T, S, K, "cpu", torch.Generator().manual_seed(0))
    for t in range(T):
        row = idx[t][idx[t] >= 0]
        assert row.numel() == min(t + 1, K) and row.unique().numel() == row.numel() and int(row.max()) <= t
    # rows shorter than K hold all of [0, t]
    assert sorted(idx[10][idx[10] >= 0].tolist()) == list(range(11))


def test_sample_positions_and_pair_counts():
    pos = bench.sample_positions(131072, 192)
    assert len(pos) == 192 and pos[-1] == 131071 and pos == sorted(pos)
    assert abs(sum(p + 1 for p in pos) / len(pos) - 65536) < 2000          # mean causal window ~ S / 2
    assert bench.mla_pairs(32768) == 65012736 and bench.mla_pairs(5, 3) == 1 + 2 + 3 + 3 + 3
    assert bench.causal_keys(4) == 10


def test_cpu_leg_runs_on_a_toy_sequence():
    secs, cores = bench.cpu_prefill_rows([100, 2500, 4095], 4096, 0)
    assert secs > 0 and cores >= 1


def test_reference_arm_on_other_ranks_prints_nothing():
    env = dict(os.environ, RANK="1", WORLD_SIZE="2", LOCAL_RANK="1")
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "2", "--steps", "1",
                        "--warmup", "0"], capture_output=True, text=True, env=env, timeout=120)
    assert p.returncode == 0 and p.stdout.strip() == ""
