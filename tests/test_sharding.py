"""Partitioning rules and the output all-gather, on CPU: index arithmetic directly, the
collectives as two gloo ranks with the CPU oracle standing in for the kernels."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from llmdivedeep_b200 import sharding as sh
from oracle import dsa_oracle as O


def test_row_chunks_cover_every_row_once_and_balance_causal_cost():
    for n, world, chunk in [(4096, 8, 256), (1000, 3, 128), (10, 4, 256), (0, 2, 64)]:
        seen = torch.cat([sh.rows_of(sh.row_chunks(n, world, r, chunk)) for r in range(world)])
        assert sorted(seen.tolist()) == list(range(n))
    costs = [sh.causal_cost(sh.row_chunks(131072, 8, r, 256)) for r in range(8)]
    assert max(costs) / min(costs) < 1.001                     # serpentine chunks: within 0.1 %
    slab = [sh.causal_cost([(r * 16384, (r + 1) * 16384)]) for r in range(8)]
    assert max(slab) / min(slab) > 10                          # one slab per rank would not balance
    with pytest.raises(ValueError):
        sh.row_chunks(10, 2, 2)


def test_head_and_batch_ranges():
    assert [sh.head_range(128, 8, r) for r in range(8)] == [(16 * r, 16 * r + 16) for r in range(8)]
    parts = [sh.head_range(10, 4, r) for r in range(4)]
    assert parts == [(0, 3), (3, 6), (6, 8), (8, 10)]
    assert [sh.batch_range(512, 8, r)[1] - sh.batch_range(512, 8, r)[0] for r in range(8)] == [64] * 8


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, q_out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.manual_seed(0)                                    # same data on every rank
        T, H, S, K = 70, 6, 90, 16
        q = torch.randn(T, H, 576)
        kv = torch.randn(S, 576)
        idx = torch.stack([torch.randperm(S)[:K] for _ in range(T)]).int()
        full = O.sparse_mla(q, kv, idx, 0.05)
        # rows: each rank attends its own row chunks, then all-gather
        rows = sh.rows_of(sh.row_chunks(T, world, rank, 16))
        got_rows = sh.all_gather_rows(O.sparse_mla(q[rows], kv, idx[rows], 0.05), T, world, 16)
        # heads: each rank attends all rows for its head slice, then all-gather
        a, b = sh.head_range(H, world, rank)
        got_heads = sh.all_gather_heads(O.sparse_mla(q[:, a:b], kv, idx, 0.05), H, world)
        # decode batch: contiguous slices
        a, b = sh.batch_range(T, world, rank)
        got_batch = sh.all_gather_batch(full[a:b].contiguous(), T, world)
        q_out.put((rank, float((got_rows - full).abs().max()), float((got_heads - full).abs().max()),
                   float((got_batch - full).abs().max())))
    finally:
        dist.destroy_process_group()


def test_two_rank_gloo_gathers_reassemble_the_single_process_result():
    ctx = mp.get_context("spawn")
    q_out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q_out)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q_out.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(60)
        assert p.exitcode == 0
    for rank, e_rows, e_heads, e_batch in res:
        assert e_rows < 1e-5 and e_heads < 1e-5 and e_batch == 0.0, (rank, e_rows, e_heads, e_batch)


def test_round_robin_blocks_cover_every_row_and_nearly_balance():
    for n, world, block in [(4096, 8, 256), (1000, 3, 128), (10, 4, 256), (0, 2, 64)]:
        seen = torch.cat([sh.rows_of(sh.round_robin_blocks(n, world, r, block)) for r in range(world)])
        assert sorted(seen.tolist()) == list(range(n))
    costs = [sh.causal_cost(sh.round_robin_blocks(131072, 8, r, 256)) for r in range(8)]
    assert max(costs) / min(costs) < 1.03                      # within 2 / rounds of each other


def _pipeline_worker(rank, world, port, q_out):
    """PrefillPipeline over two gloo ranks with the CPU oracle standing in for the kernels: the gathered
    output equals the single-process result, ragged last round included."""
    from llmdivedeep_b200 import layer
    from tests.helpers import indexer_inputs
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        S, H, K, blk = 150, 4, 24, 16                           # 9.4 blocks: the last round is ragged
        q8, k8, ksc, w, ks, ke = indexer_inputs(S, S, 4, 128, seed=3, window="causal")
        g = torch.Generator().manual_seed(5)
        q = torch.randn(S, H, 576, generator=g).to(torch.bfloat16)
        kv = torch.randn(S, 576, generator=g).to(torch.bfloat16)

        def select(q_idx, k_idx, k_scale, wts, ks_, ke_, k, out):
            lg = O.indexer_logits(q_idx, k_idx, k_scale, wts, ks_, ke_, relu=True)
            top = O.topk_indices(lg, k)
            pad = torch.gather(lg, 1, top) == float("-inf")
            out.copy_(torch.where(pad, torch.full_like(top, -1), top).to(torch.int32))
            return out

        def attend(qq, kvv, idx, scale, out):
            out.copy_(O.sparse_mla(qq, kvv, idx, scale).to(out.dtype))
            return out

        one = layer.PrefillPipeline(S, "cpu", n_heads=H, topk=K, chunk_rows=64, block_rows=blk, select=select, attend=attend)
        want = one.run(q8, k8, ksc, w, q, kv, torch.zeros(S, H, 512, dtype=torch.bfloat16))
        pipe = layer.PrefillPipeline(S, "cpu", n_heads=H, topk=K, chunk_rows=32, rank=rank, world=world,
                                     block_rows=blk, select=select, attend=attend)
        rows = pipe.pos.long()
        assert torch.equal(pipe.ke, ke[rows])
        got = pipe.run(q8[rows], k8, ksc, w[rows], q[rows], kv, torch.zeros(S, H, 512, dtype=torch.bfloat16))
        q_out.put((rank, bool(torch.equal(got, want)), bool(torch.equal(pipe.idx, one.idx[rows]))))
    finally:
        dist.destroy_process_group()


def test_two_rank_prefill_pipeline_equals_single_process():
    ctx = mp.get_context("spawn")
    q_out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_pipeline_worker, args=(r, 2, port, q_out)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q_out.get(timeout=180) for _ in procs]
    for p in procs:
        p.join(60)
        assert p.exitcode == 0
    for rank, same_out, same_idx in res:
        assert same_out and same_idx, (rank, same_out, same_idx)
