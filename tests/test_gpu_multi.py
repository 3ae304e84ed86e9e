"""Two GPUs, one process each (nccl): prefill sharded by query rows, decode sharded by batch,
attention output all-gathered -- the result must equal the single-GPU run bit for bit
(every row is computed by the same kernels on the same inputs).  Skipped with fewer than 2 GPUs."""
import os
import socket

import pytest
import torch
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, q_out):
    import torch.distributed as dist
    from llmdivedeep_b200 import ops, sharding as sh
    from tests.helpers import indexer_inputs
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        T, S, K, H = 700, 2048, 256, 128
        q8, k8, ksc, w, ks, ke = (t.to(dev) for t in indexer_inputs(T, S, 64, 128, seed=40, window="causal"))
        g = torch.Generator().manual_seed(41)
        q = torch.randn(T, H, 576, generator=g).to(torch.bfloat16).to(dev)
        kv = torch.randn(S, 576, generator=g).to(torch.bfloat16).to(dev)
        rows = sh.rows_of(sh.row_chunks(T, world, rank, 256), device=dev)
        idx_loc = ops.indexer_topk(q8[rows].contiguous(), k8, ksc, w[rows].contiguous(), ks[rows].contiguous(),
                                   ke[rows].contiguous(), K)
        out_loc = ops.sparse_mla_prefill(q[rows].contiguous(), kv, idx_loc, 0.05)
        out = sh.all_gather_rows(out_loc, T, world, 256)
        idx_all = sh.all_gather_rows(idx_loc, T, world, 256)
        ops.check_status(dev)
        if rank == 0:
            idx_one = ops.indexer_topk(q8, k8, ksc, w, ks, ke, K)
            out_one = ops.sparse_mla_prefill(q, kv, idx_one, 0.05)
            q_out.put((bool(torch.equal(idx_all, idx_one)), bool(torch.equal(out, out_one))))
        dist.barrier()
    finally:
        dist.destroy_process_group()


def _pipeline_worker(rank, world, port, q_out):
    """layer.PrefillPipeline over two nccl ranks (round-robin row blocks, the output all-gathered per chunk on a side
    stream) against the same pipeline on one GPU: same kernels on the same rows, so the results are identical."""
    import torch.distributed as dist
    from llmdivedeep_b200 import layer, ops
    from tests.helpers import indexer_inputs
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        S, K, H = 2900, 256, 128                                # 11.3 blocks of 256 rows: ragged last round
        q8, k8, ksc, w, ks, ke = (t.to(dev) for t in indexer_inputs(S, S, 64, 128, seed=50, window="causal"))
        g = torch.Generator().manual_seed(51)
        q = torch.randn(S, H, 576, generator=g).to(torch.bfloat16).to(dev)
        kv = torch.randn(S, 576, generator=g).to(torch.bfloat16).to(dev)
        same = []
        for transport in ("nccl", "peer"):                      # NCCL all-gather; copies into symmetric memory
            pipe = layer.PrefillPipeline(S, dev, n_heads=H, topk=K, chunk_rows=512, softmax_scale=0.05, rank=rank, world=world,
                                         transport=transport)
            rows = pipe.pos.long()
            out = pipe.output_buffer()
            for _ in range(2):                                  # twice: buffers and events are reused across runs
                out.zero_()
                pipe.run(q8.view(torch.uint8)[rows].view(q8.dtype), k8, ksc, w[rows], q[rows], kv, out)
            torch.cuda.synchronize()
            ops.check_status(dev)
            dist.barrier()
            if rank == 0:
                one = layer.PrefillPipeline(S, dev, n_heads=H, topk=K, chunk_rows=1024, softmax_scale=0.05)
                want = one.run(q8, k8, ksc, w, q, kv, torch.zeros_like(out))
                torch.cuda.synchronize()
                same += [bool(torch.equal(pipe.idx, one.idx[rows])), bool(torch.equal(out, want))]
            dist.barrier()
        if rank == 0:
            q_out.put((same[0] and same[2], same[1] and same[3]))
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_prefill_pipeline_on_two_gpus_equals_single_gpu():
    ctx = mp.get_context("spawn")
    q_out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_pipeline_worker, args=(r, 2, port, q_out)) for r in range(2)]
    for p in procs:
        p.start()
    same_idx, same_out = q_out.get(timeout=300)
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    assert same_idx and same_out


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_row_sharded_prefill_equals_single_gpu():
    ctx = mp.get_context("spawn")
    q_out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q_out)) for r in range(2)]
    for p in procs:
        p.start()
    same_idx, same_out = q_out.get(timeout=300)
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    assert same_idx and same_out
