"""Decode path through the C ABI: paged FP8 indexer scan, top-k over each sequence's context,
sparse MLA over the paged FP8 latent cache -- each stage and the composed step against the oracle."""
import pytest
import torch

from llmdivedeep_b200 import layer, ops
from oracle import dsa_oracle as O

pytestmark = pytest.mark.gpu
REL_TOL = 4e-6
ULP_TOL = 4.0


def make_cache(B, P, H, seed, ragged=True):
    g = torch.Generator().manual_seed(seed)
    n_pages = B * P + 3                                           # a few pages no sequence uses
    k = torch.randn(n_pages * 64, 128, generator=g)
    k8, ksc = O.fp8_quant_per_block(k, 128)
    table = torch.randperm(n_pages, generator=g)[: B * P].int().view(B, P)
    ctx = torch.randint(P * 64 // 2, P * 64 + 1, (B,), generator=g).int() if ragged else torch.full((B,), P * 64).int()
    q = torch.randn(B, H, 128, generator=g)
    q8, qs = O.fp8_quant_per_block(q, 128)
    w = O.fold_weights(torch.randn(B, H, generator=g) / 8, qs, 128)
    return q8, w, k8, ksc, table, ctx


@pytest.mark.parametrize("B,P,H", [(4, 6, 64), (3, 33, 64), (2, 5, 32), (5, 1, 64)])
def test_paged_logits_match_oracle(B, P, H):
    q8, w, k8, ksc, table, ctx = make_cache(B, P, H, seed=B * 7 + P)
    out = ops.fp8_paged_mqa_logits(q8.cuda(), w.cuda(), k8.cuda(), ksc.cuda(), table.cuda(), ctx.cuda(), P * 64)
    ops.check_status("cuda")
    o = out.cpu().double()
    for b in range(B):
        n = int(ctx[b])
        rows = O.physical_rows(table[b], torch.arange(n))
        ref = O.indexer_logits_fp64(q8[b:b + 1], k8[rows], ksc[rows], w[b:b + 1], torch.zeros(1, dtype=torch.int32),
                                    torch.tensor([n], dtype=torch.int32))[0]
        err = (o[b, :n] - ref).abs().max()
        assert float(err) <= REL_TOL * float(ref.abs().max()), (b, float(err))
        tile_end = min(P * 64, (n + 127) // 128 * 128)
        assert bool(torch.isinf(out[b, n:tile_end]).all())       # masked tail of the last tile


def test_paged_equals_contiguous_kernel_bitwise():
    """Same keys through the paged and the contiguous entry point give identical logits."""
    B, P, H = 2, 16, 64
    q8, w, k8, ksc, table, ctx = make_cache(B, P, H, seed=3, ragged=False)
    paged = ops.fp8_paged_mqa_logits(q8.cuda(), w.cuda(), k8.cuda(), ksc.cuda(), table.cuda(), ctx.cuda(), P * 64)
    for b in range(B):
        rows = O.physical_rows(table[b], torch.arange(P * 64))
        ke = torch.tensor([P * 64], dtype=torch.int32).cuda()
        flat = ops.fp8_mqa_logits(q8[b:b + 1].cuda(), (k8[rows].cuda(), ksc[rows].cuda()), w[b:b + 1].cuda(), None, ke)
        assert torch.equal(flat[0], paged[b])


def test_bad_page_id_is_flagged_not_read():
    q8, w, k8, ksc, table, ctx = make_cache(2, 4, 64, seed=5, ragged=False)
    table[1, 2] = 10_000
    out = ops.fp8_paged_mqa_logits(q8.cuda(), w.cuda(), k8.cuda(), ksc.cuda(), table.cuda(), ctx.cuda(), 256)
    with pytest.raises(ops.DsaError, match="out of range"):
        ops.check_status("cuda")
    assert bool(torch.isfinite(out[0]).all())


def test_decode_step_composition():
    B, P, H, K = 6, 20, 128, 256
    g = torch.Generator().manual_seed(12)
    q8, w, k8, ksc, table, ctx = make_cache(B, P, 64, seed=12)
    n_rows = k8.shape[0]
    kv = torch.randn(n_rows, 576, generator=g).to(torch.bfloat16)
    cache = O.pack_latent_cache(kv)
    q = torch.randn(B, H, 576, generator=g).to(torch.bfloat16)
    ws = layer.DecodeWorkspace(B, H, P * 64, K, "cuda")
    idx, out = layer.dsa_decode_step(q8.cuda(), w.cuda(), k8.cuda(), ksc.cuda(), table.cuda(), ctx.cuda(), q.cuda(),
                                     cache.cuda(), 0.05, ws)
    ops.check_status("cuda")
    # selection against float64 scores
    ref = O.indexer_logits_paged(q8, w, k8, ksc, table, ctx).double()
    for b in range(B):
        n = int(ctx[b])
        rows = O.physical_rows(table[b], torch.arange(n))
        ref[b, :n] = O.indexer_logits_fp64(q8[b:b + 1], k8[rows], ksc[rows], w[b:b + 1], torch.zeros(1, dtype=torch.int32),
                                           torch.tensor([n], dtype=torch.int32))[0]
    r = O.check_topk_sets(idx.cpu().numpy(), ref.numpy(), [0] * B, ctx.tolist(), K, ulp_tol=ULP_TOL)
    assert not r["bad_rows"], r
    # attention over the kernel's own selection
    want = O.sparse_mla_decode_paged(q.float(), cache, table, idx.cpu(), 0.05, round_bf16=True)
    d = (out.float().cpu() - want).abs()
    assert float(d.max()) <= 2e-2 and float(d.mean()) <= 2e-3


def test_prefill_composition_small_config():
    """The small CPU-reference configuration end to end: 2048 tokens, 4 indexer heads of 64,
    top-k 256, 16 attention heads over one shared latent KV."""
    from tests.helpers import indexer_inputs
    T, K = 2048, 256
    q8, k8, ksc, w, ks, ke = indexer_inputs(T, T, 4, 64, seed=0, window="causal")
    g = torch.Generator().manual_seed(1)
    q = torch.randn(T, 16, 576, generator=g).to(torch.bfloat16)
    kv = torch.randn(T, 576, generator=g).to(torch.bfloat16)
    idx, out = layer.dsa_prefill(q8.cuda(), k8.cuda(), ksc.cuda(), w.cuda(), ks.cuda(), ke.cuda(), K, q.cuda(), kv.cuda(),
                                 192 ** -0.5)
    ops.check_status("cuda")
    ref = O.indexer_logits_fp64(q8, k8, ksc, w, ks, ke).numpy()
    r = O.check_topk_sets(idx.cpu().numpy(), ref, ks.numpy(), ke.numpy(), K, ulp_tol=ULP_TOL)
    assert not r["bad_rows"], r
    rows = torch.arange(0, T, 37)                                   # oracle attention on a sample of rows
    want = O.sparse_mla(q[rows].float(), kv.float(), idx.cpu()[rows], 192 ** -0.5)
    d = (out.float().cpu()[rows] - want).abs()
    assert float(d.max()) <= 2e-2 and float(d.mean()) <= 2e-3
