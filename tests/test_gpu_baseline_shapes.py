"""Parity at the benchmark's own shapes: the kernels run at the full size of each named configuration on
the bench's seeded inputs, and a stated sample of their output is checked against the CPU oracle (the
whole output would take the CPU hours).  Top-k results are adjudicated in float64 on the same FP8 values;
every test prints how many sampled rows have a near-tie swap and how many of those lie further than
1 fp32 ulp from the k-th score (the test bound is 4 ulps: a 64-term fp32 head sum carries a few ulps of
rounding noise in any order)."""
import numpy as np
import pytest
import torch

import bench
from llmdivedeep_b200 import layer, ops
from oracle import dsa_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda"
ULP_TOL = 4.0


def _take(t, rows):
    """t[rows] on the CPU (float8 tensors are indexed through their bytes)."""
    rows = rows.to(t.device)
    if t.dtype == torch.float8_e4m3fn:
        return t.view(torch.uint8)[rows].view(torch.float8_e4m3fn).cpu()
    return t[rows].cpu()


def _report(name, r):
    print(f"{name}: {r['exact_rows']}/{r['rows']} rows exact, {r['swapped_rows']} with near-tie swaps, "
          f"{r['rows_over_1ulp']} over 1 ulp, max {r['max_ulp']:.2f} ulp")


def test_indexer_topk_4096_x_65536_row_sample_against_float64():
    """Standalone indexer + top-k: 4096 query rows (positions 61440-65535) x 65536 keys, k = 2048, bench seed 0.
    256 rows spread over the chunk, first and last included."""
    q8, k8, ksc, w, ks, ke = bench.make_indexer_inputs(DEV, 0)
    idx = ops.indexer_topk(q8, k8, ksc, w, ks, ke, bench.TOPK)
    ops.check_status(DEV)
    assert idx.shape == (4096, 2048)
    rows = torch.unique(torch.cat([torch.arange(0, 4096, 16), torch.tensor([4095])]))
    assert rows.numel() >= 256
    ks_s, ke_s = _take(ks, rows), _take(ke, rows)
    ref = O.indexer_logits_fp64(_take(q8, rows), k8.cpu(), ksc.cpu(), _take(w, rows).float(), ks_s, ke_s, row_chunk=16).numpy()
    r = O.check_topk_sets(_take(idx, rows).numpy(), ref, ks_s.numpy(), ke_s.numpy(), bench.TOPK, ulp_tol=ULP_TOL)
    _report("indexer+top-k 4096 x 65536 (257 sampled rows)", r)
    assert not r["bad_rows"], r


def test_sparse_mla_32768_tokens_row_sample_against_fp32():
    """Sparse MLA prefill at 32768 tokens x 128 heads, 2048 keys per token drawn without replacement from [0, t]
    (all of [0, t] for t < 2047): the kernel runs on all tokens, 72 of them are checked."""
    T = S = 32768
    g = torch.Generator(device=DEV).manual_seed(3)
    q = torch.randn(T, bench.MLA_HEADS, 576, device=DEV, dtype=torch.bfloat16, generator=g)
    kv = torch.randn(S, 576, device=DEV, dtype=torch.bfloat16, generator=g)
    idx = bench.draw_topk_positions(T, S, bench.TOPK, DEV, g)
    # the draw itself: causal, no repeats, full rows beyond t = 2047, -1 padding before
    srt = idx.sort(dim=1).values
    assert bool(((srt[:, 1:] != srt[:, :-1]) | (srt[:, 1:] < 0)).all())
    assert bool((idx.max(dim=1).values <= torch.arange(T, device=DEV)).all())
    assert bool(((idx >= 0).sum(1) == torch.arange(1, T + 1, device=DEV).clamp_max(bench.TOPK)).all())
    out = ops.sparse_mla_prefill(q, kv, idx, bench.SCALE)
    ops.check_status(DEV)
    rows = torch.unique(torch.cat([torch.tensor([0, 1, 5, 63, 64, 2046, 2047, 2048, T - 1]), torch.arange(300, T, 512)]))
    assert rows.numel() >= 64
    want = O.sparse_mla(_take(q, rows), kv.cpu(), _take(idx, rows), bench.SCALE, row_chunk=8)
    err = (_take(out, rows).float() - want).abs()
    print(f"sparse MLA 32768 tokens ({rows.numel()} sampled): max |err| {float(err.max()):.2e}, mean {float(err.mean()):.2e}")
    assert float(err.max()) <= 2e-2 and float(err.mean()) <= 2e-3


def test_decode_step_batch_64_context_131072_two_sequences_against_the_oracle():
    """One decode step at batch 64, context 131072, random page order, FP8 caches quantised from N(0,1): the step
    runs on all 64 sequences; sequences 0 and 63 are checked stage by stage (paged indexer -> top-k -> paged MLA)."""
    B, CTX, K = 64, 131072, bench.TOPK
    g = torch.Generator(device=DEV).manual_seed(5)
    q8, w, kcache, kscale, table, ctx, qd, latent = bench.make_decode_inputs(DEV, B, CTX, g)
    ws = layer.DecodeWorkspace(B, bench.MLA_HEADS, CTX, K, DEV)
    idx, out = layer.dsa_decode_step(q8, w, kcache, kscale, table, ctx, qd, latent, bench.SCALE, ws)
    ops.check_status(DEV)
    pos = torch.arange(CTX, device=DEV)
    for b in (0, B - 1):
        rows = table[b].long()[pos // 64] * 64 + pos % 64                  # this sequence's cache rows, in position order
        k_seq, ksc_seq, lat_seq = _take(kcache, rows), _take(kscale, rows), _take(latent, rows)
        ref = O.indexer_logits_fp64(q8[b:b + 1].cpu(), k_seq, ksc_seq, w[b:b + 1].cpu().float(), torch.zeros(1, dtype=torch.int32),
                                    torch.tensor([CTX], dtype=torch.int32)).numpy()
        r = O.check_topk_sets(idx[b:b + 1].cpu().numpy(), ref, [0], [CTX], K, ulp_tol=ULP_TOL)
        _report(f"decode sequence {b}: top-k of 131072", r)
        assert not r["bad_rows"], r
        ident = torch.arange(CTX // 64, dtype=torch.int32).unsqueeze(0)
        want = O.sparse_mla_decode_paged(qd[b:b + 1].cpu().float(), lat_seq, ident, idx[b:b + 1].cpu(), bench.SCALE, round_bf16=True)
        err = (out[b:b + 1].cpu().float() - want).abs()
        print(f"decode sequence {b}: output max |err| {float(err.max()):.2e}, mean {float(err.mean()):.2e}")
        assert float(err.max()) <= 2e-2 and float(err.mean()) <= 2e-3


def test_decode_step_with_context_shorter_than_topk():
    """max_ctx < top-k: k = max_ctx columns are selected and the index rows keep that stride all the way
    into the attention kernel."""
    B, P, K = 3, 4, 2048                                                   # 256 positions per sequence
    g = torch.Generator(device=DEV).manual_seed(9)
    q8, w, kcache, kscale, table, ctx, qd, latent = bench.make_decode_inputs(DEV, B, P * 64, g)
    ctx = torch.tensor([256, 100, 7], dtype=torch.int32, device=DEV)
    ws = layer.DecodeWorkspace(B, bench.MLA_HEADS, P * 64, K, DEV)
    assert ws.idx.shape == (B, 256)
    idx, out = layer.dsa_decode_step(q8, w, kcache, kscale, table, ctx, qd, latent, bench.SCALE, ws)
    ops.check_status(DEV)
    for b in range(B):
        n = int(ctx[b])
        assert sorted(idx[b][idx[b] >= 0].tolist()) == list(range(n))      # fewer keys than k: all of them
    want = O.sparse_mla_decode_paged(qd.cpu().float(), latent.cpu(), table.cpu(), idx.cpu(), bench.SCALE, round_bf16=True)
    err = (out.cpu().float() - want).abs()
    assert float(err.max()) <= 2e-2 and float(err.mean()) <= 2e-3


def test_pack_latent_cache_equals_the_oracle_records():
    kv = torch.randn(1000, 576, generator=torch.Generator().manual_seed(2)).to(torch.bfloat16)
    kv[5] = 0
    assert torch.equal(layer.pack_latent_cache(kv.cuda()).cpu(), O.pack_latent_cache(kv))
