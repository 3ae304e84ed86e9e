"""dsa_sparse_mla_prefill / dsa_sparse_mla_decode_paged (through the C ABI) against the CPU oracle.

Floating point: bf16 inputs, bf16 tensor-core products with fp32 accumulation, the two halves
of every score rounded to fp16 between the CTAs of a pair, P rounded to bf16, bf16 output.  Tolerance (the one stated for this path): max-abs 2e-2 and mean-abs 2e-3
against the oracle's fp32 computation on the same bf16 inputs.
"""
import pytest
import torch

from llmdivedeep_b200 import ops
from oracle import dsa_oracle as O

pytestmark = pytest.mark.gpu
MAX_ABS, MEAN_ABS = 2e-2, 2e-3


def make(T, H, S, K, seed, causal=True):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(T, H, 576, generator=g).to(torch.bfloat16)
    kv = torch.randn(S, 576, generator=g).to(torch.bfloat16)
    idx = torch.full((T, K), -1, dtype=torch.int32)
    for t in range(T):
        hi = (S - T + t + 1) if causal else S
        n = min(K, hi)
        idx[t, :n] = torch.randperm(hi, generator=g)[:n].int()
    return q, kv, idx


def check(out, ref):
    d = (out.float().cpu() - ref).abs()
    assert float(d.max()) <= MAX_ABS and float(d.mean()) <= MEAN_ABS, (float(d.max()), float(d.mean()))


@pytest.mark.parametrize("T,H,S,K", [(4, 128, 256, 64), (8, 128, 1000, 192), (6, 128, 3000, 2048), (5, 16, 500, 256),
                                     (3, 200, 400, 100), (2, 1, 130, 65), (70, 128, 200, 64), (3, 64, 5000, 1)])
def test_prefill_matches_oracle(T, H, S, K):
    q, kv, idx = make(T, H, S, K, seed=T * 3 + K)
    scale = 576 ** -0.5 * 2
    out = ops.sparse_mla_prefill(q.cuda(), kv.cuda(), idx.cuda(), scale)
    ops.check_status("cuda")
    check(out, O.sparse_mla(q.float(), kv.float(), idx, scale))


def test_short_rows_holes_and_empty_rows():
    """Causal rows shorter than K (the first tokens of a sequence), holes in the middle of the
    slot list, and a row with no valid slot at all (zeros)."""
    q, kv, idx = make(40, 128, 40, 128, seed=9)      # row t has t+1 valid slots
    idx[7, ::3] = -1
    idx[11] = -1
    out = ops.sparse_mla_prefill(q.cuda(), kv.cuda(), idx.cuda(), 0.05)
    ops.check_status("cuda")
    check(out, O.sparse_mla(q.float(), kv.float(), idx, 0.05))
    assert float(out[11].float().abs().max()) == 0.0


def test_large_scores_trigger_rescaling():
    """Scores that keep growing along the slot list force the running-maximum rescale path."""
    g = torch.Generator().manual_seed(3)
    T, H, S, K = 4, 128, 1024, 1024
    q = torch.randn(T, H, 576, generator=g).to(torch.bfloat16)
    kv = torch.randn(S, 576, generator=g)
    kv *= torch.linspace(0.1, 1.0, S).unsqueeze(1)          # later rows have larger norms
    kv = kv.to(torch.bfloat16)
    idx = torch.arange(K, dtype=torch.int32).repeat(T, 1)
    # scale 0.2: logits reach +-20 and the block maximum climbs by ~25 log2 units along the list (several rescales).
    # The two halves of a score cross the CTA pair as fp16 (11 significant bits each), so the error of a logit grows
    # with scale * |score|; DSA's own scale is 576^-0.5 or 192^-0.5, five to three times smaller than this one.
    out = ops.sparse_mla_prefill(q.cuda(), kv.cuda(), idx.cuda(), 0.2)
    check(out, O.sparse_mla(q.float(), kv.float(), idx, 0.2))


def test_caller_supplied_out_must_be_dense_bf16_of_the_right_shape():
    q, kv, idx = make(4, 128, 256, 64, seed=2)
    q, kv, idx = q.cuda(), kv.cuda(), idx.cuda()
    good = torch.empty(4, 128, 512, dtype=torch.bfloat16, device="cuda")
    assert ops.sparse_mla_prefill(q, kv, idx, 0.05, out=good) is good
    for bad in (torch.empty(4, 128, 512, dtype=torch.float16, device="cuda"),
                torch.empty(4, 128, 256, dtype=torch.bfloat16, device="cuda"),
                torch.empty(4, 128, 1024, dtype=torch.bfloat16, device="cuda")[:, :, ::2]):
        with pytest.raises(ops.DsaError, match="out must be"):
            ops.sparse_mla_prefill(q, kv, idx, 0.05, out=bad)


def test_out_of_range_index_is_skipped_and_flagged():
    q, kv, idx = make(2, 128, 100, 64, seed=1, causal=False)
    bad = idx.clone()
    bad[0, 5] = 100                                          # == S_kv
    out = ops.sparse_mla_prefill(q.cuda(), kv.cuda(), bad.cuda(), 0.05)
    with pytest.raises(ops.DsaError, match="out of range"):
        ops.check_status("cuda")
    ref_idx = idx.clone()
    ref_idx[0, 5] = -1
    check(out, O.sparse_mla(q.float(), kv.float(), ref_idx, 0.05))


def test_deterministic_and_permutation_invariant():
    q, kv, idx = make(3, 128, 2000, 512, seed=5, causal=False)
    a = ops.sparse_mla_prefill(q.cuda(), kv.cuda(), idx.cuda(), 0.04)
    b = ops.sparse_mla_prefill(q.cuda(), kv.cuda(), idx.cuda(), 0.04)
    assert torch.equal(a, b)
    perm = torch.randperm(512)
    c = ops.sparse_mla_prefill(q.cuda(), kv.cuda(), idx[:, perm].contiguous().cuda(), 0.04)
    assert float((a.float() - c.float()).abs().max()) <= 1e-2    # softmax does not depend on slot order


def test_full_size_row_equals_dense_attention():
    """Bench-size shape property: with every key of a 2048-key context selected, sparse MLA is
    dense softmax attention (checked against torch on the GPU in fp32)."""
    g = torch.Generator().manual_seed(8)
    T, H, S = 16, 128, 2048
    q = torch.randn(T, H, 576, generator=g).to(torch.bfloat16).cuda()
    kv = torch.randn(S, 576, generator=g).to(torch.bfloat16).cuda()
    idx = torch.stack([torch.randperm(S, generator=g) for _ in range(T)]).int().cuda()
    scale = 192 ** -0.5
    out = ops.sparse_mla_prefill(q, kv, idx, scale)
    p = torch.softmax(torch.einsum("thd,sd->ths", q.float(), kv.float()) * scale, dim=-1)
    ref = torch.einsum("ths,sd->thd", p, kv.float()[:, :512])
    d = (out.float() - ref).abs()
    assert float(d.max()) <= MAX_ABS and float(d.mean()) <= MEAN_ABS


@pytest.mark.parametrize("B,H,P,K", [(4, 128, 8, 200), (3, 128, 40, 2048), (2, 32, 4, 64)])
def test_decode_paged_matches_oracle(B, H, P, K):
    g = torch.Generator().manual_seed(B * 11 + K)
    kv = torch.randn(B * P * 64, 576, generator=g).to(torch.bfloat16)
    cache = O.pack_latent_cache(kv)
    table = torch.randperm(B * P, generator=g).int().view(B, P)
    idx = torch.stack([torch.randperm(P * 64, generator=g)[:K] for _ in range(B)]).int()
    idx[B - 1, K // 2:] = -1
    q = torch.randn(B, H, 576, generator=g).to(torch.bfloat16)
    out = ops.sparse_mla_decode_paged(q.cuda(), cache.cuda(), table.cuda(), idx.cuda(), 0.06)
    ops.check_status("cuda")
    check(out, O.sparse_mla_decode_paged(q.float(), cache, table, idx, 0.06, round_bf16=True))


def test_decode_holes_and_odd_block_counts():
    """Holes inside the slot list (empty slots are zero-filled rows with a cleared validity bit) and slot lists of one,
    three and five 64-key blocks: the gather alternates between two raw stages and two sets of rope registers."""
    for K in (40, 130, 300):
        g = torch.Generator().manual_seed(K)
        B, H, P = 3, 128, 6
        kv = torch.randn(B * P * 64, 576, generator=g).to(torch.bfloat16)
        cache = O.pack_latent_cache(kv)
        table = torch.randperm(B * P, generator=g).int().view(B, P)
        idx = torch.stack([torch.randperm(P * 64, generator=g)[:K] for _ in range(B)]).int()
        idx[0, ::3] = -1
        idx[1, 1::2] = -1
        idx[2, : K // 2] = -1                                  # leading blocks empty, trailing ones used
        q = torch.randn(B, H, 576, generator=g).to(torch.bfloat16)
        out = ops.sparse_mla_decode_paged(q.cuda(), cache.cuda(), table.cuda(), idx.cuda(), 0.06)
        ops.check_status("cuda")
        check(out, O.sparse_mla_decode_paged(q.float(), cache, table, idx, 0.06, round_bf16=True))


def test_decode_bad_page_is_flagged():
    g = torch.Generator().manual_seed(2)
    kv = torch.randn(4 * 64, 576, generator=g).to(torch.bfloat16)
    cache = O.pack_latent_cache(kv)
    table = torch.tensor([[0, 1, 2, 9]], dtype=torch.int32)      # page 9 does not exist
    idx = torch.arange(256, dtype=torch.int32).view(1, 256)
    q = torch.randn(1, 128, 576, generator=g).to(torch.bfloat16)
    out = ops.sparse_mla_decode_paged(q.cuda(), cache.cuda(), table.cuda(), idx.cuda(), 0.06)
    with pytest.raises(ops.DsaError, match="out of range"):
        ops.check_status("cuda")
    ok = idx.clone()
    ok[0, 192:] = -1
    table[0, 3] = 3
    check(out, O.sparse_mla_decode_paged(q.float(), cache, table, ok, 0.06, round_bf16=True))


def test_decode_split_parts_match_the_single_part_path():
    """Few sequences with long slot lists take the split path (parts merged by a second kernel);
    a workspace too small for it forces the single-part path.  Both must agree."""
    from llmdivedeep_b200 import _lib
    B, H, P, K = 2, 128, 40, 2048
    g = torch.Generator().manual_seed(77)
    kv = torch.randn(B * P * 64, 576, generator=g).to(torch.bfloat16)
    cache = O.pack_latent_cache(kv).cuda()
    table = torch.randperm(B * P, generator=g).int().view(B, P).cuda()
    idx = torch.stack([torch.randperm(P * 64, generator=g)[:K] for _ in range(B)]).int()
    idx[1, 300:1500] = -1                                  # whole parts of sequence 1 are empty
    idx = idx.cuda()
    q = torch.randn(B, H, 576, generator=g).to(torch.bfloat16).cuda()
    assert _lib.load().dsa_sparse_mla_decode_workspace_bytes(B, H, K) > 0
    split = ops.sparse_mla_decode_paged(q, cache, table, idx, 0.06)
    single = ops.sparse_mla_decode_paged(q, cache, table, idx, 0.06, workspace=torch.empty(16, dtype=torch.uint8, device="cuda"))
    ops.check_status("cuda")
    assert float((split.float() - single.float()).abs().max()) <= 1e-2
    check(split, O.sparse_mla_decode_paged(q.float().cpu(), cache.cpu(), table.cpu(), idx.cpu(), 0.06, round_bf16=True))
