"""dsa_block_sparse_mha (through the C ABI) against the CPU oracle.  bf16 in, fp32 accumulate, bf16 out:
max |err| <= 2e-2, mean |err| <= 2e-3 on outputs of order one (the tolerance of the sparse-MLA tests)."""
import pytest
import torch

from llmdivedeep_b200 import DSA, ops
from oracle import dsa_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda"
MAX_ABS, MEAN_ABS = 2e-2, 2e-3


def _case(B, S, H, topk, seed, ragged=False):
    g = torch.Generator().manual_seed(seed)
    q, k, v = (torch.randn(B, S, H, 128, generator=g).bfloat16() for _ in range(3))
    nb = S // 64
    lut = torch.stack([torch.randperm(nb, generator=g)[:topk] for _ in range(B * H * nb)]).view(B, H, nb, topk).int()
    num = torch.full((B, H, nb), topk, dtype=torch.int32)
    if ragged:
        num = torch.randint(0, topk + 1, (B, H, nb), generator=g, dtype=torch.int32)
    return q, k, v, lut, num


def _check(q, k, v, lut, num, scale):
    want = O.block_sparse_mha(q, k, v, lut, num, scale)
    got = ops.block_sparse_attn(q.to(DEV), k.to(DEV), v.to(DEV), lut.to(DEV), num.to(DEV), scale).float().cpu()
    err = (got - want).abs()
    assert float(err.max()) <= MAX_ABS and float(err.mean()) <= MEAN_ABS, (float(err.max()), float(err.mean()))
    ops.check_status(DEV)
    return got


@pytest.mark.parametrize("B,S,H,topk", [(1, 256, 2, 1), (1, 512, 3, 4), (2, 1024, 2, 16), (1, 2048, 24, 2)])
def test_matches_oracle(B, S, H, topk):
    _check(*_case(B, S, H, topk, seed=S + topk), 128 ** -0.5)


def test_ragged_lists_and_empty_blocks():
    q, k, v, lut, num = _case(1, 1024, 3, 8, seed=5, ragged=True)
    num[0, 0, 0] = 0                                   # a query block with an empty list: zero rows
    got = _check(q, k, v, lut, num, 0.1)
    assert float(got[0, :64, 0].abs().max()) == 0.0


def test_dense_list_equals_full_attention():
    B, S, H = 1, 512, 2
    q, k, v, _, _ = _case(B, S, H, 1, seed=9)
    nb = S // 64
    lut = torch.arange(nb, dtype=torch.int32).expand(B, H, nb, nb).contiguous()
    num = torch.full((B, H, nb), nb, dtype=torch.int32)
    got = _check(q, k, v, lut, num, 128 ** -0.5)
    full = torch.nn.functional.scaled_dot_product_attention(q.float().transpose(1, 2), k.float().transpose(1, 2),
                                                            v.float().transpose(1, 2)).transpose(1, 2)
    assert float((got - full).abs().max()) <= MAX_ABS


def test_large_scores_stay_finite():
    q, k, v, lut, num = _case(1, 512, 2, 4, seed=11)
    got = _check(q * 6, k * 6, v, lut, num, 128 ** -0.5)       # scores of order +-400: exercises the lazy rescale
    assert torch.isfinite(got).all()


def test_bad_block_id_sets_status_and_is_skipped():
    q, k, v, lut, num = _case(1, 512, 2, 4, seed=13)
    bad = lut.clone()
    bad[0, 1, 3, 2] = 99                               # outside [0, 8)
    want = O.block_sparse_mha(q, k, v, bad, num, 0.1)  # the oracle drops ids outside the range
    ops.status_word(DEV).zero_()
    got = ops.block_sparse_attn(q.to(DEV), k.to(DEV), v.to(DEV), bad.to(DEV), num.to(DEV), 0.1).float().cpu()
    torch.cuda.synchronize()
    assert int(ops.status_word(DEV).item()) == 2
    ops.status_word(DEV).zero_()
    assert float((got - want).abs().max()) <= MAX_ABS


def test_register_sparse_fa_pair_runs_like_the_reference_driver():
    pair = DSA.register_sparse_fa()
    assert pair is not None
    build_lut, run = pair
    S = 1024
    q, k, v = (torch.randn(1, S, 24, 128, device=DEV, dtype=torch.bfloat16) for _ in range(3))
    idx, num, topk = build_lut(q, S, 0.25)
    assert idx.shape == (1, 24, S // 64, topk) and num.shape == (1, 24, S // 64) and topk == 4
    out = run(q, k, v, idx, num, 128 ** -0.5)
    want = O.block_sparse_mha(q.cpu(), k.cpu(), v.cpu(), idx.cpu(), num.cpu(), 128 ** -0.5)
    assert out.shape == q.shape and float((out.float().cpu() - want).abs().max()) <= MAX_ABS
