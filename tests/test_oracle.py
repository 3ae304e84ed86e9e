"""The oracle against the golden records of the unmodified reference
(tests/golden/reference_golden.npz, made by tests/golden/make_golden.py)."""
import os

import numpy as np
import pytest
import torch

from oracle import dsa_oracle as O

G = np.load(os.path.join(os.path.dirname(__file__), "golden", "reference_golden.npz"))


def bf16(a):
    return torch.from_numpy(a.view(np.int16).copy()).view(torch.bfloat16)


def fp8(a):
    return torch.from_numpy(a.copy()).view(torch.float8_e4m3fn)


@pytest.mark.parametrize("name", ["q", "k", "two"])
def test_quantiser_bit_exact(name):
    q8, sc = O.fp8_quant_per_block(bf16(G[f"quant_{name}_in"]))
    assert np.array_equal(q8.view(torch.uint8).numpy(), G[f"quant_{name}_fp8"])
    assert np.array_equal(sc.numpy(), G[f"quant_{name}_scale"])


def test_quantiser_zero_row_and_block_assert():
    q8, sc = O.fp8_quant_per_block(torch.zeros(2, 128, dtype=torch.bfloat16))
    assert float(sc[0]) == np.float32(np.float32(1e-6) / np.float32(448.0))
    assert (q8.float() == 0).all()
    with pytest.raises(AssertionError):
        O.fp8_quant_per_block(torch.zeros(2, 64, dtype=torch.bfloat16))   # DSA.py:117
    q8, sc = O.fp8_quant_per_block(torch.ones(2, 64, dtype=torch.bfloat16), block_size=64)
    assert sc.shape == (2,) and float(q8.float().max()) == 448.0


def _sim_inputs():
    q8, k8 = fp8(G["sim_q_fp8"]), fp8(G["sim_k_fp8"])
    ksc, w = torch.from_numpy(G["sim_k_scale"]), torch.from_numpy(G["sim_w"])
    S = k8.shape[0]
    ks = torch.zeros(S, dtype=torch.int32)
    ke = torch.arange(1, S + 1, dtype=torch.int32)
    return q8, k8, ksc, w, ks, ke


def test_scorer_without_relu_reproduces_reference_order():
    """relu=False must be the reference's fallback: the full per-row descending
    order of the valid (causal) part equals the recorded one."""
    q8, k8, ksc, w, ks, ke = _sim_inputs()
    logits = O.indexer_logits(q8, k8, ksc, w, ks, ke, relu=False)
    order = O.topk_indices(logits, logits.shape[1]).numpy()
    ref = G["sim_order"]
    for t in range(order.shape[0]):
        n = t + 1
        assert np.array_equal(order[t, :n], ref[t, :n]), t
    top16 = O.topk_indices(logits, 16).numpy()
    for t in range(16, order.shape[0]):
        assert np.array_equal(top16[t], G["sim_top16"][t])


def test_relu_changes_the_selection():
    """The ReLU of the math note is not a no-op: on the same inputs the top-16
    sets differ from the reference fallback's on a good share of rows."""
    q8, k8, ksc, w, ks, ke = _sim_inputs()
    a = O.topk_indices(O.indexer_logits(q8, k8, ksc, w, ks, ke, relu=True), 16).numpy()
    differ = sum(set(a[t]) != set(G["sim_top16"][t]) for t in range(32, a.shape[0]))
    assert differ > 10


def test_fp64_scores_agree_with_fp32():
    q8, k8, ksc, w, ks, ke = _sim_inputs()
    a = O.indexer_logits(q8, k8, ksc, w, ks, ke, relu=True)
    b = O.indexer_logits_fp64(q8, k8, ksc, w, ks, ke, relu=True)
    m = torch.isfinite(a)
    assert torch.equal(m, torch.isfinite(b))
    assert float((a[m].double() - b[m]).abs().max()) < 1e-4 * float(b[m].abs().max())


def _params(tag):
    p = {k: bf16(G[f"mod_{tag}_{k}"]) for k in ("wq_b", "wk", "weights_proj", "k_norm_w", "k_norm_b")}
    if f"mod_{tag}_pool_proj" in G:
        p["pool_proj"] = bf16(G[f"mod_{tag}_pool_proj"])
    return p


@pytest.mark.parametrize("tag,interleave", [("neox", False), ("glm", True)])
def test_dsa_indexer_forward_matches_reference(tag, interleave):
    x, ql = bf16(G[f"mod_{tag}_x"]), bf16(G[f"mod_{tag}_qlora"])
    idx = O.dsa_indexer_forward(_params(tag), x, ql, 4, 128, 64, 24, interleave=interleave,
                                relu=False).numpy()
    ref = G[f"mod_{tag}_idx"]
    assert idx.shape == ref.shape
    for t in range(idx.shape[0]):
        n = min(t + 1, idx.shape[1])
        assert np.array_equal(idx[t, :n], ref[t, :n]), t


def test_dsv4_indexer_forward_matches_reference():
    x, ql = bf16(G["mod_c4_x"]), bf16(G["mod_c4_qlora"])
    idx = O.dsv4_indexer_forward(_params("c4"), x, ql, 4, 128, 64, 24, compress_ratio=4,
                                 relu=False).numpy()
    ref = G["mod_c4_idx"]
    assert idx.shape == ref.shape == (128, 6)
    for t in range(idx.shape[0]):
        n = min((t + 4) // 4, idx.shape[1])
        assert np.array_equal(idx[t, :n], ref[t, :n]), t


def test_sparse_mla_equals_dense_softmax_when_all_selected():
    torch.manual_seed(3)
    T, H, D = 12, 3, 576
    q, kv = torch.randn(T, H, D), torch.randn(T, D)
    idx = torch.full((T, T), -1, dtype=torch.int32)
    for t in range(T):
        idx[t, :t + 1] = torch.randperm(t + 1).int()
    out = O.sparse_mla(q, kv, idx, 0.07, dtype=torch.float64)
    s = torch.einsum("thd,sd->ths", q.double(), kv.double()) * 0.07
    s = s.masked_fill(~torch.tril(torch.ones(T, T, dtype=torch.bool)).unsqueeze(1), float("-inf"))
    want = torch.einsum("ths,sd->thd", torch.softmax(s, -1), kv.double()[:, :512])
    assert float((out - want).abs().max()) < 1e-12
    empty = O.sparse_mla(q[:1], kv, torch.full((1, 4), -1, dtype=torch.int32), 0.07)
    assert float(empty.abs().max()) == 0.0


def test_latent_cache_round_trip_and_paging():
    torch.manual_seed(4)
    kv = torch.randn(256, 576).to(torch.bfloat16)
    rec = O.pack_latent_cache(kv)
    assert rec.shape == (256, 656)
    back = O.unpack_latent_cache(rec)
    assert torch.equal(back[:, 512:], kv[:, 512:].float())
    err = (back[:, :512] - kv[:, :512].float()).abs().max()
    assert float(err) < 0.07 * float(kv.float().abs().max())
    table = torch.tensor([3, 1, 0, 2], dtype=torch.int32)
    pos = torch.tensor([0, 63, 64, 130, 255])
    assert O.physical_rows(table, pos).tolist() == [192, 255, 64, 2, 191]


def test_decode_paged_equals_gathered_dense():
    torch.manual_seed(5)
    B, H, P = 2, 4, 3
    kv = torch.randn(B * P * 64, 576).to(torch.bfloat16)
    cache = O.pack_latent_cache(kv)
    table = torch.randperm(B * P).int().view(B, P)
    idx = torch.stack([torch.randperm(P * 64)[:40] for _ in range(B)]).int()
    idx[1, 30:] = -1
    q = torch.randn(B, H, 576)
    out = O.sparse_mla_decode_paged(q, cache, table, idx, 0.05)
    deq = O.unpack_latent_cache(cache)
    for b in range(B):
        ii = idx[b][idx[b] >= 0].long()
        rows = O.physical_rows(table[b], ii)
        s = torch.softmax((q[b] @ deq[rows].T) * 0.05, -1)
        assert float((out[b] - s @ deq[rows][:, :512]).abs().max()) < 1e-5


def test_check_topk_sets_rules():
    sc = np.array([[5, 4, 3, 2, 1, 0]], dtype=np.float32)
    ok = O.check_topk_sets(np.array([[1, 0, 2]]), sc, [0], [6], 3)
    assert ok["exact_rows"] == 1 and not ok["bad_rows"]
    assert O.check_topk_sets(np.array([[1, 0, 3]]), sc, [0], [6], 3)["bad_rows"] == [0]
    assert O.check_topk_sets(np.array([[1, 1, 0]]), sc, [0], [6], 3)["bad_rows"] == [0]
    assert O.check_topk_sets(np.array([[1, 0, -1]]), sc, [0], [2], 3)["exact_rows"] == 1
    assert O.check_topk_sets(np.array([[1, 0, 5]]), sc, [0], [2], 3)["bad_rows"] == [0]
    tie = np.array([[1, 1, 1, 0]], dtype=np.float32)
    assert O.check_topk_sets(np.array([[3 - 1, 0]]), tie, [0], [4], 2)["exact_rows"] == 1


def test_block_sparse_oracle_with_every_block_listed_is_full_attention():
    """The block-sparse MHA restatement reduces to plain softmax attention when every key block is listed."""
    g = torch.Generator().manual_seed(0)
    q, k, v = (torch.randn(1, 256, 2, 128, generator=g) for _ in range(3))
    nb = 4
    lut = torch.arange(nb, dtype=torch.int32).expand(1, 2, nb, nb).contiguous()
    num = torch.full((1, 2, nb), nb, dtype=torch.int32)
    got = O.block_sparse_mha(q, k, v, lut, num, 128 ** -0.5)
    full = torch.nn.functional.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2),
                                                            v.transpose(1, 2)).transpose(1, 2)
    assert float((got - full).abs().max()) < 1e-5
    num[0, 1, 2] = 0
    assert float(O.block_sparse_mha(q, k, v, lut, num, 0.1)[0, 128:192, 1].abs().max()) == 0.0
