"""The DSA-module mirror (llmdivedeep_b200/DSA.py) on a GPU: same names and call surface as
the reference's sparse_attn/DSA.py, results checked against the CPU oracle (ReLU scorer)."""
import os

import numpy as np
import pytest
import torch

from llmdivedeep_b200 import DSA, ops
from oracle import dsa_oracle as O

pytestmark = pytest.mark.gpu
G = np.load(os.path.join(os.path.dirname(__file__), "golden", "reference_golden.npz"))
ULP_TOL = 4.0


def bf16(a):
    return torch.from_numpy(a.view(np.int16).copy()).view(torch.bfloat16)


def test_exports_the_names_the_reference_drivers_import():
    for n in ("INDEXER_BLOCK_SIZE INDEXER_HEAD_DIM INDEXER_N_HEADS INDEXER_TOPK SPARSE_BLOCK IndexerSimulator "
              "env_report register_dense_fn register_fa4 register_sparse_fa try_import_deep_gemm SPECS DsaIndexer "
              "Dsv4Indexer IndexerSpec fp8_quant_per_block C4Compressor").split():
        assert hasattr(DSA, n), n
    assert (DSA.INDEXER_N_HEADS, DSA.INDEXER_HEAD_DIM, DSA.INDEXER_TOPK, DSA.SPARSE_BLOCK) == (64, 128, 2048, 64)
    assert set(DSA.SPECS) == {"dsv32", "glm", "dsv4"} and DSA.SPECS["dsv4"].compress_ratio == 4
    assert hasattr(DSA.try_import_deep_gemm(), "fp8_mqa_logits")
    assert "libdsa_b200" in DSA.env_report()


@pytest.mark.parametrize("name", ["q", "k", "two"])
def test_quantiser_matches_reference_bytes(name):
    """The fused quantiser kernel against the records of the reference's CPU run: bit-exact
    (bytes and scales), including the all-zero row and the two-blocks-per-row case."""
    q8, sc = DSA.fp8_quant_per_block(bf16(G[f"quant_{name}_in"]).cuda())
    assert np.array_equal(sc.cpu().numpy(), G[f"quant_{name}_scale"])
    assert np.array_equal(q8.view(torch.uint8).cpu().numpy(), G[f"quant_{name}_fp8"])
    with pytest.raises(AssertionError):
        DSA.fp8_quant_per_block(torch.zeros(2, 64, device="cuda"))


@pytest.mark.parametrize("shape,block,dtype", [((1000, 64, 128), 128, torch.bfloat16), ((4097, 128), 128, torch.float32),
                                               ((300, 4, 64), 64, torch.float32), ((77, 256), 64, torch.bfloat16),
                                               ((5, 3, 384), 128, torch.float32)])
def test_quantiser_kernel_matches_oracle_bitwise(shape, block, dtype):
    g = torch.Generator().manual_seed(sum(shape))
    x = (torch.randn(*shape, generator=g) * torch.rand(*shape[:-1], 1, generator=g) * 30).to(dtype)
    x.view(-1, shape[-1])[::7] *= 1e-4                      # small rows: e4m3 subnormals
    x.view(-1, shape[-1])[3] = 0
    want_q, want_s = O.fp8_quant_per_block(x, block)
    q8, sc = ops.fp8_quant_per_block(x.cuda(), block)
    assert sc.shape == want_s.shape and torch.equal(sc.cpu(), want_s)
    assert torch.equal(q8.view(torch.uint8).cpu(), want_q.view(torch.uint8))


def _load_golden_weights(mod, tag):
    sd = {"wq_b.weight": bf16(G[f"mod_{tag}_wq_b"]), "wk.weight": bf16(G[f"mod_{tag}_wk"]),
          "weights_proj.weight": bf16(G[f"mod_{tag}_weights_proj"]), "k_norm.weight": bf16(G[f"mod_{tag}_k_norm_w"]),
          "k_norm.bias": bf16(G[f"mod_{tag}_k_norm_b"])}
    if f"mod_{tag}_pool_proj" in G:
        sd["compressor.pool_proj.weight"] = bf16(G[f"mod_{tag}_pool_proj"])
    mod.load_state_dict(sd)
    return mod.cuda()


@pytest.mark.parametrize("tag,cr,il", [("neox", 1, False), ("glm", 1, True), ("c4", 4, False)])
@torch.no_grad()
def test_module_forward_on_the_golden_weights(tag, cr, il):
    """Reference weights and inputs; the module's own stages (projections, RoPE) are taken from
    the GPU and the selection is checked against the oracle scoring exactly those values."""
    spec = DSA.IndexerSpec(tag, 64, 32, 4, 128, 64, 24, cr, il)
    mod = _load_golden_weights((DSA.Dsv4Indexer if cr > 1 else DSA.DsaIndexer)(spec), tag)
    x, ql = bf16(G[f"mod_{tag}_x"]).cuda(), bf16(G[f"mod_{tag}_qlora"]).cuda()
    T = x.shape[0]
    idx = mod(x, ql)
    ops.check_status("cuda")
    K = min(24 // cr, T // cr)
    assert idx.shape == G[f"mod_{tag}_idx"].shape == (T, K) and idx.dtype == torch.int64
    # recompute the stage outputs the way forward() does and score them with the oracle
    q = mod.wq_b(ql).view(T, 4, 128)
    k = mod.k_norm(mod.compressor(x) if cr > 1 else mod.wk(x))
    w = mod.weights_proj(x).float() * 4 ** -0.5
    q = DSA._rope_head(q, 64, T, il)
    k = DSA._rope_head(k, 64, T // cr, il)
    q8, qs = (t.cpu() for t in DSA.fp8_quant_per_block(q))      # the module's own FP8 values
    k8, ksc = (t.cpu() for t in DSA.fp8_quant_per_block(k))
    ks = torch.zeros(T, dtype=torch.int32)
    ke = ((torch.arange(1, T + 1) + cr - 1) // cr).to(torch.int32)
    ref = O.indexer_logits_fp64(q8, k8, ksc, O.fold_weights(w.cpu(), qs, 128), ks, ke).numpy()
    r = O.check_topk_sets(idx.cpu().numpy(), ref, ks.numpy(), ke.numpy(), K, ulp_tol=ULP_TOL)
    assert not r["bad_rows"], r


def test_rope_matches_the_oracle_forms():
    x = torch.randn(10, 3, 64)
    cos, sin = O.rope_cossin(10, 64)
    assert torch.equal(DSA._rotate(x, cos, sin, False), O.apply_rope_neox(x, cos, sin))
    assert torch.equal(DSA._rotate(x, cos, sin, True), O.apply_rope_interleave(x, cos, sin))


@torch.no_grad()
def test_indexer_simulator_surface_and_result():
    torch.manual_seed(0)
    sim = DSA.IndexerSimulator(S=1024, topk=128, hidden_size=256, q_lora_rank=64)
    q, k, w = sim.projections_step()
    assert q.shape == (1024, 64, 128) and k.shape == (1024, 128) and w.shape == (1024, 64) and w.dtype == torch.float32
    q8, qs, k8, ksc = sim.quantize_step(q, k)
    assert q8.dtype == torch.float8_e4m3fn and qs.shape == (1024, 64) and ksc.shape == (1024,)
    sim.precompute_fp8()
    idx = sim.logits_step()
    ops.check_status("cuda")
    assert idx.shape == (1024, 128) and idx.dtype == torch.int64
    q8, k8, ksc, weff = (t.cpu() for t in sim._fp8_cache)
    ref = O.indexer_logits_fp64(q8, k8, ksc, weff, sim.ks.cpu(), sim.ke.cpu()).numpy()
    r = O.check_topk_sets(idx.cpu().numpy(), ref, sim.ks.cpu().numpy(), sim.ke.cpu().numpy(), 128, ulp_tol=ULP_TOL)
    assert not r["bad_rows"], r


def test_deep_gemm_seam_returns_clean_logits():
    """What the unmodified reference would receive through try_import_deep_gemm()."""
    from tests.helpers import indexer_inputs
    q8, k8, ksc, w, ks, ke = indexer_inputs(64, 512, 64, 128, seed=6, window="causal")
    dg = DSA.try_import_deep_gemm()
    logits = dg.fp8_mqa_logits(q8.cuda(), (k8.cuda(), ksc.cuda()), w.cuda(), ks.cuda(), ke.cuda())
    assert logits.shape == (64, 512) and logits.dtype == torch.float32
    top = logits.topk(32, dim=-1).indices.cpu().numpy()
    ref = O.indexer_logits_fp64(q8, k8, ksc, w, ks, ke).numpy()
    r = O.check_topk_sets(top, ref, ks.numpy(), ke.numpy(), 32, ulp_tol=ULP_TOL)
    assert not r["bad_rows"], r


@pytest.mark.parametrize("D,rd,interleave", [(128, 64, False), (128, 64, True), (64, 64, False), (64, 32, True), (128, 128, False)])
def test_fused_rope_quantiser_equals_the_eager_chain_bitwise(D, rd, interleave):
    """dsa_rope_fp8_quant against RoPE with separate torch ops followed by the quantiser: on the GPU with the GPU's own
    cos / sin tables (what the module does), and against the CPU oracle chain with the CPU's tables."""
    T, H = 173, 5
    g = torch.Generator().manual_seed(D + rd)
    q = (torch.randn(T, H, D, generator=g) * 3).to(torch.bfloat16)
    k = torch.randn(T, D, generator=g).to(torch.bfloat16)
    k[7] = 0
    cos_c, sin_c = O.rope_cossin(T, rd)
    for x, rpp in ((q, H), (k, 1)):
        # CPU oracle chain, CPU tables
        rot = (O.apply_rope_interleave if interleave else O.apply_rope_neox)(x[..., :rd], cos_c, sin_c)
        want8, want_s = O.fp8_quant_per_block(torch.cat([rot, x[..., rd:]], dim=-1), D)
        got8, got_s = ops.rope_fp8_quant(x.cuda(), cos_c.cuda(), sin_c.cuda(), rd, interleave, rpp)
        assert torch.equal(got8.cpu().view(torch.uint8), want8.view(torch.uint8)) and torch.equal(got_s.cpu(), want_s)
        # eager GPU chain, GPU tables
        cos_g, sin_g = DSA._rope_cossin(T, rd, torch.device("cuda"))
        e8, e_s = DSA.fp8_quant_per_block(DSA._rope_head(x.cuda(), rd, T, interleave), D)
        f8, f_s = ops.rope_fp8_quant(x.cuda(), cos_g, sin_g, rd, interleave, rpp)
        assert torch.equal(f8.view(torch.uint8), e8.view(torch.uint8)) and torch.equal(f_s, e_s)


def test_fused_rope_quantiser_refuses_bad_shapes():
    x = torch.zeros(4, 128, dtype=torch.bfloat16, device="cuda")
    t = torch.zeros(4, 24, device="cuda")
    with pytest.raises(ops.DsaError):
        ops.rope_fp8_quant(x, t, t, 48, False)            # 24 dims per half = 6 lanes: not a power of two
    with pytest.raises(ops.DsaError):
        ops.rope_fp8_quant(x, t[:2, :16].contiguous(), t[:2, :16].contiguous(), 32, False)   # 4 rows, 2 positions
