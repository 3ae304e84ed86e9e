"""Generate the golden fixtures in this directory from the UNMODIFIED reference.

Run where the reference checkout is available:

    python tests/golden/make_golden.py /path/to/reference

It imports ``sparse_attn/DSA.py`` from that checkout (CPU, fp32 fallback
scorer -- none of the optional GPU backends resolve there), feeds it seeded
inputs and stores inputs and outputs in ``reference_golden.npz``.  The tests
never import the reference; they read the ``.npz``.

Recorded cases
  quant_*      fp8_quant_per_block on [T,H,128], [T,128] and a 2-block row
  sim_*        IndexerSimulator(device=cpu): FP8 cache, folded weights and the
               FULL descending order of every row (topk = S), which pins the
               scorer's values far more tightly than a top-k set would
  mod_*        DsaIndexer.forward (NeoX and interleaved RoPE) and
               Dsv4Indexer.forward: weights, inputs, returned indices; for the
               DsaIndexer cases also the FP8 bytes, scales and head gates that
               forward() hands to the scorer
"""
import os
import sys

import numpy as np
import torch


def _u16(t):  # bf16 tensor -> uint16 numpy
    return t.detach().contiguous().view(torch.int16).numpy().view(np.uint16)


def _u8(t):   # fp8 tensor -> uint8 numpy
    return t.detach().contiguous().view(torch.uint8).numpy()


@torch.no_grad()
def main(ref_root: str) -> None:
    sys.path.insert(0, os.path.join(ref_root, "sparse_attn"))
    import DSA  # the reference module

    out = {}
    cpu = torch.device("cpu")

    # ---- quantiser -------------------------------------------------------
    g = torch.Generator().manual_seed(1)
    xq = torch.randn(24, 4, 128, generator=g).to(torch.bfloat16)
    xk = torch.randn(40, 128, generator=g).to(torch.bfloat16)
    xk[3] = 0                                   # all-zero row -> clamp path
    x2 = (torch.randn(8, 256, generator=g) * 5).to(torch.bfloat16)
    for name, x in (("q", xq), ("k", xk), ("two", x2)):
        q8, sc = DSA.fp8_quant_per_block(x)
        out[f"quant_{name}_in"] = _u16(x)
        out[f"quant_{name}_fp8"] = _u8(q8)
        out[f"quant_{name}_scale"] = sc.detach().numpy()

    # ---- IndexerSimulator -------------------------------------------------
    torch.manual_seed(0)
    S, H, D = 192, 4, 128
    sim = DSA.IndexerSimulator(S=S, n_heads=H, head_dim=D, topk=S, device=cpu,
                               hidden_size=96, q_lora_rank=48)
    sim.precompute_fp8()
    q8, k8, ksc, w = sim._fp8_cache
    out["sim_q_fp8"] = _u8(q8)
    out["sim_k_fp8"] = _u8(k8)
    out["sim_k_scale"] = ksc.detach().numpy()
    out["sim_w"] = w.detach().numpy()
    out["sim_order"] = sim.logits_step().numpy().astype(np.int32)      # [S,S] full order
    sim.topk = 16
    out["sim_top16"] = sim.logits_step().numpy().astype(np.int32)

    # ---- nn.Module indexers ------------------------------------------------
    def run_module(tag, spec, cls, T):
        torch.manual_seed(7)
        mod = cls(spec, dtype=torch.bfloat16)
        with torch.no_grad():
            mod.k_norm.weight.add_(0.1 * torch.randn_like(mod.k_norm.weight))
            mod.k_norm.bias.add_(0.1 * torch.randn_like(mod.k_norm.bias))
        x = torch.randn(T, spec.hidden_size).to(torch.bfloat16)
        ql = torch.randn(T, spec.q_lora_rank).to(torch.bfloat16)
        idx = mod(x, ql)
        out[f"mod_{tag}_x"] = _u16(x)
        out[f"mod_{tag}_qlora"] = _u16(ql)
        out[f"mod_{tag}_idx"] = idx.numpy().astype(np.int32)
        sd = mod.state_dict()
        out[f"mod_{tag}_wq_b"] = _u16(sd["wq_b.weight"])
        out[f"mod_{tag}_wk"] = _u16(sd["wk.weight"])
        out[f"mod_{tag}_weights_proj"] = _u16(sd["weights_proj.weight"])
        out[f"mod_{tag}_k_norm_w"] = _u16(sd["k_norm.weight"])
        out[f"mod_{tag}_k_norm_b"] = _u16(sd["k_norm.bias"])
        if "compressor.pool_proj.weight" in sd:
            out[f"mod_{tag}_pool_proj"] = _u16(sd["compressor.pool_proj.weight"])
        else:
            # the stage outputs forward() feeds to the scorer (projections -> RoPE -> FP8 quantiser)
            q, k, w = mod.projections(x, ql)
            q, k = mod.rope(q, k)
            q8, qs = DSA.fp8_quant_per_block(q)
            k8, ksc = DSA.fp8_quant_per_block(k)
            out[f"mod_{tag}_q_fp8"] = _u8(q8)
            out[f"mod_{tag}_q_scale"] = qs.detach().numpy()
            out[f"mod_{tag}_k_fp8"] = _u8(k8)
            out[f"mod_{tag}_k_scale"] = ksc.detach().numpy()
            out[f"mod_{tag}_w"] = w.detach().numpy()

    mk = lambda name, cr, il: DSA.IndexerSpec(name=name, hidden_size=64, q_lora_rank=32,
                                              index_n_heads=4, index_head_dim=128,
                                              rope_head_dim=64, index_topk=24,
                                              compress_ratio=cr, rope_interleave=il)
    run_module("neox", mk("neox", 1, False), DSA.DsaIndexer, 96)
    run_module("glm", mk("glm", 1, True), DSA.DsaIndexer, 96)
    run_module("c4", mk("c4", 4, False), DSA.Dsv4Indexer, 128)

    dst = os.path.join(os.path.dirname(os.path.abspath(__file__)), "reference_golden.npz")
    np.savez_compressed(dst, **out)
    print("wrote", dst, os.path.getsize(dst), "bytes,", len(out), "arrays")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: python tests/golden/make_golden.py /path/to/reference")
    main(sys.argv[1])
