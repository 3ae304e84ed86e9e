"""Seeded input builders shared by the parity tests."""
import torch

from oracle import dsa_oracle as O


def indexer_inputs(T, S, H, D, seed, window="causal", w_bf16=False):
    """FP8-quantised q/k with per-row scales (sparse_attn/DSA.py:102-132 semantics),
    folded head weights and a [ks, ke) window per query row.
    window: 'causal' (queries are the last T positions of S), 'random', 'full'."""
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(T, H, D, generator=g)
    k = torch.randn(S, D, generator=g)
    q8, qs = O.fp8_quant_per_block(q, D)
    k8, ksc = O.fp8_quant_per_block(k, D)
    w = torch.randn(T, H, generator=g) / 8
    w_eff = O.fold_weights(w, qs, D)
    if w_bf16:
        w_eff = w_eff.to(torch.bfloat16)
    if window == "causal":
        ks = torch.zeros(T, dtype=torch.int32)
        ke = (torch.arange(T) + (S - T) + 1).to(torch.int32)
    elif window == "random":
        ks = torch.randint(0, max(S // 3, 1), (T,), generator=g).to(torch.int32)
        ke = torch.randint(S // 2, S + 1, (T,), generator=g).to(torch.int32)
    else:
        ks = torch.zeros(T, dtype=torch.int32)
        ke = torch.full((T,), S, dtype=torch.int32)
    return q8, k8, ksc, w_eff, ks, ke


def to_dev(*ts, device="cuda"):
    return tuple(t.to(device) for t in ts)
