"""CPU oracle for the DeepSeek Sparse Attention (DSA) hot path.

TEST INFRASTRUCTURE ONLY.  This file is the checker the CUDA kernels are
compared against; nothing in the product package imports it.  It restates, in
plain torch-on-CPU / numpy arithmetic, what the reference computes:

* ``fp8_quant_per_block``      <- sparse_attn/DSA.py:102-132
* ``fold_weights``             <- sparse_attn/DSA.py:327-331, 540-543
* ``indexer_logits``           <- sparse_attn/DSA.py:348-360 (square tril mask),
                                   661-673 (general ``arange < ke`` mask)
* ``topk_indices``             <- sparse_attn/DSA.py:361, 567, 675-676
* ``rope_cossin`` / ``apply_rope_*`` <- sparse_attn/DSA.py:430-469
* ``dsa_indexer_forward``      <- sparse_attn/DSA.py:527-568
* ``dsv4_indexer_forward``     <- sparse_attn/DSA.py:619-676
* ``sparse_mla`` (pattern)     <- sparse_attn/bench_sparse_attention_kernels.py:421-442
                                   (query-block streamed fp32 attention)

Parity pin: with ``relu=False`` the indexer functions reproduce the unmodified
reference's fp32 fallback bit for bit; ``tests/golden/make_golden.py`` imports
the reference, records its outputs, and ``tests/test_oracle.py`` checks this
file against those records.  The reference's fallback has no ReLU although its
own math note (sparse_attn/ATTENTION_MATH.md:56-60) and the production kernel
it stands in for have one, so ``relu=True`` is the parity target for the CUDA
kernels.  Sparse MLA, the paged FP8 latent cache and decode have no reference
implementation at all: those functions restate the published DSA math and are
"parity unpinned" (no reference output exists to pin them to).
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import numpy as np
import torch

FP8 = torch.float8_e4m3fn
FP8_MAX = 448.0


# --------------------------------------------------------------------------
# FP8 per-block quantiser                      (sparse_attn/DSA.py:102-132)
# --------------------------------------------------------------------------
def fp8_quant_per_block(x: torch.Tensor, block_size: int = 128):
    """fp32 absmax per block, clamp 1e-6, scale = absmax/448, q = x/scale -> e4m3.

    The scale is squeezed to the leading dims when a row is one block
    (DSA.py:127-129), otherwise it keeps a trailing ``num_blocks`` dim.
    """
    shape = x.shape
    last = shape[-1]
    if last % block_size:
        raise AssertionError(f"last dim {last} not multiple of block {block_size}")
    nb = last // block_size
    xf = x.reshape(-1, last).to(torch.float32).view(-1, nb, block_size)
    absmax = xf.abs().amax(dim=-1, keepdim=True).clamp_min(1e-6)
    scale = absmax / FP8_MAX
    q = (xf / scale).to(FP8).view(*shape)
    scale = scale.squeeze(-1).to(torch.float32)
    scale = scale.view(*shape[:-1]) if nb == 1 else scale.view(*shape[:-1], nb)
    return q, scale


def fold_weights(w: torch.Tensor, q_scale: torch.Tensor, head_dim: int) -> torch.Tensor:
    """w_eff = w * q_scale * head_dim**-0.5   (DSA.py:327-331)."""
    sm = head_dim ** -0.5
    if q_scale.dim() == 2:
        return (w.float() * q_scale.float() * sm).contiguous()
    return (w.float() * q_scale.float().mean(dim=-1) * sm).contiguous()


# --------------------------------------------------------------------------
# Lightning indexer logits
# --------------------------------------------------------------------------
def indexer_logits(q_fp8, k_fp8, k_scale, w, ks, ke, relu: bool = True,
                   row_chunk: int = 256) -> torch.Tensor:
    """logits[t,s] = sum_h w[t,h] * act(q[t,h,:] . (k[s,:]*k_scale[s])), -inf outside [ks,ke).

    Same operation order as the reference fallback (DSA.py:348-357): both
    operands go to fp32, k is scaled *before* the dot, the head products are
    multiplied by w and summed with ``Tensor.sum(dim=1)``.  ``relu=False`` is
    the reference as written; ``relu=True`` inserts the ReLU of
    ATTENTION_MATH.md:57.  Rows are streamed in chunks (the reference
    materialises [T,H,S]); chunking does not change any value because every
    output element depends on one query row only.
    """
    T, H, D = q_fp8.shape
    S = k_fp8.shape[0]
    qf = q_fp8.to(torch.float32)
    kf = k_fp8.to(torch.float32) * k_scale.to(torch.float32).unsqueeze(-1)
    wf = w.to(torch.float32)
    out = torch.empty(T, S, dtype=torch.float32)
    cols = torch.arange(S).unsqueeze(0)
    for r0 in range(0, T, row_chunk):
        r1 = min(T, r0 + row_chunk)
        sc = torch.einsum("thd,sd->ths", qf[r0:r1], kf)
        if relu:
            sc = torch.relu(sc)
        sc = (sc * wf[r0:r1].unsqueeze(-1)).sum(dim=1)
        valid = (cols >= ks[r0:r1].long().unsqueeze(1)) & (cols < ke[r0:r1].long().unsqueeze(1))
        out[r0:r1] = sc.masked_fill(~valid, float("-inf"))
    return out


def indexer_logits_fp64(q_fp8, k_fp8, k_scale, w, ks, ke, relu: bool = True,
                        row_chunk: int = 128) -> torch.Tensor:
    """The same scores in float64: e4m3*e4m3 products and 128-term sums are exact
    there, so this is the adjudicator for near-ties at the k-th score."""
    T, H, D = q_fp8.shape
    S = k_fp8.shape[0]
    qf = q_fp8.to(torch.float64)
    kf = k_fp8.to(torch.float64)
    ksc = k_scale.to(torch.float64)
    wf = w.to(torch.float64)
    out = torch.empty(T, S, dtype=torch.float64)
    cols = torch.arange(S).unsqueeze(0)
    for r0 in range(0, T, row_chunk):
        r1 = min(T, r0 + row_chunk)
        sc = torch.einsum("thd,sd->ths", qf[r0:r1], kf)
        if relu:
            sc = torch.relu(sc)
        sc = (sc * wf[r0:r1].unsqueeze(-1)).sum(dim=1) * ksc.unsqueeze(0)
        valid = (cols >= ks[r0:r1].long().unsqueeze(1)) & (cols < ke[r0:r1].long().unsqueeze(1))
        out[r0:r1] = sc.masked_fill(~valid, float("-inf"))
    return out


def topk_indices(logits: torch.Tensor, k: int) -> torch.Tensor:
    """``logits.topk(min(k, S)).indices`` (DSA.py:361): int64, sorted descending."""
    return logits.topk(min(k, logits.shape[-1]), dim=-1).indices


def check_topk_sets(sel: np.ndarray, scores: np.ndarray, ks, ke, k: int,
                    ulp_tol: float = 0.0):
    """Check selected index sets against scores.

    sel    [T, K] int (entries < 0 are padding); scores [T, S] float (the
    checker's scores; masked entries may hold anything).  For each row the
    valid window is [ks, ke).  Returns a dict with
      exact_rows      rows whose set equals the checker's top-k set exactly
                      (ties at the k-th value may be broken either way),
      bad_rows        rows that break a hard rule (out of window, duplicate,
                      wrong count, or a swap further than ``ulp_tol`` fp32 ulps
                      of the k-th score away from it),
      max_ulp         the largest distance, in fp32 ulps of the k-th score, of
                      any swapped element from the k-th score,
      swapped_rows    rows whose set differs from the checker's by near-ties,
      rows_over_1ulp  how many of those have a swap further than 1.0 ulp away
                      (whatever ``ulp_tol`` is): the count to report against a
                      1-ulp contract.
    """
    T = sel.shape[0]
    exact = 0
    bad = []
    max_ulp = 0.0
    swapped = 0
    over1 = 0
    for t in range(T):
        lo, hi = int(ks[t]), int(ke[t])
        n_valid = max(0, hi - lo)
        want = min(k, n_valid)
        row = sel[t]
        got = row[row >= 0]
        if got.size != want or np.unique(got).size != got.size or \
                (got.size and (got.min() < lo or got.max() >= hi)):
            bad.append(t)
            continue
        if (row[:want] < 0).any():      # padding must come after the valid part
            bad.append(t)
            continue
        if want == n_valid:
            exact += 1
            continue
        sc = scores[t, lo:hi].astype(np.float64)
        part = np.partition(sc, n_valid - want)
        thr = part[n_valid - want]                 # k-th largest
        chosen = np.zeros(n_valid, dtype=bool)
        chosen[got - lo] = True
        # wrongly chosen: score below thr; wrongly dropped: score above thr
        lowc = sc[chosen].min()
        highd = sc[~chosen].max()
        if lowc >= thr and highd <= thr:
            exact += 1
            continue
        ulp = float(np.spacing(np.float32(abs(thr)))) if thr != 0 else float(np.spacing(np.float32(1e-30)))
        d = max(thr - lowc, highd - thr, 0.0) / ulp
        max_ulp = max(max_ulp, d)
        swapped += 1
        over1 += d > 1.0
        if d > ulp_tol:
            bad.append(t)
    return {"exact_rows": exact, "bad_rows": bad, "max_ulp": max_ulp, "rows": T,
            "swapped_rows": swapped, "rows_over_1ulp": int(over1)}


# --------------------------------------------------------------------------
# RoPE                                          (sparse_attn/DSA.py:430-469)
# --------------------------------------------------------------------------
def rope_cossin(S: int, dim: int, base: float = 10000.0):
    half = dim // 2
    inv_freq = 1.0 / (base ** (torch.arange(0, half, dtype=torch.float32) / half))
    freqs = torch.outer(torch.arange(S, dtype=torch.float32), inv_freq)
    return freqs.cos(), freqs.sin()


def apply_rope_neox(x, cos, sin):
    half = x.shape[-1] // 2
    x1, x2 = x[..., :half], x[..., half:]
    while cos.dim() < x.dim():
        cos = cos.unsqueeze(1)
        sin = sin.unsqueeze(1)
    return torch.cat([x1 * cos - x2 * sin, x1 * sin + x2 * cos], dim=-1)


def apply_rope_interleave(x, cos, sin):
    xe, xo = x[..., 0::2], x[..., 1::2]
    while cos.dim() < xe.dim():
        cos = cos.unsqueeze(1)
        sin = sin.unsqueeze(1)
    out = torch.empty_like(x)
    out[..., 0::2] = xe * cos - xo * sin
    out[..., 1::2] = xe * sin + xo * cos
    return out


def _linear(x, weight):
    return torch.nn.functional.linear(x, weight)


def _rope_first(x, rd, cos, sin, interleave):
    fn = apply_rope_interleave if interleave else apply_rope_neox
    return torch.cat([fn(x[..., :rd], cos, sin), x[..., rd:]], dim=-1)


def dsa_indexer_inputs(params: dict, x, q_lora, n_heads, head_dim, rope_dim,
                       interleave=False, block_size=128, compress_ratio=1):
    """Everything of DsaIndexer.forward / Dsv4Indexer.forward before the scorer
    (DSA.py:530-543 and 621-650): projections, k_norm, RoPE, FP8 quant, ks/ke,
    folded weights.  ``params`` holds 'wq_b', 'wk', 'weights_proj', 'k_norm_w',
    'k_norm_b' (and 'pool_proj' when compress_ratio > 1) in the module dtype."""
    T = x.shape[0]
    q = _linear(q_lora, params["wq_b"]).view(T, n_heads, head_dim)
    if compress_ratio > 1:
        kin = _linear(x.view(T // compress_ratio, compress_ratio * x.shape[1]), params["pool_proj"])
    else:
        kin = _linear(x, params["wk"])
    k = torch.nn.functional.layer_norm(kin, (head_dim,), params["k_norm_w"], params["k_norm_b"])
    w = _linear(x, params["weights_proj"]).float() * (n_heads ** -0.5)
    T_kv = T // compress_ratio
    cos_q, sin_q = rope_cossin(T, rope_dim)
    cos_k, sin_k = rope_cossin(T_kv, rope_dim)
    q = _rope_first(q, rope_dim, cos_q, sin_q, interleave)
    k = _rope_first(k, rope_dim, cos_k, sin_k, interleave)
    q_fp8, q_scale = fp8_quant_per_block(q, block_size)
    k_fp8, k_scale = fp8_quant_per_block(k, block_size)
    ks = torch.zeros(T, dtype=torch.int32)
    ke = ((torch.arange(1, T + 1) + compress_ratio - 1) // compress_ratio).to(torch.int32)
    w_eff = fold_weights(w, q_scale, head_dim)
    if k_scale.dim() != 1:
        raise ValueError("oracle scorer takes one k scale per key (head_dim == block_size)")
    return q_fp8.contiguous(), k_fp8.contiguous(), k_scale.contiguous(), w_eff, ks, ke


def dsa_indexer_forward(params, x, q_lora, n_heads, head_dim, rope_dim, topk,
                        interleave=False, block_size=128, relu=True):
    """DsaIndexer.forward (DSA.py:527-568) -> int64 [T, min(topk, T)]."""
    a = dsa_indexer_inputs(params, x, q_lora, n_heads, head_dim, rope_dim, interleave, block_size)
    logits = indexer_logits(*a, relu=relu)
    return topk_indices(logits, min(topk, x.shape[0]))


def dsv4_indexer_forward(params, x, q_lora, n_heads, head_dim, rope_dim, topk,
                         compress_ratio=4, interleave=False, block_size=128, relu=True):
    """Dsv4Indexer.forward (DSA.py:619-676) -> int64 [T, min(topk//cr, T//cr)]."""
    a = dsa_indexer_inputs(params, x, q_lora, n_heads, head_dim, rope_dim, interleave,
                           block_size, compress_ratio)
    logits = indexer_logits(*a, relu=relu)
    K = min(topk // compress_ratio, x.shape[0] // compress_ratio)
    return logits.topk(K, dim=-1).indices


# --------------------------------------------------------------------------
# Sparse MLA (MQA over the shared latent KV) -- no reference code; restated math
# --------------------------------------------------------------------------
def sparse_mla(q: torch.Tensor, kv: torch.Tensor, idx: torch.Tensor, scale: float,
               d_v: int = 512, dtype=torch.float32, row_chunk: int = 64) -> torch.Tensor:
    """o[t,h,:] = sum_j softmax_j(scale * q[t,h,:] . kv[idx[t,j],:]) * kv[idx[t,j],:d_v].

    q [T,H,Dqk], kv [S,Dqk], idx [T,K] int (negative = empty slot).  A row with
    no valid slot yields zeros.  Streams over query rows like the reference's
    ``_dense_reference`` (bench_sparse_attention_kernels.py:431-441)."""
    T, H, D = q.shape
    out = torch.zeros(T, H, d_v, dtype=dtype)
    kvf = kv.to(dtype)
    for r0 in range(0, T, row_chunk):
        r1 = min(T, r0 + row_chunk)
        ii = idx[r0:r1].long()
        valid = ii >= 0
        g = kvf[ii.clamp_min(0)]                                   # [r,K,D]
        s = torch.einsum("thd,tkd->thk", q[r0:r1].to(dtype), g) * scale
        s = s.masked_fill(~valid.unsqueeze(1), float("-inf"))
        m = s.amax(dim=-1, keepdim=True)
        m = torch.where(torch.isinf(m), torch.zeros_like(m), m)
        p = torch.exp(s - m)
        l = p.sum(dim=-1, keepdim=True)
        p = torch.where(l > 0, p / l.clamp_min(1e-300), torch.zeros_like(p))
        out[r0:r1] = torch.einsum("thk,tkd->thd", p, g[..., :d_v])
    return out


# --------------------------------------------------------------------------
# Paged FP8 latent cache (layout fixed by the decode configuration, not by the
# reference, which has "no KV cache, paged layout" -- DSA.py:475-477)
# --------------------------------------------------------------------------
LATENT_DIM = 512
ROPE_DIM = 64
LATENT_GROUP = 128
TOKEN_BYTES = LATENT_DIM + 4 * (LATENT_DIM // LATENT_GROUP) + 2 * ROPE_DIM     # 656
PAGE_TOKENS = 64


def pack_latent_cache(kv: torch.Tensor) -> torch.Tensor:
    """kv [N, 576] (bf16/fp32) -> uint8 [N, 656]: 512 e4m3 | 4 fp32 scales | 64 bf16.

    Each 128-element group of the latent part gets scale = max(absmax,1e-6)/448
    (the indexer quantiser's rule, DSA.py:121-124)."""
    N = kv.shape[0]
    lat = kv[:, :LATENT_DIM].float().view(N, LATENT_DIM // LATENT_GROUP, LATENT_GROUP)
    scale = lat.abs().amax(-1, keepdim=True).clamp_min(1e-6) / FP8_MAX
    q8 = (lat / scale).to(FP8).view(N, LATENT_DIM)
    out = torch.empty(N, TOKEN_BYTES, dtype=torch.uint8)
    out[:, :LATENT_DIM] = q8.view(torch.uint8)
    out[:, LATENT_DIM:LATENT_DIM + 16] = scale.squeeze(-1).contiguous().view(torch.uint8).view(N, 16)
    out[:, LATENT_DIM + 16:] = kv[:, LATENT_DIM:].to(torch.bfloat16).contiguous().view(torch.uint8).view(N, 128)
    return out


def unpack_latent_cache(rec: torch.Tensor, round_bf16: bool = False) -> torch.Tensor:
    """uint8 [N,656] -> fp32 [N,576] (latent = e4m3 * group scale; rope bf16).
    ``round_bf16`` rounds the dequantised latent to bf16 first, which is what a
    kernel feeding bf16 tensor cores sees."""
    N = rec.shape[0]
    q8 = rec[:, :LATENT_DIM].contiguous().view(FP8).float().view(N, 4, LATENT_GROUP)
    scale = rec[:, LATENT_DIM:LATENT_DIM + 16].contiguous().view(torch.float32).view(N, 4, 1)
    lat = (q8 * scale).view(N, LATENT_DIM)
    if round_bf16:
        lat = lat.to(torch.bfloat16).float()
    rope = rec[:, LATENT_DIM + 16:].contiguous().view(torch.bfloat16).float().view(N, ROPE_DIM)
    return torch.cat([lat, rope], dim=-1)


def physical_rows(block_table_row: torch.Tensor, pos: torch.Tensor) -> torch.Tensor:
    """Logical token position -> physical row: table[pos // 64] * 64 + pos % 64."""
    p = pos.long()
    return block_table_row.long()[p // PAGE_TOKENS] * PAGE_TOKENS + p % PAGE_TOKENS


def sparse_mla_decode_paged(q, cache, block_table, idx, scale, round_bf16=False,
                            dtype=torch.float32) -> torch.Tensor:
    """Decode step over the paged FP8 cache.  q [B,H,576], cache uint8
    [num_pages*64, 656], block_table [B, pages_per_seq] int32, idx [B,K] logical
    positions (negative = empty).  Returns [B,H,512]."""
    B, H, D = q.shape
    out = torch.zeros(B, H, LATENT_DIM, dtype=dtype)
    for b in range(B):
        ii = idx[b].long()
        valid = ii >= 0
        rows = physical_rows(block_table[b], ii.clamp_min(0))
        kv = unpack_latent_cache(cache[rows], round_bf16)
        local = torch.where(valid, torch.arange(ii.numel()), torch.full_like(ii, -1))
        out[b] = sparse_mla(q[b:b + 1], kv, local.unsqueeze(0), scale, LATENT_DIM, dtype)[0]
    return out


def indexer_logits_paged(q_fp8, w, kcache, kscale, block_table, ctx_len, relu=True):
    """Decode indexer: one query token per sequence against its paged k cache.
    q_fp8 [B,H,128] e4m3, w [B,H] fp32 (q scale folded), kcache e4m3
    [num_pages*64,128], kscale fp32 [num_pages*64], block_table [B,P],
    ctx_len [B].  Returns fp32 [B, P*64] with -inf at positions >= ctx_len[b]."""
    B, H, D = q_fp8.shape
    P = block_table.shape[1]
    out = torch.full((B, P * PAGE_TOKENS), float("-inf"), dtype=torch.float32)
    for b in range(B):
        n = int(ctx_len[b])
        rows = physical_rows(block_table[b], torch.arange(n))
        zero = torch.zeros(1, dtype=torch.int32)
        lg = indexer_logits(q_fp8[b:b + 1], kcache[rows], kscale[rows], w[b:b + 1],
                            zero, torch.tensor([n], dtype=torch.int32), relu=relu)
        out[b, :n] = lg[0]
    return out


# --------------------------------------------------------------------------
# Whole layer for the small CPU configuration (seq 2048, 4 indexer heads of 64,
# top-k 256, 16 MLA heads): indexer -> top-k -> sparse MLA
# --------------------------------------------------------------------------
def dsa_layer_forward(params, x, q_lora, q_mla, kv, n_heads, head_dim, rope_dim, topk,
                      scale, block_size, relu=True):
    idx = dsa_indexer_forward(params, x, q_lora, n_heads, head_dim, rope_dim, topk,
                              block_size=block_size, relu=relu)
    T = x.shape[0]
    ke = torch.arange(1, T + 1).unsqueeze(1)
    # rows shorter than top-k: the reference pads with masked positions (DSA.py:361
    # on -inf entries); the sparse step must ignore them.
    idx32 = torch.where(idx < ke, idx, torch.full_like(idx, -1)).to(torch.int32)
    return idx32, sparse_mla(q_mla, kv, idx32, scale)


def block_sparse_mha(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, lut: torch.Tensor, num: torch.Tensor,
                     sm_scale: float, block: int = 64) -> torch.Tensor:
    """Block-sparse multi-head attention, the arithmetic behind register_sparse_fa().run
    (sparse_attn/DSA.py:232-247; the Triton kernel it calls is not part of the reference, so this restates
    the published semantics of that call: non-causal softmax attention of every 64-row query block over the
    key blocks its list names).  q, k, v [B, S, H, D]; lut [B, H, S/block, topk]; num [B, H, S/block].
    fp32 arithmetic; returns fp32 [B, S, H, D].  Parity unpinned: the reference holds no vectors for it."""
    B, S, H, D = q.shape
    nqb = S // block
    qf, kf, vf = q.float(), k.float(), v.float()
    out = torch.zeros(B, S, H, D, dtype=torch.float32)
    for b in range(B):
        for h in range(H):
            for qb in range(nqb):
                n = int(num[b, h, qb])
                ids = [int(i) for i in lut[b, h, qb, :n].tolist() if 0 <= int(i) < nqb]
                if not ids:
                    continue
                cols = torch.cat([torch.arange(i * block, (i + 1) * block) for i in ids])
                qs = qf[b, qb * block:(qb + 1) * block, h]                  # [block, D]
                sc = (qs @ kf[b, cols, h].T) * sm_scale                      # [block, n*block]
                p = torch.softmax(sc, dim=-1)
                out[b, qb * block:(qb + 1) * block, h] = p @ vf[b, cols, h]
    return out
