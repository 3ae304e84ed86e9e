"""Composition of the DSA kernels: indexer -> top-k -> sparse MLA, for prefill and for one
decode step over paged caches.  The reference has no counterpart for the attention half
(its sparse step is a block-sparse stand-in, sparse_attn/DSA.py:208-249) nor for decode
(no cache, sparse_attn/DSA.py:475-477); the call shapes follow the DSA formula of
sparse_attn/ATTENTION_MATH.md:56-64."""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn

from . import _lib, ops


class SparseMLA(nn.Module):
    """MQA over the shared latent KV restricted to the selected positions.

    forward(q [T,H,576] bf16, kv, topk_idx [T,K] int (negative = empty), block_table=None)
      kv = [S,576] bf16 (prefill) or the paged FP8 latent cache uint8 [num_pages*64, 656]
      together with block_table [T, P] (decode, one query token per sequence).
    Returns bf16 [T,H,512]."""

    def __init__(self, softmax_scale: float):
        super().__init__()
        self.softmax_scale = float(softmax_scale)

    @torch.no_grad()
    def forward(self, q, kv, topk_idx, block_table: Optional[torch.Tensor] = None):
        idx = topk_idx if topk_idx.dtype == torch.int32 else topk_idx.to(torch.int32)
        if kv.dtype == torch.uint8:
            if block_table is None:
                raise ops.DsaError("the paged FP8 latent cache needs a block_table")
            return ops.sparse_mla_decode_paged(q, kv, block_table, idx, self.softmax_scale)
        return ops.sparse_mla_prefill(q, kv, idx, self.softmax_scale)


@torch.no_grad()
def dsa_prefill(q_idx_fp8, k_idx_fp8, k_scale, w, ks, ke, topk: int, q, kv, softmax_scale: float):
    """Prefill: indexer logits + top-k (one library call), then sparse MLA over the selection.
    Returns (idx int32 [T,k], out bf16 [T,H,512])."""
    idx = ops.indexer_topk(q_idx_fp8, k_idx_fp8, k_scale, w, ks, ke, topk)
    return idx, ops.sparse_mla_prefill(q, kv, idx, softmax_scale)


class DecodeWorkspace:
    """Buffers of one decode step, allocated once and reused every step."""

    def __init__(self, batch: int, heads: int, max_ctx: int, topk: int, device):
        ld = (max_ctx + 3) // 4 * 4
        self.logits = torch.empty(batch, ld, dtype=torch.float32, device=device)
        self.k = min(topk, max_ctx)                    # selected keys per sequence (the kernels write rows at this stride)
        self.idx = torch.empty(batch, self.k, dtype=torch.int32, device=device)
        self.out = torch.empty(batch, heads, 512, dtype=torch.bfloat16, device=device)
        need = _lib.load().dsa_sparse_mla_decode_workspace_bytes(batch, heads, min(topk, max_ctx))
        self.mla_ws = torch.empty(max(need, 16), dtype=torch.uint8, device=device)
        self.max_ctx, self.topk = max_ctx, topk


@torch.no_grad()
def dsa_decode_step(q_idx_fp8, w, kcache, kscale, block_table, ctx_len, q, latent_cache, softmax_scale: float,
                    ws: DecodeWorkspace):
    """One decode step for a batch of sequences: paged indexer scan, top-k over each sequence's
    context, sparse MLA over the paged FP8 latent cache.  Returns (idx, out) views of ``ws``."""
    B = q.shape[0]
    logits = ops.fp8_paged_mqa_logits(q_idx_fp8, w, kcache, kscale, block_table, ctx_len, ws.max_ctx, out=ws.logits)
    ops.topk_select(logits, ws.k, None, ctx_len, out=ws.idx[:B])
    ops.sparse_mla_decode_paged(q, latent_cache, block_table, ws.idx[:B], softmax_scale, ws.max_ctx, out=ws.out[:B],
                                workspace=ws.mla_ws)
    return ws.idx[:B], ws.out[:B]
