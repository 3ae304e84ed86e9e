"""Drop-in for the reference's ``sparse_attn/DSA.py`` module surface, on the sm_100a kernels.

The reference's benchmark drivers do ``from DSA import ...`` (bench_sparse_attention_kernels.py:71-83,
bench_sparse_attention_modules.py:73-85).  This module exports the same names with the same call
signatures and return conventions; the scorer and the top-k run through libdsa_b200 (no deep_gemm,
no Triton, no CPU fallback -- tensors must live on a CUDA device).  Projections, LayerNorm and RoPE
stay torch ops: they are linear in sequence length and outside the hot path
(sparse_attn/DSA.py:267-270).

Differences from the reference, on purpose:
  * the scorer applies the ReLU of the DSA formula (sparse_attn/ATTENTION_MATH.md:56-60); the
    reference's fp32 fallback omits it (sparse_attn/DSA.py:356-357);
  * a row whose causal window holds fewer than top-k keys gets ``-1`` in the unused slots where the
    reference returns arbitrary masked positions (sparse_attn/DSA.py:361 on -inf entries);
  * returned indices are int64 like ``torch.topk``'s but in no particular order.
"""
from __future__ import annotations

import types
from dataclasses import dataclass
from typing import Callable, Dict, Optional, Tuple

import torch
import torch.nn as nn

from . import ops

INDEXER_N_HEADS = 64
INDEXER_HEAD_DIM = 128
INDEXER_TOPK = 2048
INDEXER_BLOCK_SIZE = 128
SPARSE_BLOCK = 64

_FP8 = torch.float8_e4m3fn
_FP8_MAX = 448.0


def env_report() -> Dict[str, str]:
    """What this environment runs on (reference: sparse_attn/DSA.py:53-84)."""
    from . import _lib
    rep = {"torch": f"{torch.__version__} (cuda={torch.version.cuda})",
           "cuda_available": str(torch.cuda.is_available())}
    if torch.cuda.is_available():
        rep["device"] = torch.cuda.get_device_name(0)
    try:
        rep["libdsa_b200"] = f"version {_lib.load().dsa_version()} ({_lib.LIB_PATH})"
    except RuntimeError as e:
        rep["libdsa_b200"] = f"MISSING: {e}"
    rep["deep_gemm"] = "replaced by libdsa_b200 (dsa_indexer_logits)"
    rep["flash_attn.cute"] = "not used (dense baseline is outside this package)"
    return rep


def try_import_deep_gemm():
    """The plugin seam of sparse_attn/DSA.py:87-95: an object with ``fp8_mqa_logits``."""
    shim = types.ModuleType("deep_gemm")
    shim.fp8_mqa_logits = ops.fp8_mqa_logits
    return shim


def fp8_quant_per_block(x: torch.Tensor, block_size: int = INDEXER_BLOCK_SIZE) -> Tuple[torch.Tensor, torch.Tensor]:
    """bf16/fp32 -> e4m3 with one fp32 scale per ``block_size`` values of the last dim
    (sparse_attn/DSA.py:102-132): scale = max(absmax, 1e-6) / 448; the scale tensor drops its last
    dim when a row is a single block.  One fused kernel; its bytes and scales equal the
    reference's CPU result (both divisions are IEEE round-to-nearest)."""
    return ops.fp8_quant_per_block(x, block_size)


def _fold(w: torch.Tensor, q_scale: torch.Tensor, head_dim: int) -> torch.Tensor:
    """Head gates with the q scale and head_dim**-0.5 folded in (sparse_attn/DSA.py:327-331)."""
    qs = q_scale if q_scale.dim() == 2 else q_scale.mean(dim=-1)
    return (w.float() * qs.float() * head_dim ** -0.5).contiguous()


def _score_topk(q_fp8, k_fp8, k_scale, w_eff, ks, ke, k: int) -> torch.Tensor:
    ksc = k_scale if k_scale.dim() == 1 else k_scale.squeeze(-1)
    return ops.indexer_topk(q_fp8.contiguous(), k_fp8.contiguous(), ksc.contiguous(), w_eff, ks, ke, k).long()


# ---- dense / block-sparse registration hooks (reference: sparse_attn/DSA.py:139-249) -------------
def register_fa4() -> Optional[Callable]:
    """Dense FA4 baseline: not part of this package."""
    return None


def register_sgl_fa4() -> Optional[Callable]:
    return None


def register_dense_fn() -> Optional[Callable]:
    return register_fa4() or register_sgl_fa4()


def register_sparse_fa() -> Optional[Tuple[Callable, Callable]]:
    """(build_lut, run) like the reference (sparse_attn/DSA.py:208-249), with `run` on this package's
    block-sparse MHA kernel ([B,S,H,128] bf16, 64-token blocks, non-causal) instead of the external Triton
    kernel the reference imports.  build_lut draws a random per-query-block list the same way (:232-241)."""
    if not torch.cuda.is_available():
        return None

    def build_lut(q: torch.Tensor, S: int, sparsity: float) -> Tuple[torch.Tensor, torch.Tensor, int]:
        B, _, H, _ = q.shape
        Nq = Nkv = S // SPARSE_BLOCK
        topk = max(1, int(round(sparsity * Nkv)))
        scores = torch.rand(B, H, Nq, Nkv, device=q.device)
        idx = scores.topk(topk, dim=-1).indices.to(torch.int32).contiguous()
        q2k_num = torch.full((B, H, Nq), topk, dtype=torch.int32, device=q.device)
        return idx, q2k_num, topk

    def run(q, k, v, idx, num, sm_scale):
        return ops.block_sparse_attn(q, k, v, idx, num, sm_scale)

    return build_lut, run


# ---- kernel-level simulator (reference: sparse_attn/DSA.py:256-362) ---------------------------------
class IndexerSimulator:
    """Synthetic-tensor driver of the indexer hot path with the reference's method surface."""

    def __init__(self, S: int, n_heads: int = INDEXER_N_HEADS, head_dim: int = INDEXER_HEAD_DIM,
                 topk: int = INDEXER_TOPK, device: torch.device = torch.device("cuda"),
                 hidden_size: int = 7168, q_lora_rank: int = 1536):
        self.S, self.n_heads, self.head_dim, self.topk, self.device = S, n_heads, head_dim, topk, device
        self.dg = try_import_deep_gemm()
        bf = dict(dtype=torch.bfloat16, device=device)
        self.q_lora_a = torch.randn(S, q_lora_rank, **bf)
        self.x = torch.randn(S, hidden_size, **bf)
        self.positions = torch.arange(S, device=device, dtype=torch.int32)
        self.wq_b = nn.Linear(q_lora_rank, n_heads * head_dim, bias=False, **bf)
        self.wk = nn.Linear(hidden_size, head_dim, bias=False, **bf)
        self.weights_proj = nn.Linear(hidden_size, n_heads, bias=False, **bf)
        self.ks = torch.zeros(S, dtype=torch.int32, device=device)
        self.ke = (self.positions + 1).to(torch.int32)
        self._fp8_cache = None

    @torch.no_grad()
    def projections_step(self):
        q = self.wq_b(self.q_lora_a).view(self.S, self.n_heads, self.head_dim)
        return q, self.wk(self.x), self.weights_proj(self.x).float() * self.n_heads ** -0.5

    def quantize_step(self, q_bf16, k_bf16):
        q_fp8, q_scale = fp8_quant_per_block(q_bf16, min(INDEXER_BLOCK_SIZE, self.head_dim))
        k_fp8, k_scale = fp8_quant_per_block(k_bf16, min(INDEXER_BLOCK_SIZE, self.head_dim))
        return q_fp8, q_scale, k_fp8, k_scale

    def precompute_fp8(self) -> None:
        q, k, w = self.projections_step()
        q_fp8, q_scale, k_fp8, k_scale = self.quantize_step(q, k)
        self._fp8_cache = (q_fp8.contiguous(), k_fp8.contiguous(), k_scale.contiguous(),
                           _fold(w, q_scale, self.head_dim))

    def logits_step(self) -> torch.Tensor:
        """Score + top-k: one library call.  int64 [S, min(topk, S)]."""
        assert self._fp8_cache is not None
        q_fp8, k_fp8, k_scale, w = self._fp8_cache
        return _score_topk(q_fp8, k_fp8, k_scale, w, self.ks, self.ke, min(self.topk, self.S))


# ---- nn.Module indexers (reference: sparse_attn/DSA.py:369-676) -------------------------------------
@dataclass
class IndexerSpec:
    name: str
    hidden_size: int
    q_lora_rank: int
    index_n_heads: int
    index_head_dim: int
    rope_head_dim: int
    index_topk: int
    compress_ratio: int = 1
    rope_interleave: bool = False


SPECS: Dict[str, IndexerSpec] = {
    "dsv32": IndexerSpec("DSv3.2", 7168, 1536, 64, 128, 64, 2048, 1, False),
    "glm": IndexerSpec("GLM-5 / 5.2", 6144, 2048, 64, 128, 64, 2048, 1, True),
    "dsv4": IndexerSpec("DSv4", 7168, 1536, 64, 128, 64, 2048, 4, False),
}

_ROPE_TABLES: Dict[Tuple[int, int, torch.device], Tuple[torch.Tensor, torch.Tensor]] = {}


def _rope_cossin(S: int, dim: int, device, base: float = 10000.0):
    key = (S, dim, torch.device(device))
    if key not in _ROPE_TABLES:
        half = dim // 2
        inv = 1.0 / (base ** (torch.arange(0, half, device=device, dtype=torch.float32) / half))
        ang = torch.outer(torch.arange(S, device=device, dtype=torch.float32), inv)
        _ROPE_TABLES[key] = (ang.cos(), ang.sin())
    return _ROPE_TABLES[key]


def _rotate(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, interleave: bool) -> torch.Tensor:
    """RoPE on the whole last dim of x: NeoX halves or GPT-J even/odd pairs (DSA.py:444-469).
    Like the reference, the NeoX form returns the fp32 products unrounded (bf16 x times the fp32 table
    promotes, so q and k reach the quantiser as fp32 with the un-rotated dims holding bf16 values);
    the interleaved form rounds back to x's dtype (the reference writes into ``empty_like(x)``)."""
    if x.dim() == 3:
        cos, sin = cos.unsqueeze(1), sin.unsqueeze(1)
    if interleave:
        a, b = x[..., 0::2], x[..., 1::2]
        return torch.stack((a * cos - b * sin, a * sin + b * cos), dim=-1).flatten(-2).to(x.dtype)
    h = x.shape[-1] // 2
    a, b = x[..., :h], x[..., h:]
    return torch.cat((a * cos - b * sin, a * sin + b * cos), dim=-1)      # fp32 for bf16 x: no rounding here


def _rope_head(x: torch.Tensor, rd: int, S: int, interleave: bool) -> torch.Tensor:
    cos, sin = _rope_cossin(S, rd, x.device)
    return torch.cat((_rotate(x[..., :rd], cos, sin, interleave), x[..., rd:]), dim=-1)


class DsaIndexer(nn.Module):
    """DSv3.2 / GLM-5 indexer: x [T,hidden], q_lora_a [T,q_lora] -> top-k key positions [T, min(topk,T)]."""

    def __init__(self, spec: IndexerSpec, dtype: torch.dtype = torch.bfloat16):
        super().__init__()
        self.spec, self.dtype = spec, dtype
        self.wq_b = nn.Linear(spec.q_lora_rank, spec.index_n_heads * spec.index_head_dim, bias=False, dtype=dtype)
        self.wk = nn.Linear(spec.hidden_size, spec.index_head_dim, bias=False, dtype=dtype)
        self.weights_proj = nn.Linear(spec.hidden_size, spec.index_n_heads, bias=False, dtype=dtype)
        self.k_norm = nn.LayerNorm(spec.index_head_dim, dtype=dtype)
        self.softmax_scale = spec.index_head_dim ** -0.5
        self._dg = try_import_deep_gemm()

    def _quant_block(self) -> int:
        return min(INDEXER_BLOCK_SIZE, self.spec.index_head_dim)

    @torch.no_grad()
    def projections(self, x, q_lora_a):
        T = x.shape[0]
        q = self.wq_b(q_lora_a).view(T, self.spec.index_n_heads, self.spec.index_head_dim)
        return q, self.k_norm(self.wk(x)), self.weights_proj(x).float() * self.spec.index_n_heads ** -0.5

    @torch.no_grad()
    def rope(self, q, k):
        rd, il = self.spec.rope_head_dim, self.spec.rope_interleave
        return _rope_head(q, rd, q.shape[0], il), _rope_head(k, rd, k.shape[0], il)

    def _rope_quant(self, x: torch.Tensor, n_pos: int, rows_per_pos: int):
        """RoPE on the first rope_head_dim values of every head row, then the per-row FP8 quantiser: one fused kernel
        for bf16 rows of one FP8 block (its bytes and scales equal the eager chain's), the eager chain otherwise."""
        rd, il = self.spec.rope_head_dim, self.spec.rope_interleave
        if x.dtype == torch.bfloat16 and x.shape[-1] == self._quant_block() and x.shape[-1] in (64, 128):
            cos, sin = _rope_cossin(n_pos, rd, x.device)
            return ops.rope_fp8_quant(x, cos, sin, rd, il, rows_per_pos)
        return fp8_quant_per_block(_rope_head(x, rd, n_pos, il), self._quant_block())

    def _select(self, q, k, w, ke, topk: int) -> torch.Tensor:
        """q [T,H,D], k [T_kv,D] straight from the projections (before RoPE), head gates w, windows ke."""
        q_fp8, q_scale = self._rope_quant(q, q.shape[0], q.shape[1])
        k_fp8, k_scale = self._rope_quant(k, k.shape[0], 1)
        ks = torch.zeros_like(ke)
        return _score_topk(q_fp8, k_fp8, k_scale, _fold(w, q_scale, self.spec.index_head_dim), ks, ke, topk)

    @torch.no_grad()
    def forward(self, x, q_lora_a):
        q, k, w = self.projections(x, q_lora_a)
        T = x.shape[0]
        ke = torch.arange(1, T + 1, dtype=torch.int32, device=x.device)
        return self._select(q, k, w, ke, min(self.spec.index_topk, T))


class C4Compressor(nn.Module):
    """Pools every ``compress_ratio`` tokens into one key token by a linear map (DSA.py:571-595)."""

    def __init__(self, hidden_size: int, head_dim: int, compress_ratio: int, dtype: torch.dtype = torch.bfloat16):
        super().__init__()
        self.compress_ratio, self.head_dim = compress_ratio, head_dim
        self.pool_proj = nn.Linear(hidden_size * compress_ratio, head_dim, bias=False, dtype=dtype)

    @torch.no_grad()
    def forward(self, x):
        T, Hd = x.shape
        assert T % self.compress_ratio == 0
        return self.pool_proj(x.view(T // self.compress_ratio, self.compress_ratio * Hd))


class Dsv4Indexer(DsaIndexer):
    """DSA-C4: keys are the 4x-compressed stream; indices are in compressed-token space (DSA.py:598-676)."""

    def __init__(self, spec: IndexerSpec, dtype: torch.dtype = torch.bfloat16):
        super().__init__(spec, dtype=dtype)
        assert spec.compress_ratio > 1, "Dsv4Indexer requires compress_ratio > 1"
        self.compressor = C4Compressor(spec.hidden_size, spec.index_head_dim, spec.compress_ratio, dtype)

    @torch.no_grad()
    def forward(self, x, q_lora_a):
        T, cr = x.shape[0], self.spec.compress_ratio
        T_kv = T // cr
        q = self.wq_b(q_lora_a).view(T, self.spec.index_n_heads, self.spec.index_head_dim)
        k = self.k_norm(self.compressor(x))
        w = self.weights_proj(x).float() * self.spec.index_n_heads ** -0.5
        ke = ((torch.arange(1, T + 1, device=x.device) + cr - 1) // cr).to(torch.int32)
        return self._select(q, k, w, ke, min(self.spec.index_topk // cr, T_kv))
