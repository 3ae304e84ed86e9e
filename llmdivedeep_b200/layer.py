"""Composition of the DSA kernels: indexer -> top-k -> sparse MLA, for prefill and for one
decode step over paged caches.  The reference has no counterpart for the attention half
(its sparse step is a block-sparse stand-in, sparse_attn/DSA.py:208-249) nor for decode
(no cache, sparse_attn/DSA.py:475-477); the call shapes follow the DSA formula of
sparse_attn/ATTENTION_MATH.md:56-64."""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn

from . import _lib, ops, sharding


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


class DSALayer(nn.Module):
    """One DSA attention layer from hidden states: lightning indexer -> top-k -> sparse MLA.

    forward(x [T, hidden]) -> bf16 [T, n_heads, 512].  The indexer half is the reference's DsaIndexer
    (sparse_attn/DSA.py:472-568) on this package's kernels; the attention half -- which the reference
    only stands in for with a block-sparse MHA call (sparse_attn/DSA.py:208-249) -- is MQA over one
    shared latent KV row per token (576 = 512 latent + 64 rope dims, V = the 512 latent dims),
    restricted to the selected positions.  Projections are bias-free Linears like the reference's:
        q_lora = q_a(x);  indices = indexer(x, q_lora);  q = wq(q_lora) -> [T, n_heads, 576];
        kv = wkv(x) -> [T, 576];  out = SparseMLA(q, kv, indices).
    Defaults are the small configuration the CPU reference run uses: hidden 1024, 4 indexer heads of
    dim 64 (FP8 block 64), top-k 256, 16 query heads; weights ~ N(0, init_std^2), LayerNorm at 1 / 0."""

    def __init__(self, hidden_size: int = 1024, q_lora_rank: int = 256, index_n_heads: int = 4,
                 index_head_dim: int = 64, rope_head_dim: int = 64, index_topk: int = 256, n_heads: int = 16,
                 softmax_scale: float = 192 ** -0.5, rope_interleave: bool = False, init_std: float = 0.02,
                 dtype: torch.dtype = torch.bfloat16, seed: Optional[int] = None):
        super().__init__()
        from . import DSA
        self.n_heads, self.dtype = n_heads, dtype
        self.spec = DSA.IndexerSpec("dsa-layer", hidden_size, q_lora_rank, index_n_heads, index_head_dim,
                                    rope_head_dim, index_topk, 1, rope_interleave)
        self.q_a = nn.Linear(hidden_size, q_lora_rank, bias=False, dtype=dtype)
        self.indexer = DSA.DsaIndexer(self.spec, dtype=dtype)
        self.wq = nn.Linear(q_lora_rank, n_heads * 576, bias=False, dtype=dtype)
        self.wkv = nn.Linear(hidden_size, 576, bias=False, dtype=dtype)
        self.attn = SparseMLA(softmax_scale)
        g = torch.Generator().manual_seed(seed) if seed is not None else None
        with torch.no_grad():
            for lin in (self.q_a, self.wq, self.wkv, self.indexer.wq_b, self.indexer.wk, self.indexer.weights_proj):
                lin.weight.copy_((torch.randn(lin.weight.shape, generator=g) * init_std).to(dtype))

    @torch.no_grad()
    def stages(self, x: torch.Tensor) -> dict:
        """forward() with every intermediate kept: q_lora, the indexer's selection (int32, -1 = unused
        slot), the attention operands and the output."""
        x = x.to(self.dtype)
        T = x.shape[0]
        q_lora = self.q_a(x)
        idx = self.indexer(x, q_lora).to(torch.int32)
        q = self.wq(q_lora).view(T, self.n_heads, 576)
        kv = self.wkv(x)
        out = self.attn(q, kv, idx)
        return {"x": x, "q_lora": q_lora, "idx": idx, "q": q, "kv": kv, "out": out}

    @torch.no_grad()
    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.stages(x)["out"]


@torch.no_grad()
def dsa_prefill(q_idx_fp8, k_idx_fp8, k_scale, w, ks, ke, topk: int, q, kv, softmax_scale: float):
    """Prefill: indexer logits + top-k (one library call), then sparse MLA over the selection.
    Returns (idx int32 [T,k], out bf16 [T,H,512])."""
    idx = ops.indexer_topk(q_idx_fp8, k_idx_fp8, k_scale, w, ks, ke, topk)
    return idx, ops.sparse_mla_prefill(q, kv, idx, softmax_scale)


class IndexShare:
    """Index reuse across consecutive layers (GLM-5.2's IndexShare; the ``index_topk_freq`` by which the reference's
    module driver divides the indexer time, bench_sparse_attention_modules.py:193): the indexer runs on every
    ``freq``-th layer, and the layers in between attend over the indices of the last layer that ran it.

        share = IndexShare(freq=4)
        for i, layer in enumerate(layers):
            idx = share.select(i, layer.indexer, x, q_lora)      # runs the indexer when i % 4 == 0
            out = layer.attn(q, kv, idx)
    """

    def __init__(self, freq: int = 1):
        if freq < 1:
            raise ValueError("freq must be >= 1")
        self.freq, self.idx, self.runs = int(freq), None, 0

    def select(self, layer_idx: int, indexer, *inputs):
        if self.idx is None or layer_idx % self.freq == 0:
            self.idx = indexer(*inputs)
            self.runs += 1
        return self.idx

    def reset(self):
        self.idx = None


class PrefillPipeline:
    """Chunked DSA prefill of one sequence (batch 1, causal, S queries over S keys).

    Per chunk of query rows: indexer logits + top-k (one library call over a reused logits workspace),
    then sparse MLA over the selection.  With world > 1 the query rows are dealt to the ranks in
    `block_rows`-row blocks round-robin (sharding.round_robin_blocks): a rank runs only its own blocks --
    keys and latent KV are replicated, nothing is exchanged before the output -- and the attention output
    of every finished chunk is all-gathered on a side stream, one collective per round of `world` blocks
    straight into its place in the full output, while the next chunk computes.  With transport="peer" there
    is no collective kernel at all: the output lives in symmetric memory (output_buffer()), and a finished
    block is written into every rank's copy by plain device-to-device copies on the side stream -- the copy
    engines move it over NVLink and the SMs stay with the attention kernel, whose CTAs fill every SM's
    shared memory so that a collective's CTAs can only run in the gaps between its waves.  Two 4-byte
    all-reduces per run() order the ranks: one before the first copy (every rank is done with the previous
    output), one after the last (every rank's copies have landed).

    Tensors given to run() hold the rank's rows in local order (for world == 1 that is the sequence
    itself): q_idx [T_loc, Hi, Di] e4m3, w [T_loc, Hi], q [T_loc, H, 576] bf16; replicated k_idx [S, Di]
    e4m3, k_scale [S], kv [S, 576] bf16; out_full [S, H, 512] bf16 is complete on every rank afterwards.
    `select` / `attend` default to the library kernels; tests pass CPU stand-ins."""

    def __init__(self, S: int, device, n_heads: int = 128, topk: int = 2048, chunk_rows: int = 4096,
                 softmax_scale: float = 192 ** -0.5, rank: int = 0, world: int = 1, block_rows: int = 256,
                 group=None, select=None, attend=None, transport: str = "nccl"):
        if transport not in ("nccl", "peer"):
            raise ValueError("transport must be 'nccl' or 'peer'")
        if chunk_rows % block_rows:
            raise ValueError("chunk_rows must be a whole number of row blocks")
        self.S, self.device, self.H, self.k = S, torch.device(device), n_heads, min(topk, S)
        self.scale, self.rank, self.world, self.block, self.group = float(softmax_scale), rank, world, block_rows, group
        self.blocks = sharding.round_robin_blocks(S, world, rank, block_rows)      # global [start, end) of local blocks
        self.T_loc = sum(b - a for a, b in self.blocks)
        self.pos = sharding.rows_of(self.blocks, device=self.device).to(torch.int32)   # global position of each local row
        self.ks = torch.zeros(self.T_loc, dtype=torch.int32, device=self.device)
        self.ke = self.pos + 1
        per = chunk_rows // block_rows
        self.chunks = []                               # (first local row, last local row, first local block, last local block)
        row = 0
        for b0 in range(0, len(self.blocks), per):
            b1 = min(len(self.blocks), b0 + per)
            n = sum(e - a for a, e in self.blocks[b0:b1])
            self.chunks.append((row, row + n, b0, b1))
            row += n
        self.rows_max = max((c[1] - c[0] for c in self.chunks), default=0)
        self.idx = torch.empty(self.T_loc, self.k, dtype=torch.int32, device=self.device)
        self.cuda = self.device.type == "cuda"
        self.select, self.attend = select or self._select, attend or self._attend
        self.ws = None
        if select is None and self.rows_max:
            nbytes = _lib.load().dsa_indexer_topk_workspace_bytes(self.rows_max, S)
            self.ws = torch.empty(nbytes, dtype=torch.uint8, device=self.device)
        self.transport = transport if (world > 1 and self.cuda) else "nccl"
        self._peers = None                             # transport "peer": every rank's output, as seen from this GPU
        self._symm = None
        self.local = None
        if world > 1:
            self.local = [torch.empty(self.rows_max, n_heads, 512, dtype=torch.bfloat16, device=self.device)
                          for _ in range(2)]
            self._gathered = [None, None]              # per local buffer: event after the collectives that read it
            # high priority: the collective's CTAs are scheduled ahead of the attention kernel's waiting CTAs whenever an SM
            # frees up (the attention kernel fills every SM's shared memory, so a collective cannot squeeze in beside it)
            self.comm = torch.cuda.Stream(device=self.device, priority=-1) if self.cuda else None
        self.launches_per_run = 3 * len(self.chunks)   # indexer, top-k, sparse MLA per chunk

    def _select(self, q_idx, k_idx, k_scale, w, ks, ke, k, out):
        return ops.indexer_topk(q_idx, k_idx, k_scale, w, ks, ke, k, workspace=self.ws, out=out)

    def _attend(self, q, kv, idx, scale, out):
        return ops.sparse_mla_prefill(q, kv, idx, scale, out=out)

    def output_buffer(self) -> torch.Tensor:
        """The [S, H, 512] bf16 tensor to pass to run() as out_full.  Plain device memory, or -- transport "peer" --
        symmetric memory mapped into every rank of the group (a collective call: every rank makes it, once)."""
        shape = (self.S, self.H, 512)
        if self.transport != "peer":
            return torch.empty(shape, dtype=torch.bfloat16, device=self.device)
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm
        out = symm.empty(*shape, dtype=torch.bfloat16, device=self.device)
        handle = symm.rendezvous(out, self.group if self.group is not None else dist.group.WORLD)
        self._peers = [handle.get_buffer(r, shape, torch.bfloat16) for r in range(self.world)]
        self._symm = (out, handle)
        self._token = torch.zeros(1, dtype=torch.int32, device=self.device)
        return out

    def _order_ranks(self):
        """A 4-byte all-reduce on the current stream: passes once every rank's stream has reached this point."""
        import torch.distributed as dist
        dist.all_reduce(self._token, group=self.group)

    def begin(self, out_full):
        """Start of one prefill: with transport "peer" no rank may write into another's output before that rank is done
        with the previous one (everything it enqueued on its stream before this call)."""
        if self.transport == "peer":
            if self._symm is None or out_full.data_ptr() != self._symm[0].data_ptr():
                raise ValueError('transport "peer" writes into the tensor output_buffer() returned')
            self._order_ranks()

    def _gather_chunk(self, out_full, local, b0, b1):
        off = 0
        for j in range(b0, b1):
            a, e = self.blocks[j]
            if self.transport == "peer":
                for peer in self._peers:               # own copy included; contiguous rows: one memcpy each
                    peer[a:e].copy_(local[off:off + (e - a)], non_blocking=True)
            else:
                sharding.all_gather_round(out_full, local[off:off + (e - a)], j, self.S, self.world, self.block, self.group)
            off += e - a

    @torch.no_grad()
    def run_chunk(self, c: int, q_idx, k_idx, k_scale, w, q, kv, out_full, out_chunk=None):
        """Chunk c of run(): rows [a, b) of the local tensors (pass slices starting at a row 0 = a through
        `q_idx`, `w`, `q` already cut to the chunk).  Returns the tensor holding the chunk's output."""
        a, b, b0, b1 = self.chunks[c]
        idx = self.idx[a:b]
        self.select(q_idx, k_idx, k_scale, w, self.ks[a:b], self.ke[a:b], self.k, idx)
        if self.world == 1:
            dst = out_full[a:b] if out_chunk is None else out_chunk
            self.attend(q, kv, idx, self.scale, dst)
            return dst
        slot = c & 1
        main = torch.cuda.current_stream(self.device) if self.cuda else None
        if self.cuda and self._gathered[slot] is not None:
            main.wait_event(self._gathered[slot])      # the collectives that read this buffer two chunks ago
        dst = self.local[slot][: b - a]
        self.attend(q, kv, idx, self.scale, dst)
        if not self.cuda:
            self._gather_chunk(out_full, dst, b0, b1)
            return dst
        computed = torch.cuda.Event()
        computed.record(main)
        with torch.cuda.stream(self.comm):
            self.comm.wait_event(computed)
            self._gather_chunk(out_full, dst, b0, b1)
            ev = torch.cuda.Event()
            ev.record(self.comm)
            self._gathered[slot] = ev
        return dst

    @torch.no_grad()
    def run(self, q_idx, k_idx, k_scale, w, q, kv, out_full):
        self.begin(out_full)
        for c, (a, b, _, _) in enumerate(self.chunks):
            self.run_chunk(c, q_idx[a:b], k_idx, k_scale, w[a:b], q[a:b], kv, out_full)
        self.finish()
        return out_full

    def finish(self):
        """The current stream waits for the output collectives (copies: of every rank) issued so far."""
        if self.world > 1 and self.cuda:
            if self.transport == "peer":
                with torch.cuda.stream(self.comm):
                    self._order_ranks()                # behind this rank's copies; passes when every rank's have landed
            torch.cuda.current_stream(self.device).wait_stream(self.comm)


class HostPrefillPipeline:
    """PrefillPipeline for inputs and outputs that live in (pinned) host memory: while chunk c computes,
    chunk c+1's q_idx / w / q travel host -> device on a copy stream and chunk c-1's attention output
    travels device -> host on another, so the PCIe time overlaps the kernels.  Host tensors hold the
    rank's local rows (PrefillPipeline order); keys and latent KV are copied whole at the start of a call."""

    def __init__(self, pipe: PrefillPipeline, idx_heads: int = 64, idx_dim: int = 128, w_dtype=torch.bfloat16):
        self.p = pipe
        dev, S, R, H = pipe.device, pipe.S, pipe.rows_max, pipe.H
        self.k_idx = torch.empty(S, idx_dim, dtype=ops.FP8, device=dev)
        self.k_scale = torch.empty(S, dtype=torch.float32, device=dev)
        self.kv = torch.empty(S, 576, dtype=torch.bfloat16, device=dev)
        self.q_idx = [torch.empty(R, idx_heads, idx_dim, dtype=ops.FP8, device=dev) for _ in range(2)]
        self.w = [torch.empty(R, idx_heads, dtype=w_dtype, device=dev) for _ in range(2)]
        self.q = [torch.empty(R, H, 576, dtype=torch.bfloat16, device=dev) for _ in range(2)]
        self.out = [torch.empty(R, H, 512, dtype=torch.bfloat16, device=dev) for _ in range(2)] if pipe.world == 1 else None
        self.copy_in = torch.cuda.Stream(device=dev)
        self.copy_out = torch.cuda.Stream(device=dev)
        self._slot_busy = [None, None]
        self._out_busy = [None, None]
        self._keys_busy = None
        self._first = True

    @torch.no_grad()
    def submit(self, q_idx_h, k_idx_h, k_scale_h, w_h, q_h, kv_h, out_h, out_full=None):
        """Enqueue one prefill.  out_h [T_loc, H, 512] (host) receives the rank's rows; out_full (device,
        [S, H, 512]) is required when world > 1 and receives the gathered output.  Returns the event after
        which out_h is complete; nothing waits on the host."""
        p = self.p
        main = torch.cuda.current_stream(p.device)
        if self._first:
            self.copy_in.wait_stream(main)
            self.copy_out.wait_stream(main)
            self._first = False
        n = len(p.chunks)
        ready = [torch.cuda.Event() for _ in range(n)]
        p.begin(out_full)

        def stage(c):
            a, b, _, _ = p.chunks[c]
            s = c & 1
            with torch.cuda.stream(self.copy_in):
                if c == 0:
                    if self._keys_busy is not None:
                        self.copy_in.wait_event(self._keys_busy)
                    self.k_idx.copy_(k_idx_h, non_blocking=True)
                    self.k_scale.copy_(k_scale_h, non_blocking=True)
                    self.kv.copy_(kv_h, non_blocking=True)
                if self._slot_busy[s] is not None:
                    self.copy_in.wait_event(self._slot_busy[s])
                self.q_idx[s][: b - a].copy_(q_idx_h[a:b], non_blocking=True)
                self.w[s][: b - a].copy_(w_h[a:b], non_blocking=True)
                self.q[s][: b - a].copy_(q_h[a:b], non_blocking=True)
                ready[c].record(self.copy_in)

        stage(0)
        computed = None
        for c, (a, b, _, _) in enumerate(p.chunks):
            s = c & 1
            if c + 1 < n:
                stage(c + 1)
            main.wait_event(ready[c])
            if p.world == 1 and self._out_busy[s] is not None:
                main.wait_event(self._out_busy[s])
            dst = p.run_chunk(c, self.q_idx[s][: b - a], self.k_idx, self.k_scale, self.w[s][: b - a],
                              self.q[s][: b - a], self.kv, out_full, out_chunk=None if p.world > 1 else self.out[s][: b - a])
            computed = torch.cuda.Event()
            computed.record(main)
            self._slot_busy[s] = computed
            with torch.cuda.stream(self.copy_out):
                self.copy_out.wait_event(computed)
                out_h[a:b].copy_(dst, non_blocking=True)
                drained = torch.cuda.Event()
                drained.record(self.copy_out)
                if p.world == 1:
                    self._out_busy[s] = drained
                else:
                    # the rank's local output buffer is also read by this copy: the next writer must wait for it
                    if p._gathered[s] is not None:
                        self.copy_out.wait_event(p._gathered[s])
                    both = torch.cuda.Event()
                    both.record(self.copy_out)
                    p._gathered[s] = both
        self._keys_busy = computed
        p.finish()
        done = torch.cuda.Event()
        done.record(self.copy_out)
        return done


LATENT_TOKEN_BYTES = 656          # 512 e4m3 latent values, 4 fp32 group scales, 64 bf16 rope values


@torch.no_grad()
def pack_latent_cache(kv: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Latent KV rows [N, 576] (bf16 or fp32, CUDA) -> records of the paged FP8 latent cache, uint8
    [N, 656]: the 512 latent values as e4m3 with one fp32 scale per 128 values (the indexer quantiser's
    rule, sparse_attn/DSA.py:121-124: scale = max(absmax, 1e-6) / 448), then the 64 rope values as bf16.
    This is the write side of the cache sparse_mla_decode_paged reads; rows go to
    cache[block_table[b, pos // 64] * 64 + pos % 64]."""
    N = kv.shape[0]
    if kv.dim() != 2 or kv.shape[1] != 576:
        raise ops.DsaError(f"latent KV must be [N, 576], got {tuple(kv.shape)}")
    if out is None:
        out = torch.empty(N, LATENT_TOKEN_BYTES, dtype=torch.uint8, device=kv.device)
    q8, scale = ops.fp8_quant_per_block(kv[:, :512].contiguous(), 128)      # [N,512] e4m3, [N,4] fp32
    out[:, :512] = q8.view(torch.uint8)
    out[:, 512:528] = scale.contiguous().view(torch.uint8).view(N, 16)
    out[:, 528:] = kv[:, 512:].to(torch.bfloat16).contiguous().view(torch.uint8).view(N, 128)
    return out


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
