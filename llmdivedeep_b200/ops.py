"""Torch-facing wrappers over the C ABI: tensors in, tensors out, current stream.

Every function checks dtypes/shapes, passes raw device pointers to
libdsa_b200.so and raises ``DsaError`` when the library refuses the call.
Nothing here computes on the CPU.
"""
from __future__ import annotations

from typing import Optional

import torch

from . import _lib
from ._lib import DsaError, check

FP8 = torch.float8_e4m3fn
_status = {}


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


def _need_cuda(*ts) -> torch.device:
    """All tensors must live on ONE CUDA device; returns it.  The library launches on the current
    device (tensor maps, SM count and the stream follow it), so every wrapper below makes this
    device current around its call: a tensor of another GPU would otherwise be handed to a kernel
    running on the wrong one."""
    dev = None
    for t in ts:
        if t is None:
            continue
        if not t.is_cuda:
            raise DsaError("libdsa_b200 kernels take CUDA tensors only (there is no CPU path)")
        if dev is None:
            dev = t.device
        elif t.device != dev:
            raise DsaError(f"all tensors of one call must be on one device, got {dev} and {t.device}")
    if dev is None:
        raise DsaError("no tensor argument")
    return dev


def _dev_index(device) -> int:
    d = torch.device(device)
    if d.type != "cuda":
        raise DsaError(f"not a CUDA device: {d}")
    return torch.cuda.current_device() if d.index is None else d.index


def status_word(device) -> torch.Tensor:
    """The per-device int32 the kernels report soft errors into (a device without an index means
    the current one)."""
    key = _dev_index(device)
    if key not in _status:
        _status[key] = torch.zeros(1, dtype=torch.int32, device=f"cuda:{key}")
    return _status[key]


def check_status(device) -> None:
    """Synchronise and raise if a kernel flagged a soft error since the last check."""
    w = status_word(device)
    v = int(w.item())
    if v:
        w.zero_()
        what = {1: "a bounded wait inside a kernel expired", 2: "an index or page id was out of range"}.get(v, "?")
        raise DsaError(f"device status {v}: {what}")


def _w_dtype(w: torch.Tensor) -> int:
    if w.dtype == torch.float32:
        return 0
    if w.dtype == torch.bfloat16:
        return 1
    raise DsaError(f"head weights must be fp32 or bf16, got {w.dtype}")


def _as_i32(t: Optional[torch.Tensor], n: int, name: str) -> Optional[torch.Tensor]:
    if t is None:
        return None
    if t.dtype != torch.int32 or t.numel() != n or not t.is_contiguous():
        raise DsaError(f"{name} must be a contiguous int32 tensor of {n} elements")
    return t


def _check_idx_out(out: Optional[torch.Tensor], T: int, k: int, device) -> torch.Tensor:
    """The kernels write index rows at stride k: a caller-supplied ``out`` must be exactly that."""
    if out is None:
        return torch.empty(T, k, dtype=torch.int32, device=device)
    if out.dtype != torch.int32 or tuple(out.shape) != (T, k) or not out.is_contiguous():
        raise DsaError(f"out must be a contiguous int32 [{T}, {k}] tensor, got {out.dtype} {tuple(out.shape)} "
                       f"strides {tuple(out.stride())}")
    return out


def _check_attn_out(out: Optional[torch.Tensor], shape, device) -> torch.Tensor:
    """The attention kernels write dense bf16 rows: a caller-supplied ``out`` must be exactly that."""
    if out is None:
        return torch.empty(shape, dtype=torch.bfloat16, device=device)
    if out.dtype != torch.bfloat16 or tuple(out.shape) != tuple(shape) or not out.is_contiguous():
        raise DsaError(f"out must be a contiguous bfloat16 {list(shape)} tensor, got {out.dtype} {tuple(out.shape)} "
                       f"strides {tuple(out.stride())}")
    return out


def fp8_mqa_logits(q_fp8, kv, weights, ks, ke, clean_logits: bool = True,
                   out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Drop-in for ``deep_gemm.fp8_mqa_logits(q_fp8, (k_fp8, k_scale), w, ks, ke)``
    as the reference calls it (sparse_attn/DSA.py:343-345).  Returns fp32 [T, S]."""
    k_fp8, k_scale = kv
    dev = _need_cuda(q_fp8, k_fp8, k_scale, weights, ks, ke, out)
    if q_fp8.dtype != FP8 or k_fp8.dtype != FP8:
        raise DsaError("q and k must be float8_e4m3fn")
    if q_fp8.dim() != 3 or k_fp8.dim() != 2 or q_fp8.shape[2] != k_fp8.shape[1]:
        raise DsaError(f"bad shapes q {tuple(q_fp8.shape)} k {tuple(k_fp8.shape)}")
    T, H, D = q_fp8.shape
    S = k_fp8.shape[0]
    q_fp8, k_fp8 = q_fp8.contiguous(), k_fp8.contiguous()
    k_scale = k_scale.reshape(-1).to(torch.float32).contiguous()
    weights = weights.contiguous()
    if k_scale.numel() != S or tuple(weights.shape) != (T, H):
        raise DsaError("k_scale must have S entries and weights must be [T, H]")
    ks = _as_i32(ks, T, "ks")
    ke = _as_i32(ke, T, "ke")
    ld = (S + 3) // 4 * 4
    if out is None:
        out = torch.empty(T, ld, dtype=torch.float32, device=q_fp8.device)
    elif out.dtype != torch.float32 or out.dim() != 2 or out.shape[0] < T or out.stride(1) != 1 or out.stride(0) < S:
        raise DsaError("out must be fp32 [>=T, >=S] with unit column stride")
    else:
        ld = out.stride(0)
    lib = _lib.load()
    with torch.cuda.device(dev):
        check(lib.dsa_indexer_logits(_ptr(q_fp8), _ptr(k_fp8), _ptr(k_scale), _ptr(weights), _w_dtype(weights),
                                     _ptr(ks), _ptr(ke), _ptr(out), ld, T, S, H, D, int(bool(clean_logits)),
                                     _ptr(status_word(q_fp8.device)), _stream()))
    return out[:T, :S]


def fp8_paged_mqa_logits(q_fp8, weights, kcache, kscale, block_table, ctx_len, max_ctx: int,
                         out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Decode indexer over the paged FP8 key cache.  q_fp8 [B,H,128], weights [B,H],
    kcache [num_pages*64,128] e4m3, kscale [num_pages*64] fp32, block_table [B,P] int32,
    ctx_len [B] int32.  Returns fp32 [B, max_ctx]; columns >= ctx_len[b] inside a
    processed 128-key tile hold -inf, columns beyond are uninitialised."""
    dev = _need_cuda(q_fp8, weights, kcache, kscale, block_table, ctx_len, out)
    B, H, D = q_fp8.shape
    if kcache.dtype != FP8 or q_fp8.dtype != FP8 or kcache.dim() != 2 or kcache.shape[1] != D:
        raise DsaError("kcache must be float8_e4m3fn [num_pages*64, D]")
    if kcache.shape[0] % 64:
        raise DsaError("kcache rows must be a multiple of the 64-token page")
    block_table = block_table.contiguous()
    if block_table.dtype != torch.int32 or block_table.shape[0] != B:
        raise DsaError("block_table must be int32 [B, pages]")
    ctx_len = _as_i32(ctx_len, B, "ctx_len")
    q_fp8, kcache, weights = q_fp8.contiguous(), kcache.contiguous(), weights.contiguous()
    kscale = kscale.reshape(-1).to(torch.float32).contiguous()
    ld = (max_ctx + 3) // 4 * 4
    if out is None:
        out = torch.empty(B, ld, dtype=torch.float32, device=q_fp8.device)
    else:
        ld = out.stride(0)
    lib = _lib.load()
    with torch.cuda.device(dev):
        check(lib.dsa_indexer_logits_paged(_ptr(q_fp8), _ptr(weights), _w_dtype(weights), _ptr(kcache), _ptr(kscale),
                                           _ptr(block_table), block_table.stride(0), _ptr(ctx_len), _ptr(out), ld,
                                           B, H, D, kcache.shape[0] // 64, max_ctx,
                                           _ptr(status_word(q_fp8.device)), _stream()))
    return out[:B, :max_ctx]


def topk_select(logits: torch.Tensor, k: int, ks=None, ke=None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Indices (int32, unsorted) of the k largest entries of each row's window
    [ks, ke); -1 padding when the window holds fewer than k columns."""
    dev = _need_cuda(logits, ks, ke, out)
    if logits.dtype != torch.float32 or logits.dim() != 2 or logits.stride(1) != 1:
        raise DsaError("logits must be fp32 [T, S] with unit column stride")
    T, S = logits.shape
    ks = _as_i32(ks, T, "ks")
    ke = _as_i32(ke, T, "ke")
    out = _check_idx_out(out, T, k, logits.device)
    lib = _lib.load()
    with torch.cuda.device(dev):
        check(lib.dsa_topk_select(_ptr(logits), logits.stride(0) if T > 1 else max(S, logits.stride(0)), _ptr(ks),
                                  _ptr(ke), T, S, k, _ptr(out), _stream()))
    return out


_workspaces = {}


def _workspace(device, nbytes: int) -> torch.Tensor:
    key = _dev_index(device)
    w = _workspaces.get(key)
    if w is None or w.numel() < nbytes:
        _workspaces[key] = w = torch.empty(nbytes, dtype=torch.uint8, device=f"cuda:{key}")
    return w


def indexer_topk(q_fp8, k_fp8, k_scale, weights, ks, ke, k: int, workspace: Optional[torch.Tensor] = None,
                 max_workspace_bytes: int = 8 << 30, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Indexer logits + top-k (IndexerSimulator.logits_step, sparse_attn/DSA.py:336-362)
    in one library call.  Returns int32 [T, min(k, S)]."""
    dev = _need_cuda(q_fp8, k_fp8, k_scale, weights, ks, ke, workspace, out)
    T, H, D = q_fp8.shape
    S = k_fp8.shape[0]
    k = min(k, S)
    q_fp8, k_fp8, weights = q_fp8.contiguous(), k_fp8.contiguous(), weights.contiguous()
    k_scale = k_scale.reshape(-1).to(torch.float32).contiguous()
    ks = _as_i32(ks, T, "ks")
    ke = _as_i32(ke, T, "ke")
    lib = _lib.load()
    if workspace is None:
        full = lib.dsa_indexer_topk_workspace_bytes(T, S)
        row = full // max(T, 1)
        workspace = _workspace(q_fp8.device, min(full, max(max_workspace_bytes, 256 * row)))
    out = _check_idx_out(out, T, k, q_fp8.device)
    with torch.cuda.device(dev):
        check(lib.dsa_indexer_topk(_ptr(q_fp8), _ptr(k_fp8), _ptr(k_scale), _ptr(weights), _w_dtype(weights),
                                   _ptr(ks), _ptr(ke), T, S, H, D, k, _ptr(out), _ptr(workspace), workspace.numel(),
                                   _ptr(status_word(q_fp8.device)), _stream()))
    return out


def indexer_topk_static(q_fp8, k_fp8, k_scale, weights, ks, ke, k: int, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``indexer_topk`` for callers that may not allocate: the logits scratch is the
    64 MiB array built into the library (shared by every call on the device, so
    calls that overlap on the GPU race).  ``out`` should be passed by such callers;
    it is only created here when omitted.  Sizes beyond the array are refused."""
    dev = _need_cuda(q_fp8, k_fp8, k_scale, weights, ks, ke, out)
    T, H, D = q_fp8.shape
    S = k_fp8.shape[0]
    k = min(k, S)
    for t in (q_fp8, k_fp8, weights, k_scale):
        if not t.is_contiguous():
            raise DsaError("indexer_topk_static takes contiguous tensors (it will not copy)")
    if k_scale.dtype != torch.float32 or k_scale.numel() != S:
        raise DsaError("k_scale must be fp32 with one entry per key")
    ks = _as_i32(ks, T, "ks")
    ke = _as_i32(ke, T, "ke")
    out = _check_idx_out(out, T, k, q_fp8.device)
    lib = _lib.load()
    with torch.cuda.device(dev):
        check(lib.dsa_indexer_topk_static(_ptr(q_fp8), _ptr(k_fp8), _ptr(k_scale), _ptr(weights), _w_dtype(weights),
                                          _ptr(ks), _ptr(ke), T, S, H, D, k, _ptr(out),
                                          _ptr(status_word(q_fp8.device)), _stream()))
    return out


def sparse_mla_prefill(q, kv, idx, scale: float, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Sparse MLA over selected latent-KV rows.  q [T,H,576] bf16, kv [S,576] bf16,
    idx [T,K] int32 (negative = empty slot).  Returns bf16 [T,H,512]."""
    dev = _need_cuda(q, kv, idx, out)
    if q.dtype != torch.bfloat16 or kv.dtype != torch.bfloat16 or idx.dtype != torch.int32:
        raise DsaError("sparse_mla_prefill takes bf16 q/kv and int32 idx")
    if q.dim() != 3 or q.shape[2] != 576 or kv.dim() != 2 or kv.shape[1] != 576 or idx.dim() != 2 or idx.shape[0] != q.shape[0]:
        raise DsaError(f"bad shapes q {tuple(q.shape)} kv {tuple(kv.shape)} idx {tuple(idx.shape)}")
    q, kv, idx = q.contiguous(), kv.contiguous(), idx.contiguous()
    T, H, _ = q.shape
    out = _check_attn_out(out, (T, H, 512), q.device)
    lib = _lib.load()
    with torch.cuda.device(dev):
        check(lib.dsa_sparse_mla_prefill(_ptr(q), _ptr(kv), _ptr(idx), _ptr(out), T, H, kv.shape[0], idx.shape[1],
                                         float(scale), _ptr(status_word(q.device)), _stream()))
    return out


def block_sparse_attn(q, k, v, lut, num, sm_scale: float, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Block-sparse multi-head attention with the reference's stand-in signature (sparse_attn/DSA.py:232-247):
    q, k, v [B, S, H, 128] bf16; lut [B, H, S/64, topk] int32 key-block ids per 64-row query block;
    num [B, H, S/64] int32 = how many entries of each list count.  Non-causal.  Returns bf16 [B, S, H, 128]."""
    dev = _need_cuda(q, k, v, lut, num, out)
    if any(t.dtype != torch.bfloat16 for t in (q, k, v)) or lut.dtype != torch.int32 or num.dtype != torch.int32:
        raise DsaError("block_sparse_attn takes bf16 q/k/v and int32 lut/num")
    if q.dim() != 4 or k.shape != q.shape or v.shape != q.shape:
        raise DsaError(f"bad shapes q {tuple(q.shape)} k {tuple(k.shape)} v {tuple(v.shape)}")
    B, S, H, D = q.shape
    if lut.dim() != 4 or tuple(lut.shape[:3]) != (B, H, S // 64) or tuple(num.shape) != (B, H, S // 64):
        raise DsaError(f"bad shapes lut {tuple(lut.shape)} num {tuple(num.shape)} for q {tuple(q.shape)}")
    q, k, v, lut, num = q.contiguous(), k.contiguous(), v.contiguous(), lut.contiguous(), num.contiguous()
    if out is None:
        out = torch.empty_like(q)
    lib = _lib.load()
    with torch.cuda.device(dev):
        check(lib.dsa_block_sparse_mha(_ptr(q), _ptr(k), _ptr(v), _ptr(lut), _ptr(num), _ptr(out), B, S, H, D,
                                       lut.shape[3], float(sm_scale), _ptr(status_word(q.device)), _stream()))
    return out


def sparse_mla_decode_paged(q, cache, block_table, idx, scale: float, max_ctx: Optional[int] = None,
                            out: Optional[torch.Tensor] = None, workspace: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Decode step over the paged FP8 latent cache.  q [B,H,576] bf16, cache uint8
    [num_pages*64, 656], block_table [B,P] int32, idx [B,K] int32 logical positions."""
    dev = _need_cuda(q, cache, block_table, idx, out, workspace)
    if q.dtype != torch.bfloat16 or cache.dtype != torch.uint8 or idx.dtype != torch.int32 or block_table.dtype != torch.int32:
        raise DsaError("sparse_mla_decode_paged takes bf16 q, uint8 cache, int32 block_table/idx")
    if cache.dim() != 2 or cache.shape[1] != 656 or cache.shape[0] % 64:
        raise DsaError("cache must be uint8 [num_pages*64, 656]")
    q, cache, block_table, idx = q.contiguous(), cache.contiguous(), block_table.contiguous(), idx.contiguous()
    B, H, _ = q.shape
    if max_ctx is None:
        max_ctx = block_table.shape[1] * 64
    out = _check_attn_out(out, (B, H, 512), q.device)
    lib = _lib.load()
    if workspace is None:
        need = lib.dsa_sparse_mla_decode_workspace_bytes(B, H, idx.shape[1])
        workspace = _workspace(q.device, need) if need else None
    with torch.cuda.device(dev):
        check(lib.dsa_sparse_mla_decode_paged(_ptr(q), _ptr(cache), _ptr(block_table), block_table.stride(0), _ptr(idx),
                                              _ptr(out), B, H, idx.shape[1], cache.shape[0] // 64, max_ctx, float(scale),
                                              _ptr(workspace), workspace.numel() if workspace is not None else 0,
                                              _ptr(status_word(q.device)), _stream()))
    return out


class HostIndexerPipeline:
    """indexer_topk for inputs and outputs that live in (pinned) host memory.

    The call is cut into chunks of query rows: while chunk i is scored on the compute stream,
    chunk i+1's q / weights / windows travel host -> device on a copy stream and chunk i-1's
    indices travel device -> host, so the PCIe time hides behind the kernels instead of adding
    to them.  The keys (shared by every chunk) are copied first.  Device staging buffers are
    allocated once per shape and reused."""

    def __init__(self, T: int, S: int, H: int, D: int, k: int, device, chunks: int = 4, w_dtype=torch.float32):
        self.T, self.S, self.H, self.D, self.k, self.device = T, S, H, D, min(k, S), torch.device(device)
        self.bounds = self.chunk_bounds(T, chunks)
        rows = max(b - a for a, b in self.bounds)
        dev = self.device
        self.k_fp8 = [torch.empty(S, D, dtype=FP8, device=dev) for _ in range(2)]       # alternate between calls
        self.k_scale = [torch.empty(S, dtype=torch.float32, device=dev) for _ in range(2)]
        self._calls = 0
        self._k_busy = [None, None]        # per key buffer: event after the last kernels that read it
        self._slot_busy = [None, None]     # per input staging slot: event after the kernels that read it
        self._out_busy = [None, None]      # per output slot: event after its device -> host copy
        self.q = [torch.empty(rows, H, D, dtype=FP8, device=dev) for _ in range(2)]
        self.w = [torch.empty(rows, H, dtype=w_dtype, device=dev) for _ in range(2)]
        self.ks = [torch.empty(rows, dtype=torch.int32, device=dev) for _ in range(2)]
        self.ke = [torch.empty(rows, dtype=torch.int32, device=dev) for _ in range(2)]
        self.out = [torch.empty(rows, self.k, dtype=torch.int32, device=dev) for _ in range(2)]
        lib = _lib.load()
        self.ws = torch.empty(lib.dsa_indexer_topk_workspace_bytes(rows, S), dtype=torch.uint8, device=dev)
        self.copy_in = torch.cuda.Stream(device=dev)
        self.copy_out = torch.cuda.Stream(device=dev)

    @staticmethod
    def chunk_bounds(T: int, chunks: int):
        """Row ranges of the chunks, in whole 256-row groups.  With four or more chunks the first one is
        small (its host -> device copy, together with the keys', is the part no kernel can hide) and so is
        the last (its device -> host copy is exposed the same way); the rows between are split evenly."""
        groups = -(-T // 256)
        if chunks < 4 or groups < 2 * chunks:
            per = max(1, -(-groups // max(chunks, 1)))
            sizes = [per] * (-(-groups // per))
        else:
            first = max(1, groups // 16)
            last = 2 * first
            mid = groups - first - last
            per, extra = divmod(mid, chunks - 2)
            sizes = [first] + [per + (1 if i >= chunks - 2 - extra else 0) for i in range(chunks - 2)] + [last]
        bounds, a = [], 0
        for g in sizes:
            b = min(T, a + g * 256)
            if b > a:
                bounds.append((a, b))
            a = b
        return bounds

    def submit(self, q_host, k_host, k_scale_host, w_host, ks_host, ke_host, out_host) -> "torch.cuda.Event":
        """Enqueue one call; all arguments are host tensors (pinned for real overlap), out_host int32 [T, k].
        Returns the event after which out_host holds the result.  Nothing here waits on the host, and the
        current stream is not made to wait for the output copy, so a caller that submits call after call
        gets the next call's input copies under this call's kernels (staging slots and the two key buffers
        are handed over by events)."""
        main = torch.cuda.current_stream(self.device)
        n = len(self.bounds)
        in_ready = [torch.cuda.Event() for _ in range(n)]
        kb = self._calls & 1
        if self._calls == 0:                       # staging buffers were allocated on the current stream
            self.copy_in.wait_stream(main)
            self.copy_out.wait_stream(main)
        k_fp8, k_scale = self.k_fp8[kb], self.k_scale[kb]

        def stage(i):          # enqueue the host -> device copies of chunk i (events it waits on are already recorded)
            a, b = self.bounds[i]
            s = i & 1
            with torch.cuda.stream(self.copy_in):
                if i == 0:
                    if self._k_busy[kb] is not None:
                        self.copy_in.wait_event(self._k_busy[kb])    # last kernels that read this key buffer
                    k_fp8.copy_(k_host, non_blocking=True)
                    k_scale.copy_(k_scale_host, non_blocking=True)
                if self._slot_busy[s] is not None:
                    self.copy_in.wait_event(self._slot_busy[s])      # staging slot free again
                self.q[s][: b - a].copy_(q_host[a:b], non_blocking=True)
                self.w[s][: b - a].copy_(w_host[a:b], non_blocking=True)
                self.ke[s][: b - a].copy_(ke_host[a:b], non_blocking=True)
                if ks_host is not None:
                    self.ks[s][: b - a].copy_(ks_host[a:b], non_blocking=True)
                else:
                    self.ks[s].zero_()
                in_ready[i].record(self.copy_in)

        stage(0)
        if n > 1:
            stage(1)
        computed = None
        for i, (a, b) in enumerate(self.bounds):
            s = i & 1
            main.wait_event(in_ready[i])
            if self._out_busy[s] is not None:
                main.wait_event(self._out_busy[s])                   # output slot copied out
            indexer_topk(self.q[s][: b - a], k_fp8, k_scale, self.w[s][: b - a], self.ks[s][: b - a],
                         self.ke[s][: b - a], self.k, workspace=self.ws, out=self.out[s][: b - a])
            computed = torch.cuda.Event()
            computed.record(main)
            self._slot_busy[s] = computed
            if i + 2 < n:
                stage(i + 2)
            with torch.cuda.stream(self.copy_out):
                self.copy_out.wait_event(computed)
                out_host[a:b].copy_(self.out[s][: b - a], non_blocking=True)
                drained = torch.cuda.Event()
                drained.record(self.copy_out)
                self._out_busy[s] = drained
        self._k_busy[kb] = computed
        self._calls += 1
        done = torch.cuda.Event()
        done.record(self.copy_out)
        return done

    def __call__(self, q_host, k_host, k_scale_host, w_host, ks_host, ke_host, out_host) -> torch.Tensor:
        """submit(), then the current stream waits for the output copy: work queued after this call (or a
        synchronize of the current stream) sees out_host filled."""
        done = self.submit(q_host, k_host, k_scale_host, w_host, ks_host, ke_host, out_host)
        torch.cuda.current_stream(self.device).wait_event(done)
        return out_host


def fp8_quant_per_block(x: torch.Tensor, block_size: int = 128):
    """One-kernel FP8 e4m3 quantiser with the reference's semantics (sparse_attn/DSA.py:102-132):
    returns (q float8_e4m3fn with x's shape, scale fp32); the scale drops its last dim when a row
    is one block.  x is bf16 or fp32 on a CUDA device."""
    dev = _need_cuda(x)
    last = x.shape[-1]
    assert last % block_size == 0, f"last dim {last} not multiple of block {block_size}"
    if x.dtype not in (torch.float32, torch.bfloat16):
        x = x.float()
    x = x.contiguous()
    nb = last // block_size
    n_blocks = x.numel() // block_size
    q = torch.empty(x.shape, dtype=FP8, device=x.device)
    scale = torch.empty(n_blocks, dtype=torch.float32, device=x.device)
    lib = _lib.load()
    with torch.cuda.device(dev):
        check(lib.dsa_fp8_quant_per_block(_ptr(x), 1 if x.dtype == torch.bfloat16 else 0, n_blocks, block_size,
                                          _ptr(q), _ptr(scale), _stream()))
    return q, (scale.view(x.shape[:-1]) if nb == 1 else scale.view(*x.shape[:-1], nb))


def rope_fp8_quant(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, rope_dim: int, interleave: bool,
                   rows_per_pos: int = 1):
    """RoPE on the first ``rope_dim`` values of every head row followed by the per-row FP8 quantiser, one kernel
    (DsaIndexer.rope + fp8_quant_per_block, sparse_attn/DSA.py:513-524, 530-531).  x bf16 [..., head_dim] with
    head_dim 64 or 128; cos / sin fp32 [positions, rope_dim / 2]; the row with flat index r sits at position
    r // rows_per_pos.  Returns (q float8_e4m3fn like x, scale fp32 x.shape[:-1]), bit-identical to the eager chain."""
    dev = _need_cuda(x, cos, sin)
    if x.dtype != torch.bfloat16 or cos.dtype != torch.float32 or sin.dtype != torch.float32:
        raise DsaError("rope_fp8_quant takes bf16 x and fp32 cos / sin tables")
    D = x.shape[-1]
    x, cos, sin = x.contiguous(), cos.contiguous(), sin.contiguous()
    if cos.shape != sin.shape or cos.dim() != 2 or cos.shape[1] * 2 != rope_dim:
        raise DsaError(f"cos / sin must be [positions, {rope_dim // 2}], got {tuple(cos.shape)}")
    n_rows = x.numel() // D
    q = torch.empty(x.shape, dtype=FP8, device=x.device)
    scale = torch.empty(x.shape[:-1], dtype=torch.float32, device=x.device)
    lib = _lib.load()
    with torch.cuda.device(dev):
        check(lib.dsa_rope_fp8_quant(_ptr(x), n_rows, D, rope_dim, int(bool(interleave)), rows_per_pos, _ptr(cos), _ptr(sin),
                                     cos.shape[0], _ptr(q), _ptr(scale), _stream()))
    return q, scale
