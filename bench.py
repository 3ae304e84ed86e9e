#!/usr/bin/env python
"""Benchmark of the DSA hot path: one full prefill at 128K context, and the decode step.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (one "step"): DSA prefill of ONE sequence of 131072 tokens, causal -- lightning indexer
(64 heads x 128, FP8 e4m3 with per-token scales, ReLU, head-weighted sum) -> top-k 2048 per query
row -> sparse MLA over the selected keys (128 query heads, qk 576 / v 512, bf16, one shared latent
KV row per token) -- run through ``layer.PrefillPipeline`` in chunks of query rows.  Inputs are
seeded synthetic N(0,1) tensors quantised the way the reference's own drivers do; the reference
measures on synthetic tensors only, so no external data stands behind them.

With N > 1 (launched by torch.distributed.run, one rank per GPU) the SAME sequence is split over the
ranks (strong scaling): 256-row blocks of query rows dealt round-robin, keys and latent KV replicated,
and the attention output of every finished chunk all-gathered over NCCL on a side stream while the
next chunk computes, so that every rank ends with the full [131072, 128, 512] output.

Rank 0 prints ONE JSON line.  `value` is device-resident tokens/s, `e2e` the same step with every
input copied from pinned host memory and the attention output copied back inside the timed region,
`roofline` is for the kernel that takes the largest share of the step, `cpu_baseline` times the CPU
oracle on a bounded sample of query rows, `parity` checks a sample of the timed output against the
oracle, and `sub` holds the other named configurations (indexer + top-k 4096 x 65536, sparse MLA at
32768 tokens, the decode step at batch 64 / context 131072) each with its own roofline block.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch

S_PREFILL = 131072
HEADS, DIM, TOPK = 64, 128, 2048          # indexer heads, indexer head dim, selected keys per query
MLA_HEADS, SCALE = 128, 192 ** -0.5
T_ROWS, S_KEYS = 4096, 65536              # the standalone indexer + top-k configuration
BLOCK_ROWS = 256
FP8 = torch.float8_e4m3fn
METRIC = "DSA prefill tokens/s @128K ctx (lightning indexer -> top-k 2048 -> sparse MLA, one 131072-token sequence)"
WORKLOAD = ("full DSA prefill, batch 1, seq 131072, causal: indexer 64 heads x 128 fp8 e4m3 -> top-k 2048 -> sparse MLA "
            "128 heads, qk 576 / v 512, bf16, shared latent KV [131072, 576]")


# ---------------------------------------------------------------------------------------------------
# synthetic inputs
# ---------------------------------------------------------------------------------------------------
def _quant_rows(x):
    """Per-row absmax e4m3 quantisation (sparse_attn/DSA.py:102-132 semantics, one block per row)."""
    scale = x.abs().amax(-1, keepdim=True).clamp_min(1e-6) / 448.0
    return (x / scale).to(FP8), scale.squeeze(-1)


def make_indexer_inputs(device, seed, rows=T_ROWS, n_keys=S_KEYS):
    """The standalone indexer configuration: `rows` queries at the last positions of `n_keys` keys.
    Seeded N(0,1) q/k, per-row e4m3, q scale and 128**-0.5 folded into bf16 head weights ~N(0,1)/8."""
    g = torch.Generator(device=device).manual_seed(seed)
    q = torch.randn(rows, HEADS, DIM, device=device, generator=g)
    k = torch.randn(n_keys, DIM, device=device, generator=g)
    w = torch.randn(rows, HEADS, device=device, generator=g) / 8
    q8, qs = _quant_rows(q)
    k8, ksc = _quant_rows(k)
    w_eff = (w * qs * DIM ** -0.5).to(torch.bfloat16)
    ks = torch.zeros(rows, dtype=torch.int32, device=device)
    ke = (torch.arange(rows, device=device) + (n_keys - rows) + 1).to(torch.int32)
    return q8, k8, ksc.contiguous(), w_eff.contiguous(), ks, ke


def make_prefill_inputs(device, seed, S, pos):
    """Inputs of one prefill for the rows at global positions `pos` (int tensor, this rank's rows):
    replicated keys / latent KV from `seed` (identical on every rank), per-row tensors from a generator
    seeded by the row's 256-row block, so that a row's values do not depend on how rows are dealt."""
    g = torch.Generator(device=device).manual_seed(seed)
    k8, ksc = _quant_rows(torch.randn(S, DIM, device=device, generator=g))
    kv = torch.randn(S, 576, device=device, generator=g).to(torch.bfloat16)
    T = pos.numel()
    q8 = torch.empty(T, HEADS, DIM, dtype=FP8, device=device)
    w = torch.empty(T, HEADS, dtype=torch.bfloat16, device=device)
    q = torch.empty(T, MLA_HEADS, 576, dtype=torch.bfloat16, device=device)
    for a in range(0, T, BLOCK_ROWS):
        b = min(T, a + BLOCK_ROWS)
        gb = torch.Generator(device=device).manual_seed(seed * 1000003 + int(pos[a]) // BLOCK_ROWS + 1)
        qq, qs = _quant_rows(torch.randn(b - a, HEADS, DIM, device=device, generator=gb))
        q8[a:b] = qq
        w[a:b] = (torch.randn(b - a, HEADS, device=device, generator=gb) / 8 * qs * DIM ** -0.5).to(torch.bfloat16)
        q[a:b] = torch.randn(b - a, MLA_HEADS, 576, device=device, generator=gb).to(torch.bfloat16)
    return q8, k8, ksc.contiguous(), w, q, kv


def draw_topk_positions(T, S, K, device, g, first=0):
    """idx [T, K] int32 for queries at positions first..first+T-1: K positions drawn uniformly WITHOUT
    replacement from [0, t]; all of [0, t] then -1 when t + 1 < K."""
    idx = torch.empty(T, K, dtype=torch.int32, device=device)
    cols = torch.arange(S, device=device).unsqueeze(0)
    for r0 in range(0, T, 2048):
        r1 = min(T, r0 + 2048)
        t = torch.arange(first + r0, first + r1, device=device).unsqueeze(1)
        r = torch.rand(r1 - r0, S, device=device, generator=g)
        r.masked_fill_(cols > t, 2.0)                               # never drawn
        val, sel = r.topk(K, dim=1, largest=False)
        idx[r0:r1] = torch.where(val < 2.0, sel, torch.full_like(sel, -1)).int()
    return idx


def make_decode_inputs(dev, B, CTX, g):
    """Paged FP8 caches of a decode batch: values ~N(0,1) before quantisation, 64-token pages in random order."""
    from llmdivedeep_b200 import layer, ops
    P = CTX // 64
    n_rows = B * P * 64
    kcache = torch.empty(n_rows, DIM, dtype=FP8, device=dev)
    kscale = torch.empty(n_rows, dtype=torch.float32, device=dev)
    latent = torch.empty(n_rows, 656, dtype=torch.uint8, device=dev)
    step = 1 << 19
    for a in range(0, n_rows, step):
        b = min(n_rows, a + step)
        k8, ksc = _quant_rows(torch.randn(b - a, DIM, device=dev, generator=g))
        kcache[a:b], kscale[a:b] = k8, ksc
        layer.pack_latent_cache(torch.randn(b - a, 576, device=dev, generator=g).to(torch.bfloat16), out=latent[a:b])
    table = torch.randperm(B * P, device=dev, generator=g).int().view(B, P)
    ctx = torch.full((B,), CTX, dtype=torch.int32, device=dev)
    q8, qs = _quant_rows(torch.randn(B, HEADS, DIM, device=dev, generator=g))
    w = (torch.randn(B, HEADS, device=dev, generator=g) / 8 * qs * DIM ** -0.5).contiguous()
    qd = torch.randn(B, MLA_HEADS, 576, device=dev, generator=g).to(torch.bfloat16)
    return q8, w, kcache, kscale, table, ctx, qd, latent


# ---------------------------------------------------------------------------------------------------
# helpers
# ---------------------------------------------------------------------------------------------------
class ClockSampler:
    """Samples SM clock and throttle reasons through NVML while a timed region runs."""

    def __init__(self, index):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _run(self):
        nv = self.nv
        names = {
            getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8): "hw_slowdown",
            getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40): "hw_thermal_slowdown",
            getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20): "sw_thermal_slowdown",
            getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4): "sw_power_cap",
        }
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                try:
                    r = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                except Exception:
                    r = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for bit, name in names.items():
                    if r & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(0.004)

    def start(self):
        if self.nv:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        return self

    def stop(self):
        if self._thread:
            self._stop.set()
            self._thread.join()
        return {"sm_mhz": statistics.median(self.samples) if self.samples else None,
                "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": len(self.samples)}


def _time_ms(fn, iters, warm=2):
    """The reference's timing convention (common/bench_utils.py:15-28): warm-up, then CUDA events
    around `iters` back-to-back calls on the current stream, one synchronise."""
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def _sustained(fn, local, seconds=2.0):
    """`fn` back to back for about `seconds`: ms per call and the median SM clock sampled meanwhile."""
    one = _time_ms(fn, 1, warm=1)
    iters = max(2, int(seconds * 1e3 / max(one, 1e-3)))
    s = ClockSampler(local).start()
    ms = _time_ms(fn, iters, warm=0)
    c = s.stop()
    return {"ms": ms, "iters": iters, "sm_mhz_median": c["sm_mhz"], "reasons": c["reasons"]}


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        return json.load(open(p)), "measured"
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}, "fallback"


def causal_keys(S):
    return S * (S + 1) // 2


def mla_pairs(S, K=TOPK):
    """sum_t min(t + 1, K): selected (query, key) pairs of a causal prefill."""
    return sum(min(t + 1, K) for t in range(min(S, K))) + max(0, S - K) * K


# ---------------------------------------------------------------------------------------------------
# CPU legs (the only code here that runs the oracle)
# ---------------------------------------------------------------------------------------------------
def cpu_prefill_rows(rows_pos, S, seed):
    """CPU oracle (the reference's fp32 fallback arithmetic with the ReLU, row-chunked, + torch.topk,
    + the fp32 sparse-MLA restatement) on the query rows at positions rows_pos of the S-token prefill.
    Inputs are generated before the clock starts.  Returns (seconds, threads)."""
    from oracle import dsa_oracle as O
    torch.set_num_threads(len(os.sched_getaffinity(0)))
    g = torch.Generator().manual_seed(seed)
    R = len(rows_pos)
    q8, qs = _quant_rows(torch.randn(R, HEADS, DIM, generator=g))
    k8, ksc = _quant_rows(torch.randn(S, DIM, generator=g))
    w = (torch.randn(R, HEADS, generator=g) / 8 * qs * DIM ** -0.5)
    q = torch.randn(R, MLA_HEADS, 576, generator=g).to(torch.bfloat16)
    kv = torch.randn(S, 576, generator=g).to(torch.bfloat16)
    ks = torch.zeros(R, dtype=torch.int32)
    ke = (torch.tensor(rows_pos) + 1).to(torch.int32)
    t0 = time.perf_counter()
    lg = O.indexer_logits(q8, k8, ksc, w, ks, ke, relu=True, row_chunk=8)
    top = O.topk_indices(lg, TOPK)
    idx = torch.where(torch.gather(lg, 1, top) == float("-inf"), torch.full_like(top, -1), top).to(torch.int32)
    O.sparse_mla(q, kv, idx, SCALE, row_chunk=8)
    return time.perf_counter() - t0, torch.get_num_threads()


def sample_positions(S, n):
    """n query positions spread evenly over the sequence (mean causal window = S / 2), the last row included."""
    return [min(S - 1, (2 * i + 1) * S // (2 * n)) for i in range(n - 1)] + [S - 1]


def run_reference(args, rank):
    """Reference arm: the reference's own CPU path for this workload -- its fp32 fallback scorer +
    torch.topk (sparse_attn/DSA.py:348-361), restated with row streaming because the original
    materialises [T,H,S] fp32, and with the ReLU of its math note; the sparse-MLA step, which the
    reference does not implement, is the oracle's fp32 restatement.  All host threads; each step is a
    bounded sample of query rows spread evenly over the 131072-token sequence."""
    if rank != 0:
        return
    rows = sample_positions(S_PREFILL, 192)
    for _ in range(args.warmup):
        cpu_prefill_rows(rows[:4], S_PREFILL, 0)
    total, cores = 0.0, 1
    for i in range(args.steps):
        dt, cores = cpu_prefill_rows(rows, S_PREFILL, i)
        total += dt
    value = len(rows) * args.steps / total
    sample = (f"{len(rows)} of the 131072 query rows per step, spread evenly over the sequence (mean causal window 65536 keys), "
              "indexer fp32 + top-k + sparse MLA fp32; input generation outside the clock")
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": total / args.steps * 1e3,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "fp8_e4m3+bf16", "data": "synthetic",
        "config": {"workload": WORKLOAD},
        "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def parity_sample(dev, pipe, inputs, out_full, n=12):
    """A sample of the timed output (rank 0's rows) against the oracle: selection adjudicated in float64
    on the same FP8 values, attention output against the fp32 restatement on the kernel's own selection."""
    from oracle import dsa_oracle as O
    import numpy as np
    q8, k8, ksc, w, q, kv = inputs
    loc = sorted(set(min(pipe.T_loc - 1, (2 * i + 1) * pipe.T_loc // (2 * n)) for i in range(n - 1)) | {pipe.T_loc - 1, 0})
    li = torch.tensor(loc, device=dev)
    pos = pipe.pos[li].cpu()
    ks, ke = torch.zeros(len(loc), dtype=torch.int32), (pos + 1).to(torch.int32)
    idx = pipe.idx[li].cpu()
    q8s = q8.view(torch.uint8)[li].view(FP8).cpu()                  # float8 rows are picked through their bytes
    ref = O.indexer_logits_fp64(q8s, k8.cpu(), ksc.cpu(), w[li].cpu().float(), ks, ke, row_chunk=4).numpy()
    r = O.check_topk_sets(idx.numpy(), ref, ks.numpy(), ke.numpy(), pipe.k, ulp_tol=4.0)
    want = O.sparse_mla(q[li].cpu(), kv.cpu(), idx, SCALE, row_chunk=4)
    got = out_full[pos.long().to(dev)].cpu().float()
    err = (got - want).abs()
    ok = (not r["bad_rows"]) and float(err.max()) <= 2e-2 and float(err.mean()) <= 2e-3
    return {"rows_checked": len(loc), "positions": [int(p) for p in pos], "topk_exact_rows": r["exact_rows"],
            "topk_rows_with_near_tie_swaps": r["swapped_rows"], "topk_rows_over_1ulp": r["rows_over_1ulp"],
            "topk_max_ulp": r["max_ulp"], "topk_bad_rows": len(r["bad_rows"]),
            "out_max_abs_err": float(err.max()), "out_mean_abs_err": float(err.mean()),
            "tolerance": "sets equal to the float64 oracle's except near-ties within 4 fp32 ulps of the k-th score "
                         "(rows over 1 ulp counted); outputs max-abs 2e-2 / mean-abs 2e-3 vs fp32",
            "ok": bool(ok)}


# ---------------------------------------------------------------------------------------------------
# secondary measurements (rank 0, one GPU)
# ---------------------------------------------------------------------------------------------------
def sub_measurements(dev, local, peaks):
    from llmdivedeep_b200 import DSA as dsa_mod, layer, ops
    out = {}
    g = torch.Generator(device=dev).manual_seed(7)
    hbm, bf16_s, bf16_b = peaks["hbm_gbs"], peaks["bf16_tflops_sustained"], peaks["bf16_tflops"]

    # ---- standalone indexer + top-k, 4096 query rows x 65536 keys -------------------------------------
    sets = [make_indexer_inputs(dev, i) for i in range(4)]                 # 168 MB of inputs > L2
    ws = torch.empty(T_ROWS * S_KEYS * 4, dtype=torch.uint8, device=dev)
    logits = ws.view(torch.float32).view(T_ROWS, S_KEYS)
    oi = torch.empty(T_ROWS, TOPK, dtype=torch.int32, device=dev)
    it = [0]

    def both():
        s = sets[it[0] % 4]; it[0] += 1
        ops.indexer_topk(*s, TOPK, workspace=ws, out=oi)

    def only_logits():
        s = sets[it[0] % 4]; it[0] += 1
        ops.fp8_mqa_logits(s[0], (s[1], s[2]), s[3], s[4], s[5], clean_logits=False, out=logits)

    ms_both, ms_lg = _time_ms(both, 20, 5), _time_ms(only_logits, 20, 3)
    ke = sets[0][5]
    ms_tk = _time_ms(lambda: ops.topk_select(logits, TOPK, sets[0][4], ke, out=oi), 20, 3)
    flops = 2.0 * HEADS * DIM * float(ke.sum().item())
    tk_bytes = 4.0 * float(ke.sum().item()) + T_ROWS * TOPK * 4
    sus = _sustained(only_logits, local)
    out["indexer_topk_4096x65536"] = {
        "workload": "4096 query rows (pos 61440-65535) x 65536 keys, 64 heads x 128, fp8 e4m3, k=2048; 4 rotating input sets",
        "ms_per_step": ms_both, "tokens_per_s": T_ROWS / ms_both * 1e3,
        "roofline": {"bound": "tensor", "kernel": "indexer_logits_rw_kernel", "achieved": flops / ms_lg / 1e9,
                     "peak": 2 * bf16_b, "unit": "TFLOP/s", "frac": flops / ms_lg / 1e9 / (2 * bf16_b),
                     "peak_source": "2 x bf16_tflops (burst): fp8 dense = 2 x bf16, no fp8 entry is recorded",
                     "ms_per_launch": ms_lg, "flops_per_launch": flops,
                     "traffic": None, "algorithmic_bytes": 33.5e6 + 8.4e6 + 0.8e6 + 4.0 * float(ke.sum().item()),
                     "sustained": {**sus, "tflops": flops / sus["ms"] / 1e9, "frac_of_2x_bf16_sustained": flops / sus["ms"] / 1e9 / (2 * bf16_s)}},
        "topk": {"ms": ms_tk, "gbs": tk_bytes / ms_tk / 1e6, "frac_of_hbm": tk_bytes / ms_tk / 1e6 / hbm, "algorithmic_bytes": tk_bytes}}
    del sets, ws, logits, oi
    torch.cuda.empty_cache()

    # ---- the reference's published indexer table: square causal, logits + top-k --------------------------
    published = {8192: 1.71, 16384: 5.49, 32768: 19.97}     # sparse_attn/README.md:259-261 (deep_gemm + torch.topk, 1x B200)
    rows = []
    for S in (8192, 16384, 32768):
        q8 = (torch.randn(S, HEADS, DIM, device=dev, generator=g) * 60).to(FP8)
        k8 = (torch.randn(S, DIM, device=dev, generator=g) * 60).to(FP8)
        ksc = torch.rand(S, device=dev, generator=g) * 0.01 + 0.001
        w = torch.randn(S, HEADS, device=dev, generator=g) * 0.01
        ks = torch.zeros(S, dtype=torch.int32, device=dev)
        ke = torch.arange(1, S + 1, dtype=torch.int32, device=dev)
        wsq = torch.empty(ops._lib.load().dsa_indexer_topk_workspace_bytes(S, S), dtype=torch.uint8, device=dev)
        oi = torch.empty(S, min(TOPK, S), dtype=torch.int32, device=dev)
        ms = _time_ms(lambda: ops.indexer_topk(q8, k8, ksc, w, ks, ke, TOPK, workspace=wsq, out=oi), iters=5)
        rows.append({"seq_len": S, "ms": ms, "reference_published_ms": published[S], "speedup": published[S] / ms})
        del q8, k8, ksc, w, wsq, oi
    torch.cuda.empty_cache()
    out["indexer_logits_topk_square_causal"] = {
        "what": "IndexerSimulator.logits_step shape: S queries x S keys, causal, 64 heads x 128, k=2048; the reference's "
                "published numbers are deep_gemm.fp8_mqa_logits + torch.topk on one B200 (its README table)",
        "rows": rows}

    # ---- fused FP8 quantiser ---------------------------------------------------------------------------
    xq = torch.randn(32768, HEADS, DIM, device=dev, dtype=torch.bfloat16, generator=g)        # 537 MB in, 268 MB out
    ms = _time_ms(lambda: ops.fp8_quant_per_block(xq, 128), 10, 2)
    qbytes = xq.numel() * 3.0 + xq.numel() / 128 * 4
    out["fp8_quant_per_block"] = {"workload": "q [32768, 64, 128] bf16 -> e4m3 + one fp32 scale per 128 values", "ms": ms,
                                  "gbs": qbytes / ms / 1e6, "frac_of_hbm": qbytes / ms / 1e6 / hbm,
                                  "reference_published_ms_q_and_k_at_32768": 2.53}
    del xq
    torch.cuda.empty_cache()

    # ---- sparse MLA prefill, 32768 tokens -----------------------------------------------------------------
    T = S = 32768
    q = torch.randn(T, MLA_HEADS, 576, device=dev, dtype=torch.bfloat16, generator=g)
    kv = torch.randn(S, 576, device=dev, dtype=torch.bfloat16, generator=g)
    idx = draw_topk_positions(T, S, TOPK, dev, g)
    o = torch.empty(T, MLA_HEADS, 512, dtype=torch.bfloat16, device=dev)
    fn = lambda: ops.sparse_mla_prefill(q, kv, idx, SCALE, out=o)
    ms = _time_ms(fn, iters=3, warm=1)
    flops = 2.0 * MLA_HEADS * (576 + 512) * float((idx >= 0).sum().item())
    sus = _sustained(fn, local)
    out["sparse_mla_prefill_32768"] = {
        "workload": "32768 tokens x 128 heads, qk 576 / v 512, bf16, 2048 keys per token drawn without replacement from "
                    "[0, t] (all of [0, t] for t < 2047), scale 192**-0.5",
        "ms": ms, "tokens_per_s": T / ms * 1e3,
        "roofline": {"bound": "tensor", "kernel": "sparse_mla_kernel", "achieved": flops / ms / 1e9, "peak": bf16_s,
                     "unit": "TFLOP/s", "frac": flops / ms / 1e9 / bf16_s, "frac_of_burst": flops / ms / 1e9 / bf16_b,
                     "peak_source": "bf16_tflops_sustained (a launch runs for tens of ms under the power cap)",
                     "flops_per_launch": flops, "traffic": None,
                     "algorithmic_bytes": 4.83e9 + 4.29e9 + 37.7e6 + 268e6, "l2_gather_bytes": float((idx >= 0).sum().item()) * 1152,
                     "sustained": {**sus, "tflops": flops / sus["ms"] / 1e9}}}
    del q, kv, idx, o
    torch.cuda.empty_cache()

    # ---- block-sparse MHA: the reference's register_sparse_fa().run shape ------------------------------
    build_lut, run = dsa_mod.register_sparse_fa()
    rows_bs = []
    for S_bs, ref_ms in ((8192, 0.12), (16384, 0.36), (32768, 1.23)):
        qb_, kb_, vb_ = (torch.randn(1, S_bs, 24, 128, device=dev, dtype=torch.bfloat16, generator=g) for _ in range(3))
        lut, num, topk_b = build_lut(qb_, S_bs, 0.05)
        ms = _time_ms(lambda: run(qb_, kb_, vb_, lut, num, 128 ** -0.5), iters=10)
        rows_bs.append({"seq_len": S_bs, "key_blocks_per_query_block": topk_b, "ms": ms,
                        "tflops": 4.0 * 24 * S_bs * topk_b * 64 * 128 / ms / 1e9,
                        "reference_published_ms": ref_ms, "speedup": ref_ms / ms})
        del qb_, kb_, vb_, lut, num
    out["block_sparse_mha"] = {
        "what": "[1, S, 24, 128] bf16, 64-token blocks, 5 % of the key blocks per query block, non-causal: the shape of "
                "the reference's block-sparse stand-in (its README table, one B200, an external Triton kernel)",
        "rows": rows_bs}
    torch.cuda.empty_cache()

    # ---- one decode step: batch 64, context 131072 ---------------------------------------------------------
    B, CTX = 64, 131072
    q8, w, kcache, kscale, table, ctx, qd, latent = make_decode_inputs(dev, B, CTX, g)
    dws = layer.DecodeWorkspace(B, MLA_HEADS, CTX, TOPK, dev)
    step = lambda: layer.dsa_decode_step(q8, w, kcache, kscale, table, ctx, qd, latent, SCALE, dws)
    t_all = _time_ms(step, iters=10)
    t_idx = _time_ms(lambda: ops.fp8_paged_mqa_logits(q8, w, kcache, kscale, table, ctx, CTX, out=dws.logits), iters=10)
    t_top = _time_ms(lambda: ops.topk_select(dws.logits, TOPK, None, ctx, out=dws.idx), iters=10)
    t_mla = _time_ms(lambda: ops.sparse_mla_decode_paged(qd, latent, table, dws.idx, SCALE, CTX, out=dws.out, workspace=dws.mla_ws), iters=10)
    ops.check_status(dev)
    scan_bytes, gather_bytes = B * CTX * 132.0, B * TOPK * 656.0
    step_bytes = scan_bytes + 2 * B * CTX * 4 + gather_bytes
    sus = _sustained(step, local)
    out["decode_step_b64_ctx131072"] = {
        "workload": "batch 64, context 131072, one new token each, 64-token pages in random order, FP8 e4m3 caches quantised "
                    "from N(0,1) (indexer keys + per-token scale; latent 512 e4m3 + 4 scales + 64 bf16 rope), 64 indexer "
                    "heads, top-k 2048, 128 heads",
        "us_per_step": t_all * 1e3, "indexer_us": t_idx * 1e3, "topk_us": t_top * 1e3, "sparse_mla_us": t_mla * 1e3,
        "roofline": {"bound": "hbm", "kernel": "indexer_logits_kernel (paged scan) + topk_select_kernel + sparse_mla_kernel<paged fp8>",
                     "achieved": step_bytes / t_all / 1e6, "peak": hbm, "unit": "GB/s", "frac": step_bytes / t_all / 1e6 / hbm,
                     "algorithmic_bytes": step_bytes, "traffic": None,
                     "indexer_scan": {"achieved": scan_bytes / t_idx / 1e6, "frac": scan_bytes / t_idx / 1e6 / hbm},
                     "sparse_mla_gather": {"achieved": gather_bytes / t_mla / 1e6, "frac": gather_bytes / t_mla / 1e6 / hbm,
                                           "tflops": 2.0 * B * MLA_HEADS * TOPK * 1088 / t_mla / 1e9},
                     "lower_bound_us": step_bytes / hbm / 1e3,
                     "sustained": {"us_per_step": sus["ms"] * 1e3, "iters": sus["iters"], "sm_mhz_median": sus["sm_mhz_median"],
                                   "reasons": sus["reasons"]}}}
    return out


def incumbent_measurement():
    """deep_gemm.fp8_mqa_logits (the kernel the reference calls when it is installed, sparse_attn/DSA.py:87-95,
    343-345) + torch.topk on this box, as a library call in a child process with a time limit: its JIT may be
    unable to build here."""
    code = r'''
import json, sys, torch
try:
    from vllm.third_party import deep_gemm as dg
    fn = dg.fp8_mqa_logits
except Exception as e:
    print(json.dumps({"unavailable": f"import failed: {type(e).__name__}: {e}"[:300]})); sys.exit(0)
rows = []
g = torch.Generator(device="cuda").manual_seed(7)
try:
    for S in (8192, 16384, 32768):
        q8 = (torch.randn(S, 64, 128, device="cuda", generator=g) * 60).to(torch.float8_e4m3fn)
        k8 = (torch.randn(S, 128, device="cuda", generator=g) * 60).to(torch.float8_e4m3fn)
        ksc = torch.rand(S, device="cuda", generator=g) * 0.01 + 0.001
        w = torch.randn(S, 64, device="cuda", generator=g) * 0.01
        ks = torch.zeros(S, dtype=torch.int32, device="cuda"); ke = torch.arange(1, S + 1, dtype=torch.int32, device="cuda")
        f = lambda: fn(q8, (k8, ksc), w, ks, ke).topk(2048, dim=-1).indices
        for _ in range(2): f()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(5): f()
        e1.record(); torch.cuda.synchronize()
        rows.append({"seq_len": S, "incumbent_ms": e0.elapsed_time(e1) / 5})
    print(json.dumps({"rows": rows}))
except Exception as e:
    print(json.dumps({"unavailable": f"call failed: {type(e).__name__}: {e}"[:300], "rows": rows}))
'''
    try:
        p = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=240)
        lines = [l for l in p.stdout.splitlines() if l.startswith("{")]
        return json.loads(lines[-1]) if lines else {"unavailable": f"no output (rc {p.returncode}): {p.stderr[-200:]}"}
    except subprocess.TimeoutExpired:
        return {"unavailable": "timed out after 240 s (JIT build of the library kernel did not finish)"}
    except Exception as e:                                             # noqa: BLE001
        return {"unavailable": f"{type(e).__name__}: {e}"[:300]}


# ---------------------------------------------------------------------------------------------------
# multi-GPU extras
# ---------------------------------------------------------------------------------------------------
def decode_sharded_measurement(dev, rank, world, steps=10):
    """Decode at a TOTAL batch of 512 sequences (context 131072) split over the ranks by batch; every step's
    attention output (batch x 128 x 512 bf16) is all-gathered on a side stream under the next step's scan."""
    import torch.distributed as dist
    from llmdivedeep_b200 import layer, sharding as sh
    B_total, CTX = 512, 131072
    a, b = sh.batch_range(B_total, world, rank)
    B = b - a
    g = torch.Generator(device=dev).manual_seed(100 + rank)
    q8, w, kcache, kscale, table, ctx, qd, latent = make_decode_inputs(dev, B, CTX, g)
    dws = [layer.DecodeWorkspace(B, MLA_HEADS, CTX, TOPK, dev) for _ in range(2)]
    full = torch.empty(B_total, MLA_HEADS, 512, dtype=torch.bfloat16, device=dev)
    comm = torch.cuda.Stream(device=dev)
    main = torch.cuda.current_stream(dev)
    gathered = [None, None]

    def run(n):
        for i in range(n):
            s = i & 1
            if gathered[s] is not None:
                main.wait_event(gathered[s])
            _, o = layer.dsa_decode_step(q8, w, kcache, kscale, table, ctx, qd, latent, SCALE, dws[s])
            if world > 1:
                ev = torch.cuda.Event(); ev.record(main)
                with torch.cuda.stream(comm):
                    comm.wait_event(ev)
                    dist.all_gather_into_tensor(full, o)
                    gathered[s] = torch.cuda.Event(); gathered[s].record(comm)
        main.wait_stream(comm)

    run(3)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(); run(steps); e1.record()
    torch.cuda.synchronize()
    ms = torch.tensor([e0.elapsed_time(e1) / steps], device=dev)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    del q8, w, kcache, kscale, table, ctx, qd, latent, dws, full
    torch.cuda.empty_cache()
    return {"workload": "decode, total batch 512 at context 131072 split over the ranks by batch, output all-gathered "
                        "(67 MB) on a side stream under the next step", "n_gpus": world, "batch_per_gpu": B,
            "us_per_step": float(ms.item()) * 1e3, "sequences_per_s": B_total / float(ms.item()) * 1e3}


def head_vs_row_measurement(dev, rank, world):
    """Sparse MLA prefill of one 8192-token stretch split over the ranks by heads (128 / world per rank, the
    layout that needs every rank to gather every row) against the row split, both with the NCCL all-gather."""
    import torch.distributed as dist
    from llmdivedeep_b200 import ops, sharding as sh
    T, S, H, K = 8192, 32768, 128, TOPK
    g = torch.Generator(device=dev).manual_seed(11)               # same tensors on every rank
    q = torch.randn(T, H, 576, device=dev, dtype=torch.bfloat16, generator=g)
    kv = torch.randn(S, 576, device=dev, dtype=torch.bfloat16, generator=g)
    idx = (torch.rand(T, K, device=dev, generator=g) * S).int()
    rows = sh.rows_of(sh.row_chunks(T, world, rank, 256), device=dev)
    q_rows, idx_rows = q[rows].contiguous(), idx[rows].contiguous()
    h0, h1 = sh.head_range(H, world, rank)
    q_heads = q[:, h0:h1].contiguous()
    res = {}
    for name, fn in (("rows", lambda: sh.all_gather_rows(ops.sparse_mla_prefill(q_rows, kv, idx_rows, SCALE), T, world, 256)),
                     ("heads", lambda: sh.all_gather_heads(ops.sparse_mla_prefill(q_heads, kv, idx, SCALE), H, world))):
        ms = torch.tensor([_time_ms(fn, iters=3, warm=1)], device=dev)
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        res[name + "_ms"] = float(ms.item())
    res.update({"n_gpus": world, "workload": "8192 tokens x 128 heads x 2048 selected keys, bf16; one blocking all-gather after "
                                             "the kernel (the head split cannot overlap it: every rank needs all rows first)"})
    return res


# ---------------------------------------------------------------------------------------------------
# profiler cases
# ---------------------------------------------------------------------------------------------------
def run_profile_case(args):
    """Reduced cases sized for a profiler capture (inputs larger than L2, a few hundred MB on the device)."""
    from llmdivedeep_b200 import DSA as dsa_mod, layer, ops
    dev = torch.device("cuda", 0)
    g = torch.Generator(device=dev).manual_seed(3)
    it, warm = max(1, args.steps), args.warmup
    if args.case == "indexer_small":
        rows = 512
        sets = [make_indexer_inputs(dev, i, rows) for i in range(2)]
        ws = torch.empty(rows * S_KEYS * 4, dtype=torch.uint8, device=dev)
        oi = torch.empty(rows, TOPK, dtype=torch.int32, device=dev)
        ms = _time_ms(lambda: ops.indexer_topk(*sets[0], TOPK, workspace=ws, out=oi), it, warm)
        info = {"rows": rows, "keys": S_KEYS, "ms": ms}
    elif args.case == "mla_prefill_small":
        T, S = 512, 32768
        q = torch.randn(T, MLA_HEADS, 576, device=dev, dtype=torch.bfloat16, generator=g)
        kv = torch.randn(S, 576, device=dev, dtype=torch.bfloat16, generator=g)
        idx = (torch.rand(T, TOPK, device=dev, generator=g) * S).int()
        o = torch.empty(T, MLA_HEADS, 512, dtype=torch.bfloat16, device=dev)
        ms = _time_ms(lambda: ops.sparse_mla_prefill(q, kv, idx, SCALE, out=o), it, warm)
        info = {"tokens": T, "ms": ms, "tflops_algorithmic": 2.0 * MLA_HEADS * 1088 * T * TOPK / ms / 1e9}
    elif args.case == "block_sparse_small":
        S = 8192
        q, k, v = (torch.randn(1, S, 24, 128, device=dev, dtype=torch.bfloat16, generator=g) for _ in range(3))
        build_lut, run = dsa_mod.register_sparse_fa()
        lut, num, topk_b = build_lut(q, S, 0.05)
        ms = _time_ms(lambda: run(q, k, v, lut, num, 128 ** -0.5), it, warm)
        info = {"seq_len": S, "key_blocks_per_query_block": topk_b, "ms": ms}
    else:                                                        # decode_small
        B, CTX = 8, 131072
        q8, w, kcache, kscale, table, ctx, qd, latent = make_decode_inputs(dev, B, CTX, g)
        dws = layer.DecodeWorkspace(B, MLA_HEADS, CTX, TOPK, dev)
        ms = _time_ms(lambda: layer.dsa_decode_step(q8, w, kcache, kscale, table, ctx, qd, latent, SCALE, dws), it, warm)
        info = {"batch": B, "context": CTX, "us_per_step": ms * 1e3}
    ops.check_status(dev)
    print(json.dumps({"profile_case": args.case, "not_a_bench_value": True, **info}))


# ---------------------------------------------------------------------------------------------------
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extra", action="store_true", help="skip the sub-records and the incumbent comparison")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer leg (profiling runs)")
    ap.add_argument("--gather", choices=("peer", "nccl"), default="peer",
                    help="N > 1: how the ranks exchange the attention output (copies into symmetric memory, or NCCL all-gather)")
    ap.add_argument("--chunk-rows", type=int, default=0, help="query rows per pipeline chunk (default: 4096 on one GPU, 2048 on several)")
    ap.add_argument("--seq", type=int, default=S_PREFILL,
                    help="prefill length; anything but 131072 is a reduced case for profiler captures, not a bench value")
    ap.add_argument("--case", default="headline",
                    choices=["headline", "indexer_small", "mla_prefill_small", "decode_small", "block_sparse_small"],
                    help="anything but 'headline' runs a few launches of a reduced case for profiler captures and prints a "
                         "line marked as such, not a bench value")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank)
        return
    if args.case != "headline":
        run_profile_case(args)
        return
    args.warmup = max(args.warmup, 3)
    S = args.seq
    workload = WORKLOAD if S == S_PREFILL else f"REDUCED profiling case (seq {S}) of: " + WORKLOAD

    from llmdivedeep_b200 import layer, ops
    import torch.distributed as dist
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        # NCCL prints its version banner on stdout when the first communicator is created; stdout must carry
        # the JSON line only, so file descriptor 1 points at stderr until that has happened
        sys.stdout.flush()
        saved = os.dup(1)
        os.dup2(2, 1)
        try:
            opts = dist.ProcessGroupNCCL.Options(is_high_priority_stream=True)     # see layer.PrefillPipeline: the gathers overlap compute
            dist.init_process_group("nccl", device_id=dev, pg_options=opts)
            dist.barrier()
            torch.cuda.synchronize()
        finally:
            os.dup2(saved, 1)
            os.close(saved)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms):
        t = torch.tensor([ms], device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    chunk_rows = args.chunk_rows or (4096 if world == 1 else 2048)
    # Output exchange between the ranks: plain copies into symmetric memory (copy engines, no SMs) unless --gather nccl;
    # if symmetric memory cannot be set up on any rank, every rank falls back to the NCCL all-gather.
    transport = "peer" if (world > 1 and args.gather == "peer") else "nccl"
    pipe = out_full = None
    while out_full is None:
        pipe = layer.PrefillPipeline(S, dev, n_heads=MLA_HEADS, topk=TOPK, chunk_rows=chunk_rows, softmax_scale=SCALE,
                                     rank=rank, world=world, block_rows=BLOCK_ROWS, transport=transport)
        try:
            out_full, made = pipe.output_buffer(), 1
        except Exception as exc:                               # noqa: BLE001 - reported below, then the NCCL path
            made = 0
            print(f"rank {rank}: symmetric memory unavailable ({exc!r}); output exchange by NCCL all-gather", file=sys.stderr)
        if world > 1:
            agreed = torch.tensor([made], device=dev)
            dist.all_reduce(agreed, op=dist.ReduceOp.MIN)
            if int(agreed.item()) == 0:
                if transport == "nccl":
                    raise RuntimeError("no output buffer could be allocated")
                out_full, transport = None, "nccl"
    inputs = make_prefill_inputs(dev, 0, S, pipe.pos)
    q8, k8, ksc, w, q, kv = inputs

    # ---- device-resident throughput -----------------------------------------------------------------
    for _ in range(args.warmup):
        pipe.run(q8, k8, ksc, w, q, kv, out_full)
    barrier()
    sampler = ClockSampler(local).start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        pipe.run(q8, k8, ksc, w, q, kv, out_full)
    e1.record()
    barrier()
    clocks = sampler.stop()
    total_ms = max_over_ranks(e0.elapsed_time(e1))
    ops.check_status(dev)

    # ---- per-kernel times over the whole sequence (this rank's rows), for the roofline ---------------------
    def stage_ms(fn):
        for _ in range(1):
            for c in range(len(pipe.chunks)):
                fn(c)
        torch.cuda.synchronize()
        a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a0.record()
        for c in range(len(pipe.chunks)):
            fn(c)
        a1.record()
        torch.cuda.synchronize()
        return a0.elapsed_time(a1)

    lg = pipe.ws.view(torch.float32)
    ld = (S + 3) // 4 * 4

    def f_idx(c):
        a, b, _, _ = pipe.chunks[c]
        ops.fp8_mqa_logits(q8[a:b], (k8, ksc), w[a:b], pipe.ks[a:b], pipe.ke[a:b], clean_logits=False,
                           out=lg[: (b - a) * ld].view(b - a, ld))

    def f_topk(c):
        a, b, _, _ = pipe.chunks[c]
        ops.topk_select(lg[: (b - a) * ld].view(b - a, ld)[:, :S], pipe.k, pipe.ks[a:b], pipe.ke[a:b], out=pipe.idx[a:b])

    scratch = torch.empty(pipe.rows_max, MLA_HEADS, 512, dtype=torch.bfloat16, device=dev)

    def f_mla(c):
        a, b, _, _ = pipe.chunks[c]
        ops.sparse_mla_prefill(q[a:b], kv, pipe.idx[a:b], SCALE, out=scratch[: b - a])

    ms_idx, ms_topk, ms_mla = stage_ms(f_idx), stage_ms(f_topk), stage_ms(f_mla)
    del scratch
    peaks, peak_kind = measured_peaks()
    my_keys = float(pipe.ke.sum().item())
    my_pairs = float((pipe.idx >= 0).sum().item())
    flops_idx, flops_mla = 2.0 * HEADS * DIM * my_keys, 2.0 * MLA_HEADS * 1088 * my_pairs
    roof_idx = {"bound": "tensor", "kernel": "indexer_logits_rw_kernel (fp8 e4m3, 64 heads x 128)",
                "achieved": flops_idx / ms_idx / 1e9, "peak": 2 * peaks["bf16_tflops_sustained"], "unit": "TFLOP/s",
                "frac": flops_idx / ms_idx / 1e9 / (2 * peaks["bf16_tflops_sustained"]),
                "frac_of_2x_bf16_burst": flops_idx / ms_idx / 1e9 / (2 * peaks["bf16_tflops"]),
                "peak_source": f"2 x bf16_tflops_sustained of {peak_kind} peaks (fp8 dense = 2 x bf16; no fp8 entry is recorded; "
                               "the launches of one step run back to back for tens of ms)",
                "ms_all_launches": ms_idx, "launches": len(pipe.chunks), "flops_all_launches": flops_idx,
                "ms_per_launch": ms_idx / max(1, len(pipe.chunks)), "flops_per_launch": flops_idx / max(1, len(pipe.chunks)),
                # traffic: the reduced case's logits partly stay in L2, so its DRAM bytes do not scale to a full launch
                "traffic": None, "algorithmic_bytes": 4.0 * my_keys + pipe.T_loc * (HEADS * DIM + HEADS * 2) + S * 132.0}
    roof_mla = {"bound": "tensor", "kernel": "sparse_mla_kernel (bf16, 128 heads, qk 576 / v 512)",
                "achieved": flops_mla / ms_mla / 1e9, "peak": peaks["bf16_tflops_sustained"], "unit": "TFLOP/s",
                "frac": flops_mla / ms_mla / 1e9 / peaks["bf16_tflops_sustained"],
                "frac_of_bf16_burst": flops_mla / ms_mla / 1e9 / peaks["bf16_tflops"],
                "peak_source": f"bf16_tflops_sustained of {peak_kind} peaks (the launches of one step run back to back for "
                               "tens of ms)",
                "ms_all_launches": ms_mla, "launches": len(pipe.chunks), "flops_all_launches": flops_mla,
                "ms_per_launch": ms_mla / max(1, len(pipe.chunks)), "flops_per_launch": flops_mla / max(1, len(pipe.chunks)),
                # dram__bytes_read + dram__bytes_write of one ncu capture of the 512-token reduced case (125.3 MB + 49.0 MB),
                # scaled by the tokens of one launch: q, idx and the output grow with the tokens, the latent KV does not
                "traffic": (129.19e6 + 49.12e6) * (pipe.T_loc / max(1, len(pipe.chunks))) / 512,
                "traffic_source": "ncu capture of bench.py --case mla_prefill_small (512 tokens), scaled by tokens per launch",
                "algorithmic_bytes": pipe.T_loc * MLA_HEADS * (576 + 512) * 2.0 + S * 1152.0 + pipe.T_loc * TOPK * 4.0,
                "algorithmic_bytes_per_launch": (pipe.T_loc * (MLA_HEADS * (576 + 512) * 2.0 + TOPK * 4.0)) / max(1, len(pipe.chunks)) + S * 1152.0,
                "l2_gather_bytes": my_pairs * 1152.0}
    tk_bytes = 4.0 * my_keys + pipe.T_loc * TOPK * 4.0
    roof_topk = {"bound": "hbm", "kernel": "topk_select_kernel", "achieved": tk_bytes / ms_topk / 1e6, "peak": peaks["hbm_gbs"],
                 "unit": "GB/s", "frac": tk_bytes / ms_topk / 1e6 / peaks["hbm_gbs"], "ms_all_launches": ms_topk,
                 "algorithmic_bytes": tk_bytes, "traffic": None}
    dominant = roof_mla if ms_mla >= ms_idx else roof_idx

    # ---- end to end: pinned host inputs -> device, attention output -> pinned host ----------------------
    e2e = None
    if not args.no_e2e:
        pipe.run(q8, k8, ksc, w, q, kv, out_full)
        torch.cuda.synchronize()
        host = [t.cpu().pin_memory() for t in inputs]
        out_h = torch.empty(pipe.T_loc, MLA_HEADS, 512, dtype=torch.bfloat16).pin_memory()
        want_rows = out_full[pipe.pos.long()[-BLOCK_ROWS:]].clone()
        h2d = sum(t.numel() * t.element_size() for t in host)
        d2h = out_h.numel() * 2
        del q8, w, q, inputs                                 # the device-resident copies of the per-row inputs
        torch.cuda.empty_cache()
        hp = layer.HostPrefillPipeline(pipe, HEADS, DIM, torch.bfloat16)
        submit = lambda: hp.submit(host[0], host[1], host[2], host[3], host[4], host[5], out_h, out_full)
        for _ in range(2):
            done = submit()
        done.synchronize()
        barrier()
        same = bool(torch.equal(out_h[-BLOCK_ROWS:].to(dev), want_rows))
        e0.record()
        for _ in range(args.steps):
            done = submit()
        torch.cuda.current_stream().wait_event(done)          # the last step's output is in host memory
        e1.record()
        barrier()
        e2e_ms = max_over_ranks(e0.elapsed_time(e1))
        if not same:
            raise RuntimeError("the host-buffer pipeline returned an output that differs from the device-resident run")
        e2e = {"value": S * args.steps / (e2e_ms * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": h2d * world,
               "d2h_bytes_per_step": d2h * world, "ms_per_step": e2e_ms / args.steps,
               "h2d_gbs_per_rank": h2d / (e2e_ms / args.steps) / 1e6, "d2h_gbs_per_rank": d2h / (e2e_ms / args.steps) / 1e6,
               "how": "layer.HostPrefillPipeline.submit per step: every input (q_idx fp8, head weights, keys, MLA q, latent KV) "
                      "copied from pinned host memory and this rank's attention output rows copied back, chunk by chunk on two "
                      "copy streams under the kernels; bytes are summed over the ranks; the timed region ends after the last "
                      "device -> host copy.  PCIe moves about 37.7 GB per step in total, which bounds this leg, not the kernels"}
        q8, k8, ksc, w, q, kv = (t.to(dev) for t in host)     # back on the device for the parity sample
        inputs = (q8, k8, ksc, w, q, kv)
        del hp, host, out_h
    # the per-kernel loops above reuse the pipeline's index and logit buffers: one more whole step for the parity sample
    pipe.run(q8, k8, ksc, w, q, kv, out_full)
    torch.cuda.synchronize()

    extras = {}
    if world > 1 and not args.no_extra and S == S_PREFILL:
        del out_full
        torch.cuda.empty_cache()
        extras["decode_sharded"] = decode_sharded_measurement(dev, rank, world)
        extras["sparse_mla_head_vs_row_split"] = head_vs_row_measurement(dev, rank, world)
        out_full = None
    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    line = {
        "metric": METRIC, "value": S * args.steps / (total_ms * 1e-3), "unit": "tokens/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": total_ms / args.steps,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "fp8_e4m3+bf16", "data": "synthetic",
        "config": {"workload": workload,
                   "l2": "inputs of one step are 20 GB (MLA q 19.3 GB, indexer q 1.07 GB) and the output 17.2 GB: far larger than the 126 MB L2",
                   "chunk_rows": chunk_rows,
                   "sharding": ("one sequence; 256-row blocks of query rows dealt round-robin over the ranks, keys and latent KV "
                                "replicated; " + ("every finished block copied into every rank's output (symmetric memory) by "
                                                  "device-to-device copies on a side stream, two 4-byte all-reduces per step"
                                                  if pipe.transport == "peer" else
                                                  "output all-gathered per finished chunk on a side stream (NCCL), one collective "
                                                  "per round of blocks straight into row order")) if world > 1 else "one GPU, no collective",
                   "output_exchange": pipe.transport if world > 1 else None},
        "gpu_launches": pipe.launches_per_run * args.steps,
        "clocks": clocks,
        "roofline": dominant,
        "kernels": {"indexer": roof_idx, "topk": roof_topk, "sparse_mla": roof_mla,
                    "share_of_step": {"indexer": ms_idx / (ms_idx + ms_topk + ms_mla), "topk": ms_topk / (ms_idx + ms_topk + ms_mla),
                                      "sparse_mla": ms_mla / (ms_idx + ms_topk + ms_mla)}},
    }
    if e2e is not None:
        line["e2e"] = e2e
    if out_full is not None and S == S_PREFILL:
        line["parity"] = parity_sample(dev, pipe, inputs, out_full)
    if extras:
        line["extra"] = extras
    if not args.no_extra and world == 1 and S == S_PREFILL:
        del out_full, inputs, q8, k8, ksc, w, q, kv
        pipe = None
        torch.cuda.empty_cache()
        line["sub"] = sub_measurements(dev, local, peaks)
        line["sub"]["decode_sharded_b512"] = decode_sharded_measurement(dev, 0, 1, steps=5)
        torch.cuda.empty_cache()
        inc = incumbent_measurement()
        tab = line["sub"]["indexer_logits_topk_square_causal"]
        if "rows" in inc:
            by = {r["seq_len"]: r["incumbent_ms"] for r in inc["rows"]}
            for r in tab["rows"]:
                if r["seq_len"] in by:
                    r["incumbent_ms"] = by[r["seq_len"]]
                    r["speedup_vs_incumbent_same_box"] = by[r["seq_len"]] / r["ms"]
        if "unavailable" in inc:
            tab["incumbent_unavailable"] = inc["unavailable"]
        tab["incumbent"] = "vllm.third_party.deep_gemm.fp8_mqa_logits + torch.topk, same box, child process"
    if not args.no_cpu_baseline and world == 1 and S == S_PREFILL:
        rows = sample_positions(S, 1536)                      # about 12 s of CPU work on 16 cores
        cpu_prefill_rows(rows[:4], S, 1)
        secs, cores = cpu_prefill_rows(rows, S, 0)
        line["cpu_baseline"] = {"value": len(rows) / secs, "unit": "tokens/s", "cores": cores, "kind": "port",
                                "sample": f"{len(rows)} of the 131072 query rows, spread evenly over the sequence (mean causal window "
                                          f"65536 keys), {secs:.1f} s; CPU oracle port: fp32 fallback scorer + ReLU (row-chunked) + "
                                          "torch.topk + fp32 sparse MLA; scaled linearly to tokens/s"}
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
