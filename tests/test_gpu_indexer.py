"""dsa_indexer_logits / dsa_indexer_topk (through the C ABI) against the CPU oracle.

Tolerances.  Logits are fp32 sums of 64 fp32-accumulated FP8 dot products; the
kernel applies k_scale after the head sum and sums heads in a fixed order that
differs from torch.sum's, so it is compared with the float64 oracle within
4e-6 of the largest |logit| in the case (the fp32 oracle itself sits ~1e-6 from
float64).  Top-k sets must equal the float64 oracle's except for swaps of
elements whose exact scores lie within TOPK_ULP_TOL fp32 ulps of the k-th score:
a 64-term fp32 sum of mixed-sign terms carries a few ulps of rounding noise
whatever its order (the fp32 CPU oracle shows swaps of the same size against
float64), so a 1-ulp bound holds for most rows but not for every row; measured
worst case on these seeds is 2.0 ulp.
"""
import os

import numpy as np
import pytest
import torch

from llmdivedeep_b200 import ops
from oracle import dsa_oracle as O
from tests.helpers import indexer_inputs, to_dev

pytestmark = pytest.mark.gpu
REL_TOL = 4e-6
TOPK_ULP_TOL = 4.0
G = np.load(os.path.join(os.path.dirname(__file__), "golden", "reference_golden.npz"))


def _check_logits(args, out, clean=True):
    q8, k8, ksc, w, ks, ke = args
    ref = O.indexer_logits_fp64(q8, k8, ksc, w.float(), ks, ke)
    o = out.cpu().double()
    fin = torch.isfinite(ref)
    if clean:
        assert torch.equal(torch.isfinite(o), fin), "window mask differs"
        assert bool((o[~fin] == float("-inf")).all())
    err = (o[fin] - ref[fin]).abs().max()
    assert float(err) <= REL_TOL * float(ref[fin].abs().max()), float(err)


@pytest.mark.parametrize("T,S,H,D,window", [
    (64, 1000, 64, 128, "random"), (300, 4133, 64, 128, "causal"), (128, 2048, 4, 64, "causal"),
    (256, 8192, 64, 128, "causal"), (100, 3000, 16, 128, "random"), (7, 129, 64, 128, "full"),
    (33, 640, 8, 128, "causal"), (50, 700, 32, 128, "random"), (40, 512, 64, 64, "full"), (1, 128, 64, 128, "full"),
])
def test_logits_match_oracle(T, S, H, D, window):
    args = indexer_inputs(T, S, H, D, seed=T * 7 + S, window=window)
    out = ops.fp8_mqa_logits(args[0].cuda(), (args[1].cuda(), args[2].cuda()), args[3].cuda(),
                             args[4].cuda(), args[5].cuda())
    ops.check_status("cuda")
    _check_logits(args, out)


def test_golden_simulator_inputs():
    """The recorded FP8 cache of the reference's IndexerSimulator (H=4, D=128, S=192)."""
    q8 = torch.from_numpy(G["sim_q_fp8"].copy()).view(torch.float8_e4m3fn)
    k8 = torch.from_numpy(G["sim_k_fp8"].copy()).view(torch.float8_e4m3fn)
    ksc, w = torch.from_numpy(G["sim_k_scale"]), torch.from_numpy(G["sim_w"])
    S = k8.shape[0]
    ks, ke = torch.zeros(S, dtype=torch.int32), torch.arange(1, S + 1, dtype=torch.int32)
    out = ops.fp8_mqa_logits(q8.cuda(), (k8.cuda(), ksc.cuda()), w.cuda(), ks.cuda(), ke.cuda())
    _check_logits((q8, k8, ksc, w, ks, ke), out)
    idx = ops.indexer_topk(q8.cuda(), k8.cuda(), ksc.cuda(), w.cuda(), ks.cuda(), ke.cuda(), 16)
    ref = O.indexer_logits_fp64(q8, k8, ksc, w, ks, ke).numpy()
    r = O.check_topk_sets(idx.cpu().numpy(), ref, ks.numpy(), ke.numpy(), 16, ulp_tol=TOPK_ULP_TOL)
    assert not r["bad_rows"], r


def test_bf16_weights_and_null_ks():
    args = indexer_inputs(96, 1500, 64, 128, seed=3, window="causal", w_bf16=True)
    q8, k8, ksc, w, ks, ke = args
    out = ops.fp8_mqa_logits(q8.cuda(), (k8.cuda(), ksc.cuda()), w.cuda(), None, ke.cuda())
    _check_logits(args, out)


def test_unclean_logits_leave_masked_tiles_untouched():
    T, S = 8, 2048
    q8, k8, ksc, w, ks, ke = indexer_inputs(T, S, 64, 128, seed=11, window="full")
    ks[:] = 600
    ke[:] = 700                                       # tiles 4..5 of 16
    out = torch.full((T, S), 123.0, device="cuda")
    ops.fp8_mqa_logits(q8.cuda(), (k8.cuda(), ksc.cuda()), w.cuda(), ks.cuda(), ke.cuda(),
                       clean_logits=False, out=out)
    o = out.cpu()
    assert bool((o[:, :512] == 123.0).all()) and bool((o[:, 768:] == 123.0).all())
    assert bool(torch.isinf(o[:, 512:600]).all()) and bool(torch.isfinite(o[:, 600:700]).all())
    out2 = ops.fp8_mqa_logits(q8.cuda(), (k8.cuda(), ksc.cuda()), w.cuda(), ks.cuda(), ke.cuda(),
                              clean_logits=True)
    _check_logits((q8, k8, ksc, w, ks, ke), out2)


def test_empty_windows_and_zero_rows():
    q8, k8, ksc, w, ks, ke = indexer_inputs(16, 512, 64, 128, seed=2, window="full")
    ke[3] = 0
    ks[5] = 512
    out = ops.fp8_mqa_logits(q8.cuda(), (k8.cuda(), ksc.cuda()), w.cuda(), ks.cuda(), ke.cuda())
    _check_logits((q8, k8, ksc, w, ks, ke), out)
    empty = ops.fp8_mqa_logits(q8[:0].cuda(), (k8.cuda(), ksc.cuda()), w[:0].cuda(), ks[:0].cuda(), ke[:0].cuda())
    assert empty.shape == (0, 512)


def test_unsupported_head_count_is_refused():
    q8, k8, ksc, w, ks, ke = indexer_inputs(4, 128, 12, 128, seed=1, window="full")
    with pytest.raises(ops.DsaError, match="unsupported"):
        ops.fp8_mqa_logits(q8.cuda(), (k8.cuda(), ksc.cuda()), w.cuda(), ks.cuda(), ke.cuda())


@pytest.mark.parametrize("T,S,K,window", [(256, 16384, 2048, "causal"), (300, 5000, 512, "random"),
                                          (64, 1024, 2048, "causal")])
def test_indexer_topk_sets_match_oracle(T, S, K, window):
    args = indexer_inputs(T, S, 64, 128, seed=S + K, window=window)
    q8, k8, ksc, w, ks, ke = args
    idx = ops.indexer_topk(*to_dev(*args), K)
    ops.check_status("cuda")
    assert idx.shape == (T, min(K, S)) and idx.dtype == torch.int32
    ref = O.indexer_logits_fp64(q8, k8, ksc, w, ks, ke).numpy()
    r = O.check_topk_sets(idx.cpu().numpy(), ref, ks.numpy(), ke.numpy(), min(K, S), ulp_tol=TOPK_ULP_TOL)
    assert not r["bad_rows"], r
    assert torch.equal(idx, ops.indexer_topk(*to_dev(*args), K)), "not deterministic"


def test_indexer_topk_small_workspace_chunks_rows():
    args = indexer_inputs(600, 2048, 64, 128, seed=8, window="causal")
    dev = to_dev(*args)
    full = ops.indexer_topk(*dev, 256)
    ws = torch.empty(256 * 2048 * 4, dtype=torch.uint8, device="cuda")      # one 256-row chunk
    assert torch.equal(full, ops.indexer_topk(*dev, 256, workspace=ws))
    with pytest.raises(ops.DsaError, match="workspace"):
        ops.indexer_topk(*dev, 256, workspace=ws[: 100 * 2048 * 4])


def test_full_size_linearity_property():
    """Bench-size keys (S = 65536): scores are linear in the head weights, so
    logits(w1) + logits(w2) == logits(w1 + w2) up to fp32 rounding, and doubling
    k_scale doubles every score exactly."""
    T, S = 64, 65536
    q8, k8, ksc, w, ks, ke = to_dev(*indexer_inputs(T, S, 64, 128, seed=4, window="causal"))
    w2 = torch.randn_like(w) * w.abs().mean()
    a = ops.fp8_mqa_logits(q8, (k8, ksc), w, ks, ke).clone()
    b = ops.fp8_mqa_logits(q8, (k8, ksc), w2, ks, ke).clone()
    c = ops.fp8_mqa_logits(q8, (k8, ksc), w + w2, ks, ke).clone()
    fin = torch.isfinite(a)
    assert float(((a + b)[fin] - c[fin]).abs().max()) <= 1e-5 * float(c[fin].abs().max())
    d = ops.fp8_mqa_logits(q8, (k8, ksc * 2), w, ks, ke)
    assert torch.equal(d[fin], a[fin] * 2)


def test_host_pipeline_matches_device_call():
    """Pinned-host inputs and outputs, chunked with copies on side streams: same indices, twice."""
    T, S, K = 1500, 4096, 256
    args = indexer_inputs(T, S, 64, 128, seed=31, window="random")
    want = ops.indexer_topk(*to_dev(*args), K).cpu()
    pipe = ops.HostIndexerPipeline(T, S, 64, 128, K, "cuda", chunks=3)
    assert len(pipe.bounds) == 3
    host = [t.pin_memory() for t in args]
    out = torch.empty(T, K, dtype=torch.int32).pin_memory()
    for _ in range(2):
        out.fill_(-5)
        pipe(*host, out)
        torch.cuda.synchronize()
        assert torch.equal(out, want)
    ops.check_status("cuda")


def test_host_pipeline_submits_back_to_back():
    """Several submits in a row with different inputs and separate outputs, no waiting in between: the
    staging slots and the two key buffers are handed from call to call by events alone."""
    T, S, K = 2600, 8192, 512
    pipe = ops.HostIndexerPipeline(T, S, 64, 128, K, "cuda", chunks=5)
    assert len(pipe.bounds) == 5 and pipe.bounds[0][1] - pipe.bounds[0][0] < pipe.bounds[2][1] - pipe.bounds[2][0]
    cases = [indexer_inputs(T, S, 64, 128, seed=40 + i, window="random") for i in range(4)]
    want = [ops.indexer_topk(*to_dev(*c), K).cpu() for c in cases]
    hosts = [[t.pin_memory() for t in c] for c in cases]
    outs = [torch.full((T, K), -5, dtype=torch.int32).pin_memory() for _ in cases]
    events = [pipe.submit(*h, o) for h, o in zip(hosts, outs)]
    for ev, o, w in zip(events, outs, want):
        ev.synchronize()
        assert torch.equal(o, w)
    ops.check_status("cuda")


@pytest.mark.parametrize("T,S,window", [(300, 4096, "causal"), (1021, 9000, "random"), (64, 70000, "causal")])
def test_register_weight_form_equals_general_kernel_bitwise(T, S, window):
    """64 heads x 128 takes the register-weight kernel; the test hook dsa_test_indexer_logits_general sends the
    same call through the general kernel.  Same summation order per (token, key): the logits agree bit for
    bit, for fp32 and bf16 weights."""
    from llmdivedeep_b200 import _lib
    q8, k8, ksc, w, ks, ke = to_dev(*indexer_inputs(T, S, 64, 128, seed=T + S, window=window))
    ld = (S + 3) // 4 * 4
    for wt in (w, w.bfloat16()):
        a = ops.fp8_mqa_logits(q8, (k8, ksc), wt, ks, ke).clone()
        bfull = torch.empty(T, ld, dtype=torch.float32, device="cuda")
        _lib.check(_lib.load().dsa_test_indexer_logits_general(
            q8.data_ptr(), k8.data_ptr(), ksc.data_ptr(), wt.data_ptr(), 1 if wt.dtype == torch.bfloat16 else 0,
            ks.data_ptr(), ke.data_ptr(), bfull.data_ptr(), ld, T, S, 64, 128, 1,
            ops.status_word("cuda").data_ptr(), torch.cuda.current_stream().cuda_stream))
        b = bfull[:, :S]
        assert torch.equal(a.view(torch.int32), b.view(torch.int32))
    ops.check_status("cuda")
