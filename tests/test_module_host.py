"""Host-only checks of the module mirror (llmdivedeep_b200/DSA.py) and of the oracle's stage
outputs against the reference's recorded ones: nothing here launches a kernel."""
import os

import numpy as np
import pytest
import torch

from llmdivedeep_b200 import DSA, ops
from oracle import dsa_oracle as O

G = np.load(os.path.join(os.path.dirname(__file__), "golden", "reference_golden.npz"))


def bf16(a):
    return torch.from_numpy(a.view(np.int16).copy()).view(torch.bfloat16)


def _params(tag):
    return {k: bf16(G[f"mod_{tag}_{k}"]) for k in ("wq_b", "wk", "weights_proj", "k_norm_w", "k_norm_b")}


@pytest.mark.parametrize("tag,interleave", [("neox", False), ("glm", True)])
def test_oracle_stage_outputs_equal_the_reference_bytes(tag, interleave):
    """Projections -> k_norm -> RoPE -> FP8 quantiser of the oracle give the bytes, scales and
    head gates the unmodified reference hands to its scorer (sparse_attn/DSA.py:530-543)."""
    x, ql = bf16(G[f"mod_{tag}_x"]), bf16(G[f"mod_{tag}_qlora"])
    q8, k8, ksc, w_eff, ks, ke = O.dsa_indexer_inputs(_params(tag), x, ql, 4, 128, 64, interleave=interleave)
    assert np.array_equal(q8.view(torch.uint8).numpy(), G[f"mod_{tag}_q_fp8"])
    assert np.array_equal(k8.view(torch.uint8).numpy(), G[f"mod_{tag}_k_fp8"])
    assert np.array_equal(ksc.numpy(), G[f"mod_{tag}_k_scale"])
    ref_w = O.fold_weights(torch.from_numpy(G[f"mod_{tag}_w"]), torch.from_numpy(G[f"mod_{tag}_q_scale"]), 128)
    assert torch.equal(w_eff, ref_w)


@pytest.mark.parametrize("tag,interleave", [("neox", False), ("glm", True)])
def test_mirror_rope_feeds_the_quantiser_the_reference_values(tag, interleave):
    """DSA._rope_head on the module's bf16 projections, quantised, must give the reference's FP8
    bytes and scales: the NeoX form hands the quantiser unrounded fp32 products, the interleaved
    form values rounded to bf16 (sparse_attn/DSA.py:444-469, 513-524)."""
    p = _params(tag)
    x, ql = bf16(G[f"mod_{tag}_x"]), bf16(G[f"mod_{tag}_qlora"])
    T = x.shape[0]
    q = torch.nn.functional.linear(ql, p["wq_b"]).view(T, 4, 128)
    k = torch.nn.functional.layer_norm(torch.nn.functional.linear(x, p["wk"]), (128,), p["k_norm_w"], p["k_norm_b"])
    q, k = DSA._rope_head(q, 64, T, interleave), DSA._rope_head(k, 64, T, interleave)
    assert q.dtype == (torch.bfloat16 if interleave else torch.float32)
    q8, qs = O.fp8_quant_per_block(q)
    k8, ksc = O.fp8_quant_per_block(k)
    assert np.array_equal(q8.view(torch.uint8).numpy(), G[f"mod_{tag}_q_fp8"])
    assert np.array_equal(qs.numpy(), G[f"mod_{tag}_q_scale"])
    assert np.array_equal(k8.view(torch.uint8).numpy(), G[f"mod_{tag}_k_fp8"])
    assert np.array_equal(ksc.numpy(), G[f"mod_{tag}_k_scale"])


def test_rope_forms_equal_the_oracle_on_fp32_and_bf16():
    cos, sin = O.rope_cossin(10, 64)
    for dt in (torch.float32, torch.bfloat16):
        x = torch.randn(10, 3, 64).to(dt)
        assert torch.equal(DSA._rotate(x, cos, sin, False), O.apply_rope_neox(x, cos, sin))
        assert torch.equal(DSA._rotate(x, cos, sin, True), O.apply_rope_interleave(x, cos, sin))


def test_ops_refuse_cpu_tensors():
    q8 = torch.zeros(4, 64, 128).to(torch.float8_e4m3fn)
    with pytest.raises(ops.DsaError):
        ops.fp8_mqa_logits(q8, (q8[0], torch.ones(64)), torch.ones(4, 64), None, torch.ones(4, dtype=torch.int32))


class _FakeCudaTensor:
    """Stands in for a CUDA tensor in the argument checks (which only look at is_cuda / device)."""
    is_cuda = True

    def __init__(self, index):
        self.device = torch.device("cuda", index)


def test_ops_refuse_tensors_of_different_devices():
    assert ops._need_cuda(_FakeCudaTensor(1), None, _FakeCudaTensor(1)) == torch.device("cuda", 1)
    with pytest.raises(ops.DsaError, match="one device"):
        ops._need_cuda(_FakeCudaTensor(0), _FakeCudaTensor(1))
    with pytest.raises(ops.DsaError):
        ops._need_cuda(_FakeCudaTensor(0), torch.zeros(1))
    with pytest.raises(ops.DsaError):
        ops._dev_index("cpu")
    assert ops._dev_index("cuda:3") == 3


def test_index_output_must_have_the_kernel_stride():
    ok = torch.empty(6, 8, dtype=torch.int32)
    assert ops._check_idx_out(ok, 6, 8, "cpu") is ok
    for bad in (torch.empty(6, 16, dtype=torch.int32)[:, :8], torch.empty(6, 8, dtype=torch.int64),
                torch.empty(6, 16, dtype=torch.int32)):
        with pytest.raises(ops.DsaError):
            ops._check_idx_out(bad, 6, 8, "cpu")


def test_index_share_runs_the_indexer_every_freq_layers():
    from llmdivedeep_b200 import layer
    calls = []

    def indexer(x):
        calls.append(x)
        return len(calls)

    share = layer.IndexShare(freq=4)
    got = [share.select(i, indexer, i) for i in range(10)]
    assert calls == [0, 4, 8] and got == [1, 1, 1, 1, 2, 2, 2, 2, 3, 3] and share.runs == 3
    assert [layer.IndexShare(1).select(i, indexer, i) for i in range(3)] == [4, 5, 6]
    with pytest.raises(ValueError):
        layer.IndexShare(0)
