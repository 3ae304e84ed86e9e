"""dsa_indexer_topk_static: the entry point for hosts that cannot allocate device
memory where they call the library (a runtime that owns the device heap and bans
allocation inside operator callbacks, a serving loop with a frozen pool).  Its
logits scratch is an array built into the library, so the test checks that it
gives exactly what dsa_indexer_topk gives with a caller workspace -- on two
calls in a row, because the shared array keeps the first call's contents -- and
that it refuses problems larger than the array.  Collected last on purpose."""
import pytest
import torch

from llmdivedeep_b200 import _lib, ops
from tests.helpers import indexer_inputs, to_dev

pytestmark = pytest.mark.gpu


def test_static_scratch_matches_workspace_variant_twice():
    lib = _lib.load()
    assert lib.dsa_indexer_topk_static_max_bytes() == 64 << 20
    # the start-up call such a host makes once per device: T = 0 launches nothing, but it looks up
    # the array's device address, which is when the driver creates the 64 MiB on this GPU
    assert lib.dsa_indexer_topk_static(None, None, None, None, 0, None, None, 0, 65536, 64, 128, 2048, None, None,
                                       None) == 0
    first = to_dev(*indexer_inputs(300, 65536, 64, 128, seed=21, window="causal"))   # 2 chunks of the array
    second = to_dev(*indexer_inputs(513, 3000, 64, 128, seed=22, window="random"))
    for args, k in ((first, 512), (second, 256)):
        want = ops.indexer_topk(*args, k)
        out = torch.full_like(want, -7)
        got = ops.indexer_topk_static(*args, k, out=out)
        ops.check_status("cuda")
        assert got.data_ptr() == out.data_ptr()
        assert torch.equal(got, want)          # index work: bit-exact


def test_static_scratch_refuses_oversized_problems():
    T, S = 256, 65536 + 4
    q = torch.zeros(T, 64, 128, device="cuda").to(torch.float8_e4m3fn)
    k = torch.zeros(S, 128, device="cuda").to(torch.float8_e4m3fn)
    ksc = torch.ones(S, device="cuda")
    w = torch.ones(T, 64, device="cuda")
    ke = torch.full((T,), S, dtype=torch.int32, device="cuda")
    with pytest.raises(ops.DsaError, match="scratch"):
        ops.indexer_topk_static(q, k, ksc, w, None, ke, 16)
