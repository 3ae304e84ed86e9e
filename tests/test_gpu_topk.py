"""dsa_topk_select (through the C ABI) against torch.topk / exact rules. Index work: bit-exact."""
import pytest
import torch

from llmdivedeep_b200 import ops

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _sets_equal(x, idx, ks, ke, k):
    T = x.shape[0]
    for t in range(T):
        lo = int(ks[t]) if ks is not None else 0
        hi = int(ke[t]) if ke is not None else x.shape[1]
        kk = min(k, max(hi - lo, 0))
        got = idx[t].tolist()
        assert all(v == -1 for v in got[kk:]), f"row {t}: padding"
        if kk:
            ref = set((x[t, lo:hi].topk(kk).indices + lo).tolist())
            assert set(got[:kk]) == ref, f"row {t}"


@pytest.mark.parametrize("T,S,k", [(8, 1000, 16), (16, 4096, 256), (8, 65536, 2048), (4, 131072, 2048),
                                   (5, 5000, 2048), (3, 2049, 2048), (7, 300, 1), (2, 65537, 512)])
def test_random_rows_match_torch_topk(T, S, k):
    g = torch.Generator(device=DEV).manual_seed(S * 31 + k)
    x = torch.randn(T, S, device=DEV, generator=g)
    ke = torch.randint(S // 2, S + 1, (T,), device=DEV, dtype=torch.int32, generator=g)
    ks = torch.randint(0, max(S // 4, 1), (T,), device=DEV, dtype=torch.int32, generator=g)
    idx = ops.topk_select(x, k, ks, ke)
    _sets_equal(x, idx, ks, ke, k)
    assert torch.equal(idx, ops.topk_select(x, k, ks, ke)), "not deterministic"
    idx = ops.topk_select(x, k)            # no window
    _sets_equal(x, idx, None, None, k)


def test_short_windows_pad_with_minus_one():
    x = torch.randn(4, 512, device=DEV)
    ks = torch.tensor([0, 10, 500, 300], dtype=torch.int32, device=DEV)
    ke = torch.tensor([0, 13, 512, 200], dtype=torch.int32, device=DEV)   # empty, 3, 12, inverted
    idx = ops.topk_select(x, 16, ks, ke).cpu()
    assert idx[0].tolist() == [-1] * 16
    assert idx[1].tolist() == [10, 11, 12] + [-1] * 13
    assert idx[2].tolist() == list(range(500, 512)) + [-1] * 4
    assert idx[3].tolist() == [-1] * 16


def test_all_equal_rows_take_lowest_columns():
    x = torch.full((3, 10000), 2.5, device=DEV)
    idx = ops.topk_select(x, 2048)
    assert torch.equal(idx.sort(dim=1).values, torch.arange(2048, device=DEV, dtype=torch.int32).expand(3, -1))


def test_heavy_ties_break_towards_lower_columns():
    g = torch.Generator(device=DEV).manual_seed(5)
    x = torch.randint(0, 8, (4, 30000), device=DEV, generator=g).float()
    x[:, ::7] *= -1.0
    idx = ops.topk_select(x, 2048).long()
    for t in range(4):
        sel = torch.zeros(30000, dtype=torch.bool, device=DEV)
        sel[idx[t]] = True
        assert int(sel.sum()) == 2048
        thr = x[t][sel].min()
        assert x[t][~sel].max() <= thr
        tie = (x[t] == thr).nonzero().flatten()
        n_tie = int(sel[tie].sum())
        assert bool(sel[tie[:n_tie]].all()) and not bool(sel[tie[n_tie:]].any())


def test_special_values_and_signs():
    x = torch.randn(2, 4096, device=DEV)
    x[0, 100] = float("inf")
    x[0, 200:300] = float("-inf")
    x[1] = -x[1].abs() - 1.0            # all negative
    x[1, 7] = -0.0
    x[1, 9] = 0.0
    idx = ops.topk_select(x, 64)
    _sets_equal(x, idx, None, None, 64)
    assert 100 in idx[0].tolist() and 9 in idx[1].tolist() and 7 in idx[1].tolist()


def test_unaligned_leading_dimension_uses_scalar_loads():
    base = torch.randn(6, 1001, device=DEV)
    x = base[:, :999]                    # ld = 1001: rows are not 16-byte aligned
    idx = ops.topk_select(x, 50)
    _sets_equal(x, idx, None, None, 50)


def test_many_candidates_in_one_bin_takes_extra_passes():
    # values so close together that the threshold bin of the first pass overflows
    # the in-shared-memory finish (more than 2048 candidates share 12 key bits)
    g = torch.Generator(device=DEV).manual_seed(9)
    x = 1.0 + torch.rand(3, 50000, device=DEV, generator=g) * 1e-3
    idx = ops.topk_select(x, 2048)
    _sets_equal(x, idx, None, None, 2048)
    x = 1.0 + torch.rand(2, 50000, device=DEV, generator=g) * 1e-6   # few distinct floats, massive ties
    idx = ops.topk_select(x, 2048).long()
    for t in range(2):
        sel = torch.zeros(50000, dtype=torch.bool, device=DEV)
        sel[idx[t]] = True
        assert int(sel.sum()) == 2048 and x[t][~sel].max() <= x[t][sel].min()


def test_full_size_row_property():
    """Bench-size rows: selected minimum >= unselected maximum, count == k."""
    T, S, k = 64, 131072, 2048
    x = torch.randn(T, S, device=DEV)
    idx = ops.topk_select(x, k).long()
    sel = torch.zeros(T, S, dtype=torch.bool, device=DEV)
    sel.scatter_(1, idx, True)
    assert bool((sel.sum(1) == k).all())
    lo_sel = torch.where(sel, x, torch.full_like(x, float("inf"))).amin(1)
    hi_uns = torch.where(sel, torch.full_like(x, float("-inf")), x).amax(1)
    assert bool((lo_sel >= hi_uns).all())


def _two_pass(x, k, ks=None, ke=None):
    """The same call through the test hook that keeps every row on the two-pass path."""
    from llmdivedeep_b200 import _lib
    T, S = x.shape
    out = torch.empty(T, k, dtype=torch.int32, device=x.device)
    _lib.check(_lib.load().dsa_test_topk_select_two_pass(
        x.data_ptr(), x.stride(0), None if ks is None else ks.data_ptr(), None if ke is None else ke.data_ptr(),
        T, S, k, out.data_ptr(), torch.cuda.current_stream().cuda_stream))
    return out


def _adversarial_rows(S, g):
    """Rows built to mislead a sample taken as one 128-column block in every 16: a ramp, the large
    values packed into few blocks, a two-level row with more ties than the candidate capacity, a
    near-constant row, and a row whose large values sit exactly in the sampled blocks."""
    rows = [torch.randn(S, device=DEV, generator=g),
            torch.arange(S, device=DEV, dtype=torch.float32),
            -torch.arange(S, device=DEV, dtype=torch.float32)]
    r = torch.randn(S, device=DEV, generator=g)
    r[4096:4096 + 3000] += 100.0                              # contiguous spike wider than k
    rows.append(r)
    r = torch.zeros(S, device=DEV)
    r[torch.randperm(S, device=DEV, generator=g)[:6000]] = 1.0   # 6000 tied maxima
    rows.append(r)
    rows.append(torch.full((S,), 3.0, device=DEV) + 1e-7 * torch.randn(S, device=DEV, generator=g))
    r = torch.randn(S, device=DEV, generator=g)
    blk = torch.arange(S, device=DEV) // 128
    r[(blk % 16) == 8] += 6.0                                 # only the sampled blocks are large
    rows.append(r)
    r = torch.randn(S, device=DEV, generator=g)
    r[(blk % 16) == 8] -= 6.0                                 # the sampled blocks are small
    rows.append(r)
    return torch.stack(rows)


@pytest.mark.parametrize("S,k", [(65536, 2048), (131072, 2048), (16384, 2048), (40000, 512), (300000, 2048)])
def test_sampled_pass_equals_two_pass_on_adversarial_rows(S, k):
    g = torch.Generator(device=DEV).manual_seed(S + k)
    x = _adversarial_rows(S, g)
    a = ops.topk_select(x, k)
    b = _two_pass(x, k)
    assert torch.equal(a.sort(dim=1).values, b.sort(dim=1).values)
    _sets_equal_with_ties(x, a, k)
    T = x.shape[0]
    # the output of a row does not depend on how many rows the call has
    many = ops.topk_select(x.repeat(10, 1), k)
    assert torch.equal(many[:T], a) and torch.equal(many[-T:], a)
    ks = torch.randint(0, S // 8, (T,), device=DEV, dtype=torch.int32, generator=g)
    ke = torch.randint(S - S // 8, S + 1, (T,), device=DEV, dtype=torch.int32, generator=g)
    a = ops.topk_select(x, k, ks, ke)
    assert torch.equal(a, ops.topk_select(x, k, ks, ke)), "not deterministic"
    assert torch.equal(a.sort(dim=1).values, _two_pass(x, k, ks, ke).sort(dim=1).values)


def _sets_equal_with_ties(x, idx, k):
    """Exact rule: everything above the k-th value is selected, the rest are the lowest columns equal to it."""
    for t in range(x.shape[0]):
        row = x[t]
        kth = row.topk(k).values[-1]
        above = (row > kth).nonzero().flatten()
        tied = (row == kth).nonzero().flatten()[: k - above.numel()]
        want = torch.cat([above, tied]).sort().values
        assert torch.equal(idx[t].long().sort().values, want), f"row {t}"
