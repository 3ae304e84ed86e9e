"""The bounded-wait policy of the kernels, exercised without touching a live pipeline: one thread
waits on a barrier nobody arrives at and must return the time-out status after the given number of
polls (no TMA, no MMA, no tensor memory in that kernel)."""
import pytest
import torch

from llmdivedeep_b200 import _lib

pytestmark = pytest.mark.gpu


def test_a_starved_wait_gives_up_with_status_1():
    lib = _lib.load()
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    _lib.check(lib.dsa_test_bounded_wait(1024, status.data_ptr(), torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    assert int(status.item()) == 1
    # the context is still usable and a second probe behaves the same
    status.zero_()
    _lib.check(lib.dsa_test_bounded_wait(8, status.data_ptr(), torch.cuda.current_stream().cuda_stream))
    assert int(status.item()) == 1
    assert lib.dsa_test_bounded_wait(0, status.data_ptr(), None) == -5
