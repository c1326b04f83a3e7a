"""A bounded device wait that really runs out, in the safe form: the library's self-test kernel
waits 2 ms on a barrier nothing completes, gives up, reports its site through the status word and
returns normally.  The context stays usable and the next kernels run as before."""

import pytest
import torch

pytestmark = pytest.mark.gpu

from bongard_b200 import _lib, ops  # noqa: E402


def test_a_wait_that_runs_out_is_reported_and_the_library_keeps_working():
    lib = _lib.load()
    ops.read_status()                                     # clean to start with
    finished = torch.zeros(1, dtype=torch.int32, device='cuda')
    stream = torch.cuda.current_stream().cuda_stream
    assert lib.bg_selftest_bounded_wait(2000, finished.data_ptr(), stream) == 0
    with pytest.raises(_lib.B200Error, match='901'):
        ops.read_status()                                 # synchronises, reports the site, clears the word
    assert int(finished.item()) == 1                      # the kernel fell through its teardown
    ops.read_status()                                     # cleared: a second read is clean
    # the library still works on the same context
    x = torch.randn(300, 256, device='cuda').bfloat16()
    w = torch.randn(128, 256, device='cuda').bfloat16()
    y = ops.linear(x, w)
    ops.read_status()
    assert float((y.float() - x.float() @ w.float().t()).abs().max()) < 0.25
    # argument check
    assert lib.bg_selftest_bounded_wait(0, None, stream) != 0
