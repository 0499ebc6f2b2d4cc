"""GPU tests of the library runtime: the give-up branch of the bounded device-side waits."""
import time

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_bounded_wait_runs_out_and_reports_timeout(b200, cuda):
    """A one-block kernel waits on an mbarrier nobody signals (wait limit 2 ms in that build unit).
    Both kinds of waiter give up, the status word reads B200_TIMEOUT and is cleared by the read, the
    call returns quickly, and the context keeps working.  Nothing traps and no wait is unbounded."""
    assert b200.device_status() == 0
    elapsed = torch.full((2,), -7, dtype=torch.int64, device=cuda)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    b200.wait_selftest(elapsed)
    st = b200.device_status()                      # synchronises the stream
    wall = time.perf_counter() - t0
    assert st == b200.B200_TIMEOUT
    assert b200.device_status() == 0               # the read cleared the word
    ns = elapsed.cpu().tolist()
    assert all(1.0e6 <= v <= 1.0e9 for v in ns), ns        # gave up after the limit, not instantly, not never
    assert wall < 2.0, wall
    # the context is intact: an ordinary kernel of the library runs and gives the right answer
    x = torch.empty(1000, dtype=torch.float32, device=cuda)
    b200.fill_normal_(x, 42, 1.0)
    torch.cuda.synchronize()
    ref = torch.from_numpy(b200.synth_normal_host(42, 0, 1000, 1.0))
    assert torch.equal(x.cpu(), ref)
    assert b200.device_status() == 0
