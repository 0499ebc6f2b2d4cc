"""Work split of the tensor-core router logits kernel, checked on the host (no GPU needed): the kernel's CTAs cut
their ranges of (128-token tile, 128-deep block) units into partial sums and number them per tile; the selection
kernel adds a token's partial sums by the same arithmetic.  The library's host-side walk must find consecutive
slots in order of d, every block covered once and no tile above the bound the scratch is sized with."""
import ctypes as C

import pytest


@pytest.mark.parametrize("sms", [1, 2, 74, 132, 148, 160])
@pytest.mark.parametrize("T,D", [(256, 512), (300, 1024), (512, 7168), (4096, 7168), (4097, 7168), (65536, 2048)])
def test_router_work_split_is_consistent(b200, T, D, sms):
    for chain in (0, 1, 2, 4, D // 128):
        mx = C.c_int(-1)
        rc = b200.lib().b200_tc_plan_selftest(T, D, sms, chain, C.byref(mx))
        assert rc == 0, (T, D, sms, chain, rc)
        ch = min(chain if chain > 0 else 4, D // 128)
        assert 1 <= mx.value <= 2 * -(-(D // 128) // ch) + 1


def test_router_work_split_rejects_bad_arguments(b200):
    assert b200.lib().b200_tc_plan_selftest(0, 512, 148, 0, None) != 0
    assert b200.lib().b200_tc_plan_selftest(256, 500, 148, 0, None) != 0
