"""GPU: the bounded wait that every kernel of the library uses on its mbarriers, made to run out.

A one-warp kernel waits, with the GEMM kernels' own wait routine and a 1 ms budget, on a barrier
nothing arrives on.  Nothing else is in flight, so nothing can fault or hang.  The wait must give
up, the status word must carry the code exactly once, and the device must compute correctly
afterwards."""
import numpy as np
import pytest

import oracle
from helpers import check_tf32_parity

pytestmark = pytest.mark.gpu


def test_wait_runs_out_reports_once_and_the_device_stays_usable(gpu):
    import torch
    f = gpu
    assert f.device_status() == 0
    waited_us = f.selftest_bounded_wait(1000)
    # the budget is counted in SM clock ticks at the maximum clock: at least the budget, and far
    # below a second even at idle clocks
    assert 900 <= waited_us <= 200_000, waited_us
    assert f.device_status() == 0x1F0, "the expired wait must leave its code in the status word"
    assert f.device_status() == 0, "reading the status clears it"
    rng = np.random.default_rng(4)
    a = rng.standard_normal((256, 192), dtype=np.float32)
    b = rng.standard_normal((192, 160), dtype=np.float32)
    got = f.matmul(torch.from_numpy(a).cuda(), torch.from_numpy(b).cuda())
    check_tf32_parity(got.cpu().numpy(), oracle.matmul(a, b), 192, a, b, what="GEMM after an expired wait")
    assert f.device_status() == 0


def test_wait_budget_is_checked(gpu):
    f = gpu
    with pytest.raises(f.CudaError):
        f.selftest_bounded_wait(0)
    with pytest.raises(f.CudaError):
        f.selftest_bounded_wait(10_000_000)
    assert f.device_status() == 0
