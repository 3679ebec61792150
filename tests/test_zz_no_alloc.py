"""GPU: the GEMM entry point that allocates nothing, against the ordinary entry points.

Some callers cannot let a library call cudaMalloc when they need a product: a capture may be
open on another thread, the loop may be real-time, or device memory may be budgeted up front.
For them the library offers fastnn_b200_gemm_splitk_static, whose split-K partial sums live in
a fixed 16 MiB array inside the library.  This file checks, through the C ABI, that it returns
what the allocating split-K path returns -- twice in a row with different shapes, because the
array is shared between calls and still holds the previous call's partial sums -- and that a
request that cannot fit the array is refused instead of overrunning it.

Collected last on purpose (file name), so a failure here cannot hide the other tests.
"""
import ctypes

import numpy as np
import pytest

import oracle
from helpers import check_tf32_parity

pytestmark = pytest.mark.gpu

NN, NT, TN = 0, 1, 2


def _operands(layout, m, n, k, seed):
    rng = np.random.default_rng(seed)
    sa = (k, m) if layout == TN else (m, k)
    sb = (n, k) if layout == NT else (k, n)
    return rng.standard_normal(sa, dtype=np.float32), rng.standard_normal(sb, dtype=np.float32)


def _existing(f, layout, da, db, split_k):
    f.set_policy(3, 128, split_k)          # same kernel, tile width and split as the static entry
    try:
        return [f.matmul, f.matmul_nt, f.matmul_tn][layout](da, db)
    finally:
        f.set_policy(0, 0, 0)


def test_static_scratch_entry_matches_allocating_entry_twice_in_a_row(gpu):
    import torch
    f = gpu
    # second call is smaller and has fewer splits: stale partial sums of the first call stay in
    # the array beside and behind the region it uses
    cases = [(TN, 256, 768, 8192, 12), (NN, 384, 256, 1024, 4), (NT, 128, 132, 512, 16)]
    for layout, m, n, k, split_k in cases:
        a, b = _operands(layout, m, n, k, seed=m + n + k)
        da, db = torch.from_numpy(a).cuda(), torch.from_numpy(b).cuda()
        out = torch.full((m, n), float("nan"), device="cuda")
        got = f.gemm_splitk_static(layout, da, db, m, n, k, split_k, out=out)
        want = _existing(f, layout, da, db, split_k)
        torch.cuda.synchronize()
        g, w = got.cpu().numpy(), want.cpu().numpy()
        ref = [oracle.matmul, oracle.matmul_nt, oracle.matmul_tn][layout](a, b)
        check_tf32_parity(g, ref, k, a, b, what=f"static entry L{layout} vs oracle")
        # against the existing entry point: TF32 tolerance of the suite (in practice identical,
        # both add the same partial tiles in the same order)
        check_tf32_parity(g, w, k, a, b, what=f"static entry L{layout} vs allocating entry")
        assert np.abs(g - w).max() <= 1e-5 * np.abs(w).max()
    assert f.device_status() == 0


def test_static_scratch_entry_refuses_what_does_not_fit(gpu):
    import torch
    f = gpu
    m, n, k = 2048, 2048, 256                  # 4 Mi floats per split: two splits cannot fit
    a = torch.zeros((m, k), device="cuda")
    b = torch.zeros((k, n), device="cuda")
    c = torch.full((m, n), 7.0, device="cuda")
    lib = f.lib()
    p = lambda t: ctypes.c_void_p(t.data_ptr())
    assert lib.fastnn_b200_gemm_splitk_static(NN, p(a), p(b), p(c), m, n, k, 2, None) == -2
    torch.cuda.synchronize()
    assert bool((c == 7.0).all()), "a refused call must not touch the output"
    assert lib.fastnn_b200_gemm_splitk_static(NN, p(a), p(b), p(c), m, n, k, 1, None) == 0
    torch.cuda.synchronize()
    assert bool((c == 0.0).all())
    # misaligned row length
    assert lib.fastnn_b200_gemm_splitk_static(NN, p(a), p(b), p(c), 8, 6, 8, 1, None) == -1
