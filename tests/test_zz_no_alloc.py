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


_FRESH_PROCESS = r"""
import ctypes, sys
import torch
sys.path.insert(0, {root!r})
from fastnn_b200 import _lib
lib = _lib.lib()                      # loads the library; fastnn_cuda_init is never called here
torch.cuda.set_device(0)
vp = lambda t: ctypes.c_void_p(t.data_ptr())
free = lambda: torch.cuda.mem_get_info()[0]
status = ctypes.c_uint(99)

# every buffer the calls use exists before the first measurement (torch's allocator is the
# caller's business, not the library's)
shapes = [(256, 256, 512, 2), (384, 512, 2048, 8), (1024, 1024, 1024, 4)]
bufs = []
for m, n, k, s in shapes:
    a = torch.randn(m, k, device="cuda"); b = torch.randn(k, n, device="cuda")
    bufs.append((a, b, torch.empty(m, n, device="cuda"), torch.matmul(a.double(), b.double())))
torch.cuda.synchronize()

# first call: the CUDA runtime loads the library's kernels and its 16 MiB array on first use
m, n, k, s = shapes[0]; a, b, c, want = bufs[0]
assert lib.fastnn_b200_gemm_splitk_static(0, vp(a), vp(b), vp(c), m, n, k, s, None) == 0
torch.cuda.synchronize()
assert lib.fastnn_b200_device_status(ctypes.byref(status)) == 0 and status.value == 0
before = free()
# later calls, with partial-sum footprints 4x and 32x the first one's: an entry that kept its
# partial sums in an allocated workspace would have to grow it here
for (m, n, k, s), (a, b, c, want) in zip(shapes, bufs):
    for _ in range(2):
        assert lib.fastnn_b200_gemm_splitk_static(0, vp(a), vp(b), vp(c), m, n, k, s, None) == 0
    torch.cuda.synchronize()
    assert free() == before, "device free memory changed across a call"
status.value = 99
assert lib.fastnn_b200_device_status(ctypes.byref(status)) == 0 and status.value == 0
assert free() == before
# results, checked only now: torch's own temporaries may grow its pool
for a, b, c, want in bufs:
    err = (c.double() - want).norm() / want.norm()
    assert float(err) < 5e-3, float(err)
# the entries that need fastnn_cuda_init still refuse to run without it
assert lib.fastnn_cuda_matmul_nt(vp(bufs[0][0]), vp(bufs[0][0]), vp(bufs[0][2]), 256, 256, 512) == -1
print("ok")
"""


def test_static_entry_in_a_fresh_process_without_init_allocates_nothing(built_library):
    """The two properties the entry exists for, in a process that never calls fastnn_cuda_init:
    it works, and device free memory (cudaMemGetInfo) is identical before and after its calls.
    Its status word is readable through fastnn_b200_device_status without initialisation too."""
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    proc = subprocess.run([sys.executable, "-c", _FRESH_PROCESS.format(root=root)], capture_output=True,
                          text=True, timeout=600)
    assert proc.returncode == 0, proc.stdout + proc.stderr
    assert proc.stdout.strip().endswith("ok")
