"""GPU: pins the CPU oracle against the reference's own GPU library.

oracle/_ref/libfastnn_ref.so is FastNN's unmodified cuda/kernels.cu (cuBLAS TF32) built for
sm_100a.  Replaying FastNN's tests/cuda_parity.rs -- CPU result vs GPU result on identical
SplitMix64 inputs, rtol 2e-2 / atol 2e-3 -- with the oracle in the CPU role shows that the
oracle and the reference's shipped GPU path agree the way the reference's CPU path must.
The same harness also checks this library against the reference library directly.
"""
import ctypes

import numpy as np
import pytest

import oracle
from helpers import check_tf32_parity, reference_assert_close

pytestmark = pytest.mark.gpu

_vp, _i, _f = ctypes.c_void_p, ctypes.c_int, ctypes.c_float


@pytest.fixture(scope="module")
def ref(gpu):
    path = oracle.ref_gpu_library_path()
    if path is None:
        pytest.skip("oracle/_ref/libfastnn_ref.so has not been built (needs the reference checkout)")
    lib = ctypes.CDLL(path)
    lib.fastnn_cuda_matmul.argtypes = [_vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _f, _f]
    lib.fastnn_cuda_matmul_batched.argtypes = [_vp, _vp, _vp, _i, _i, _i, _i, _f, _f]
    for name in ("fastnn_cuda_matmul_nt", "fastnn_cuda_matmul_tn"):
        getattr(lib, name).argtypes = [_vp, _vp, _vp, _i, _i, _i]
    for name in ("fastnn_cuda_matmul_batched_nt", "fastnn_cuda_matmul_batched_tn"):
        getattr(lib, name).argtypes = [_vp, _vp, _vp, _i, _i, _i, _i]
    assert lib.fastnn_cuda_init(0) == 0
    return lib


def _ref_call(lib, op, a, b):
    import torch
    da = torch.from_numpy(np.ascontiguousarray(a)).cuda()
    db = torch.from_numpy(np.ascontiguousarray(b)).cuda()
    batched = a.ndim == 3
    batch = a.shape[0] if batched else 1
    if op == "nn":
        m, k, n = a.shape[-2], a.shape[-1], b.shape[-1]
    elif op == "nt":
        m, k, n = a.shape[-2], a.shape[-1], b.shape[-2]
    else:
        k, m, n = a.shape[-2], a.shape[-1], b.shape[-1]
    out = torch.full((batch, m, n), float("nan"), device="cuda")
    p = lambda t: ctypes.c_void_p(t.data_ptr())
    if op == "nn" and not batched:
        rc = lib.fastnn_cuda_matmul(p(da), p(db), p(out), m, n, k, k, n, n, 1.0, 0.0)
    elif op == "nn":
        rc = lib.fastnn_cuda_matmul_batched(p(da), p(db), p(out), m, n, k, batch, 1.0, 0.0)
    elif not batched:
        rc = getattr(lib, f"fastnn_cuda_matmul_{op}")(p(da), p(db), p(out), m, n, k)
    else:
        rc = getattr(lib, f"fastnn_cuda_matmul_batched_{op}")(p(da), p(db), p(out), m, n, k, batch)
    assert rc == 0
    torch.cuda.synchronize()
    res = out.cpu().numpy()
    return res if batched else res[0]


def _oracle(op, a, b):
    return {"nn": oracle.matmul, "nt": oracle.matmul_nt, "tn": oracle.matmul_tn}[op](a, b)


def test_oracle_agrees_with_reference_gpu_on_reference_fixtures(ref, golden):
    for c in golden["cases"]:
        got = _ref_call(ref, c["op"], c["a"], c["b"])
        reference_assert_close(_oracle(c["op"], c["a"], c["b"]), got, what=c["name"])
        reference_assert_close(c["c"], got, what=c["name"] + " (golden)")


@pytest.mark.parametrize("op", ["nn", "nt", "tn"])
@pytest.mark.parametrize("shape", [(96, 80, 64, 0), (130, 67, 45, 0), (64, 48, 40, 3)])
def test_oracle_agrees_with_reference_gpu_mid_sizes(ref, op, shape):
    m, n, k, batch = shape
    rng = np.random.default_rng(m + n + k)
    sa = (k, m) if op == "tn" else (m, k)
    sb = (n, k) if op == "nt" else (k, n)
    if batch:
        sa, sb = (batch,) + sa, (batch,) + sb
    a = rng.uniform(-1, 1, sa).astype(np.float32)
    b = rng.uniform(-1, 1, sb).astype(np.float32)
    got = _ref_call(ref, op, a, b)
    want = _oracle(op, a, b)
    reference_assert_close(want, got, what=f"{op} {shape}")
    check_tf32_parity(got, want, k, a, b, what=f"reference GPU {op} {shape}")


@pytest.mark.parametrize("op", ["nn", "nt", "tn"])
def test_this_library_agrees_with_reference_gpu(gpu, ref, op):
    import torch
    f = gpu
    m, n, k = 512, 384, 256
    rng = np.random.default_rng(77)
    sa = (k, m) if op == "tn" else (m, k)
    sb = (n, k) if op == "nt" else (k, n)
    a = rng.standard_normal(sa, dtype=np.float32)
    b = rng.standard_normal(sb, dtype=np.float32)
    theirs = _ref_call(ref, op, a, b)
    fn = {"nn": f.matmul, "nt": f.matmul_nt, "tn": f.matmul_tn}[op]
    ours = fn(torch.from_numpy(a).cuda(), torch.from_numpy(b).cuda()).cpu().numpy()
    # two TF32 implementations (operand truncation here, cuBLAS's own rounding there): the
    # BASELINE tolerance applies between them as it does against the FP32 oracle
    check_tf32_parity(ours, theirs, k, a, b, what=f"{op} ours vs reference GPU")
    want = _oracle(op, a, b)
    e_ours = np.linalg.norm(ours - want) / np.linalg.norm(want)
    e_theirs = np.linalg.norm(theirs - want) / np.linalg.norm(want)
    assert e_ours <= 5e-3 and e_theirs <= 5e-3, (e_ours, e_theirs)
