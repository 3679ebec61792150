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


# ----------------------------------------------------------------------------------------
# The restatements beside the matmul family -- Conv2d forward and both gradients, the ReLU / GELU
# derivatives, the row softmax -- pinned the same way: FastNN's own CUDA entries for them
# (cuda/kernels.cu:896-1026, 244-282, 289-337, 407) run here on identical inputs, the oracle takes
# the CPU role of tests/cuda_parity.rs with its element rule (rtol 2e-2 / atol 2e-3 where a TF32
# GEMM is involved; 1e-5 for the elementwise kernels, which are FP32 on both sides).
# ----------------------------------------------------------------------------------------

def _dev(x):
    import torch
    return torch.from_numpy(np.ascontiguousarray(x, dtype=np.float32)).cuda()


def _p(t):
    return ctypes.c_void_p(t.data_ptr())


CONV_CASES = [
    # n, ci, co, h, w, kh, kw, stride, padding
    (2, 3, 8, 12, 12, 3, 3, (1, 1), (1, 1)),
    (3, 4, 6, 15, 17, 3, 3, (2, 2), (1, 1)),         # stride 2
    (2, 5, 7, 19, 23, 7, 7, (2, 2), (3, 3)),         # 7 x 7, stride 2
    (1, 6, 4, 9, 11, 1, 1, (1, 1), (0, 0)),          # pointwise
    (2, 2, 3, 10, 8, 5, 3, (1, 2), (2, 0)),          # rectangular kernel, uneven stride and padding
]


@pytest.mark.parametrize("cfg", CONV_CASES)
def test_conv_oracle_agrees_with_reference_gpu(ref, cfg):
    import torch
    n, ci, co, h, w, kh, kw, (sh, sw), (ph, pw) = cfg
    rng = np.random.default_rng(sum(cfg[:7]))
    x = rng.uniform(-1, 1, (n, ci, h, w)).astype(np.float32)
    wt = rng.uniform(-1, 1, (co, ci, kh, kw)).astype(np.float32)
    bias = rng.uniform(-1, 1, co).astype(np.float32)
    oh, ow = (h + 2 * ph - kh) // sh + 1, (w + 2 * pw - kw) // sw + 1
    go = rng.uniform(-1, 1, (n, co, oh, ow)).astype(np.float32)
    dx, dw, db, dgo = _dev(x), _dev(wt), _dev(bias), _dev(go)
    dims = [_i(v) for v in (n, ci, co, h, w)]
    tail = [_i(v) for v in (kh, kw, sh, sw, ph, pw)]
    out = torch.full((n, co, oh, ow), float("nan"), device="cuda")
    assert ref.fastnn_cuda_conv2d_forward(_p(dx), _p(dw), _p(db), _p(out), *dims, *tail) == 0
    gi = torch.full(x.shape, float("nan"), device="cuda")
    gw = torch.full(wt.shape, float("nan"), device="cuda")
    assert ref.fastnn_cuda_conv2d_backward_data(_p(dgo), _p(dw), _p(gi), *dims, _i(oh), _i(ow), *tail) == 0
    assert ref.fastnn_cuda_conv2d_backward_weight(_p(dx), _p(dgo), _p(gw), *dims, _i(oh), _i(ow), *tail) == 0
    torch.cuda.synchronize()
    want = oracle.conv2d(x, wt, bias, (sh, sw), (ph, pw))
    want_gi, want_gw = oracle.conv2d_backward(x, wt, go, (sh, sw), (ph, pw))
    reference_assert_close(want, out.cpu().numpy(), what=f"conv forward {cfg}")
    reference_assert_close(want_gi, gi.cpu().numpy(), what=f"conv grad_input {cfg}")
    reference_assert_close(want_gw, gw.cpu().numpy(), what=f"conv grad_weight {cfg}")


@pytest.mark.parametrize("cfg", CONV_CASES)
def test_this_library_conv_agrees_with_reference_gpu(gpu, ref, cfg):
    """The drop-in symbols against the entries they replace, same arguments."""
    import torch
    f = gpu
    n, ci, co, h, w, kh, kw, (sh, sw), (ph, pw) = cfg
    rng = np.random.default_rng(100 + sum(cfg[:7]))
    x = rng.standard_normal((n, ci, h, w)).astype(np.float32)
    wt = (rng.standard_normal((co, ci, kh, kw)) * 0.2).astype(np.float32)
    oh, ow = (h + 2 * ph - kh) // sh + 1, (w + 2 * pw - kw) // sw + 1
    go = rng.standard_normal((n, co, oh, ow)).astype(np.float32)
    dx, dw, dgo = _dev(x), _dev(wt), _dev(go)
    dims = (n, ci, co, h, w)
    tail = (kh, kw, sh, sw, ph, pw)
    outs = {}
    for name, lib in (("theirs", ref), ("ours", f.lib())):
        y = torch.full((n, co, oh, ow), float("nan"), device="cuda")
        gi = torch.full(x.shape, float("nan"), device="cuda")
        gw = torch.full(wt.shape, float("nan"), device="cuda")
        i = _i if name == "theirs" else int
        assert lib.fastnn_cuda_conv2d_forward(_p(dx), _p(dw), ctypes.c_void_p(0), _p(y), *map(i, dims), *map(i, tail)) == 0
        assert lib.fastnn_cuda_conv2d_backward_data(_p(dgo), _p(dw), _p(gi), *map(i, dims), i(oh), i(ow), *map(i, tail)) == 0
        assert lib.fastnn_cuda_conv2d_backward_weight(_p(dx), _p(dgo), _p(gw), *map(i, dims), i(oh), i(ow), *map(i, tail)) == 0
        torch.cuda.synchronize()
        outs[name] = [t.cpu().numpy() for t in (y, gi, gw)]
    for what, a, b in zip(("forward", "grad_input", "grad_weight"), outs["theirs"], outs["ours"]):
        reference_assert_close(a, b, what=f"{what} {cfg}: ours vs FastNN's entry")


def test_activation_derivative_oracle_agrees_with_reference_gpu(ref):
    """ReluBackward / GeluBackward (src/autograd/backward_ops.rs:136-160, 194-218) as restated in the
    oracle's backward epilogue against fastnn_cuda_relu_backward / fastnn_cuda_gelu_backward."""
    import torch
    rng = np.random.default_rng(8)
    rows, n = 37, 53
    pre = (rng.standard_normal((rows, n)) * 2.5).astype(np.float32)
    pre[0, :5] = [0.0, -0.0, 1e-30, -1e-30, 8.0]                       # the ReLU kink and the tails
    go = rng.uniform(-1, 1, (rows, n)).astype(np.float32)
    ident = np.eye(n, dtype=np.float32)                                # dy . I = dy exactly
    for act, name in ((oracle.ACT_RELU, "fastnn_cuda_relu_backward"), (oracle.ACT_GELU, "fastnn_cuda_gelu_backward")):
        want, colsum = oracle.linear_backward_input(go, ident, pre, act)
        gi = torch.full((rows, n), float("nan"), device="cuda")
        fn = getattr(ref, name)
        fn.argtypes = [_vp, _vp, _vp, ctypes.c_size_t]
        assert fn(_p(_dev(go)), _p(_dev(pre)), _p(gi), rows * n) == 0
        torch.cuda.synchronize()
        got = gi.cpu().numpy()
        assert np.abs(got - want).max() <= 1e-5, name
        assert np.abs(colsum - got.astype(np.float64).sum(axis=0)).max() <= 1e-4


@pytest.mark.parametrize("t", [64, 128, 320])
def test_softmax_oracle_agrees_with_reference_gpu(ref, t):
    """Tensor::softmax over the last axis (src/tensor/ops.rs:273-284), as the oracle's attention
    restatement applies it to scaled, causally masked scores, against fastnn_cuda_softmax on the
    same masked input (-1e9 above the diagonal, src/nn/transformer.rs:22-27).

    Row lengths are powers of two or at least 256: FastNN's kernel_softmax launches
    min(row length, 256) threads and halves that count in its shared-memory reduction
    (cuda/kernels.cu:304-308, 408), which drops partial sums for any other thread count (48 keys
    gave probabilities off by 1.5).  Its CPU path, which the oracle restates, has no such limit."""
    import torch
    rng = np.random.default_rng(9)
    heads = 5
    scale = np.float32(1.0 / np.sqrt(32.0))
    scores = (rng.standard_normal((heads, t, t)) * 6.0).astype(np.float32)
    want = oracle.causal_softmax(scores, float(scale))
    masked = scores * scale + np.triu(np.full((t, t), -1e9, dtype=np.float32), k=1)[None]
    out = torch.full((heads * t, t), float("nan"), device="cuda")
    ref.fastnn_cuda_softmax.argtypes = [_vp, _vp, _i, _i]
    assert ref.fastnn_cuda_softmax(_p(_dev(masked.reshape(heads * t, t))), _p(out), heads * t, t) == 0
    torch.cuda.synchronize()
    got = out.cpu().numpy().reshape(heads, t, t)
    assert np.abs(got - want).max() <= 1e-5
    assert np.abs(got.sum(axis=-1) - 1.0).max() <= 1e-5
    assert (got[:, np.triu_indices(t, 1)[0], np.triu_indices(t, 1)[1]] == 0.0).all()
