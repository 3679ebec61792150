"""GPU parity tests: every GEMM entry of the C ABI against the CPU oracle on identical inputs.

Tolerance (TF32 multiply, FP32 accumulate vs FP32 CPU): relative Frobenius error <= 5e-3 and
max-abs error <= 1e-2 * sqrt(K) * max|A| * max|B|; the reference's own element rule
(rtol 2e-2 / atol 2e-3) is checked as well on its six fixture shapes.
"""
import ctypes

import numpy as np
import pytest

import oracle
from helpers import check_tf32_parity, reference_assert_close

pytestmark = pytest.mark.gpu

NN, NT, TN = 0, 1, 2


def _dev(x):
    import torch
    return torch.from_numpy(np.ascontiguousarray(x)).cuda()


def _host(t):
    return t.detach().cpu().numpy()


def _shapes(layout, m, n, k, batch):
    sa = (k, m) if layout == TN else (m, k)
    sb = (n, k) if layout == NT else (k, n)
    if batch:
        sa, sb = (batch,) + sa, (batch,) + sb
    return sa, sb


def _oracle(layout, a, b):
    return [oracle.matmul, oracle.matmul_nt, oracle.matmul_tn][layout](a, b)


def _gpu_fn(f, layout):
    return [f.matmul, f.matmul_nt, f.matmul_tn][layout]


# ------------------------------------------------------------------ reference fixtures ---

def test_reference_fixture_shapes_forward_and_gradients(gpu, golden):
    """The six matmul-family cases of FastNN's tests/cuda_parity.rs:116-166, forward and both
    input gradients (GradFns of src/autograd/backward_ops.rs:82-134), on the fixture inputs."""
    f = gpu
    for c in golden["cases"]:
        a, b, w = c["a"], c["b"], c["w"]
        da, db, dw = _dev(a), _dev(b), _dev(w)
        if c["op"] == "nn":
            out, ga, gb = f.matmul(da, db), f.matmul_nt(dw, db), f.matmul_tn(da, dw)
        elif c["op"] == "nt":
            out, ga, gb = f.matmul_nt(da, db), f.matmul(dw, db), f.matmul_tn(dw, da)
        else:
            out, ga, gb = f.matmul_tn(da, db), f.matmul_nt(db, dw), f.matmul(da, dw)
        k = a.shape[-1] if c["op"] != "tn" else a.shape[-2]
        for got, want, what in ((out, c["c"], "forward"), (ga, c["grad_a"], "grad0"),
                                (gb, c["grad_b"], "grad1")):
            reference_assert_close(want, _host(got), what=f"{c['name']} {what}")
            check_tf32_parity(_host(got), want, k, a, b, what=f"{c['name']} {what}")


# --------------------------------------------------------------------- shape sweeps ---

ALIGNED = [  # (m, n, k, batch) -- operands meet TMA alignment: tensor-core path
    (128, 128, 32, 0), (128, 256, 512, 0), (256, 512, 256, 0), (1000, 776, 516, 0),
    (100, 60, 36, 0), (4, 8, 4, 0), (4, 4, 4, 0), (132, 260, 36, 0), (512, 256, 784, 0),
    (640, 1024, 1024, 0), (128, 128, 32, 5), (128, 32, 128, 7), (96, 40, 72, 3), (300, 132, 68, 2),
]
RAGGED = [  # leading dimensions not multiples of 4 floats: SIMT path
    (3, 5, 4, 0), (33, 17, 9, 0), (130, 67, 45, 0), (7, 3, 5, 4), (65, 129, 31, 2), (1, 1, 1, 0),
]


@pytest.mark.parametrize("policy", [3, 4])      # 3: single-CTA tiles, 4: CTA-pair tiles
@pytest.mark.parametrize("layout", [NN, NT, TN])
@pytest.mark.parametrize("shape", ALIGNED)
def test_tensor_core_path_matches_oracle(gpu, layout, shape, policy):
    f = gpu
    m, n, k, batch = shape
    rng = np.random.default_rng(1000 + 7 * layout + m + n + k)
    sa, sb = _shapes(layout, m, n, k, batch)
    a = rng.standard_normal(sa, dtype=np.float32)
    b = rng.standard_normal(sb, dtype=np.float32)
    f.set_policy(policy, 0, 0)     # that tensor-core kernel or fail
    try:
        got = _gpu_fn(f, layout)(_dev(a), _dev(b))
    finally:
        f.set_policy(0, 0, 0)
    assert f.last_path()["path"] == policy - 1
    check_tf32_parity(_host(got), _oracle(layout, a, b), k, a, b, what=f"L{layout} {shape}")


WIDE = [(512, 1024, 256, 0), (300, 1100, 132, 0), (256, 512, 64, 3), (1000, 776, 516, 0), (640, 2048, 1056, 0)]


@pytest.mark.parametrize("layout", [NN, NT, TN])
@pytest.mark.parametrize("shape", WIDE)
def test_wide_pair_tiles_match_oracle(gpu, layout, shape):
    """256 x 512 tiles on CTA pairs: two MMA groups per A stage, one accumulator set over all 512
    tensor-memory columns; ragged M, N (last tile half empty) and K, batched, with a K split."""
    f = gpu
    m, n, k, batch = shape
    rng = np.random.default_rng(3000 + 7 * layout + m + n + k)
    sa, sb = _shapes(layout, m, n, k, batch)
    a = rng.standard_normal(sa, dtype=np.float32)
    b = rng.standard_normal(sb, dtype=np.float32)
    want = _oracle(layout, a, b)
    for split in (1, 3):
        f.set_policy(4, 512, split)
        try:
            got = _gpu_fn(f, layout)(_dev(a), _dev(b))
        finally:
            f.set_policy(0, 0, 0)
        lp = f.last_path()
        assert lp["path"] == 3 and lp["block_n"] == 512, lp
        check_tf32_parity(_host(got), want, k, a, b, what=f"wide L{layout} {shape} split {split}")
    assert f.device_status() == 0


def test_wide_pair_tiles_with_bias_and_gelu(gpu):
    f = gpu
    m, n, k = 768, 1536, 512
    rng = np.random.default_rng(11)
    a = rng.standard_normal((m, k), dtype=np.float32)
    b = rng.standard_normal((k, n), dtype=np.float32)
    bias = rng.standard_normal(n, dtype=np.float32)
    f.set_policy(4, 512, 1)
    try:
        got = f.linear_forward(_dev(a), _dev(b), _dev(bias), act=f.ACT_GELU, layout=f.NN)
    finally:
        f.set_policy(0, 0, 0)
    assert f.last_path()["block_n"] == 512
    want = oracle.bias_act(oracle.matmul(a, b), bias, oracle.ACT_GELU)
    assert np.abs(_host(got) - want).max() <= 1e-2 * np.sqrt(k) * np.abs(a).max() * np.abs(b).max()
    assert f.device_status() == 0


@pytest.mark.parametrize("layout", [NN, NT, TN])
@pytest.mark.parametrize("shape", RAGGED + ALIGNED[:6])
def test_simt_path_matches_oracle(gpu, layout, shape):
    f = gpu
    m, n, k, batch = shape
    rng = np.random.default_rng(2000 + 7 * layout + m + n + k)
    sa, sb = _shapes(layout, m, n, k, batch)
    a = rng.standard_normal(sa, dtype=np.float32)
    b = rng.standard_normal(sb, dtype=np.float32)
    f.set_policy(1, 0, 0)
    try:
        got = _gpu_fn(f, layout)(_dev(a), _dev(b))
    finally:
        f.set_policy(0, 0, 0)
    assert f.last_path()["path"] == 1
    want = _oracle(layout, a, b)
    check_tf32_parity(_host(got), want, k, a, b, what=f"L{layout} {shape}")
    # the SIMT path is FP32 throughout: far tighter than the TF32 bound
    assert np.abs(_host(got) - want).max() <= 1e-5 * max(k, 1) * np.abs(a).max() * np.abs(b).max()


@pytest.mark.parametrize("layout", [NN, NT, TN])
def test_automatic_dispatch_picks_the_path_by_alignment(gpu, layout):
    f = gpu
    rng = np.random.default_rng(5)
    for (m, n, k), want_path in (((64, 64, 64), 2), ((63, 65, 61), 1)):
        sa, sb = _shapes(layout, m, n, k, 0)
        a = rng.standard_normal(sa, dtype=np.float32)
        b = rng.standard_normal(sb, dtype=np.float32)
        got = _gpu_fn(f, layout)(_dev(a), _dev(b))
        assert f.last_path()["path"] == want_path
        check_tf32_parity(_host(got), _oracle(layout, a, b), k, a, b)


@pytest.mark.parametrize("block_n", [32, 64, 96, 128, 160, 192, 224, 256])
@pytest.mark.parametrize("layout", [NN, NT, TN])
def test_every_tile_width(gpu, layout, block_n):
    f = gpu
    m, n, k = 260, 520, 200
    rng = np.random.default_rng(block_n + layout)
    sa, sb = _shapes(layout, m, n, k, 0)
    a = rng.standard_normal(sa, dtype=np.float32)
    b = rng.standard_normal(sb, dtype=np.float32)
    da, db = _dev(a), _dev(b)
    want = _oracle(layout, a, b)
    for policy in ([3, 4] if block_n % 64 == 0 else [3]):    # pair tiles come in multiples of 64
        f.set_policy(policy, block_n, 1)
        try:
            got = _gpu_fn(f, layout)(da, db)
        finally:
            f.set_policy(0, 0, 0)
        assert f.last_path()["block_n"] == block_n and f.last_path()["path"] == policy - 1
        check_tf32_parity(_host(got), want, k, a, b)


@pytest.mark.parametrize("split_k", [2, 3, 8, 64])
@pytest.mark.parametrize("layout", [NN, NT, TN])
def test_split_k_is_exact_in_structure_and_deterministic(gpu, layout, split_k):
    f = gpu
    m, n, k = 256, 264, 2052
    rng = np.random.default_rng(split_k + layout)
    sa, sb = _shapes(layout, m, n, k, 2)
    a = rng.standard_normal(sa, dtype=np.float32)
    b = rng.standard_normal(sb, dtype=np.float32)
    da, db = _dev(a), _dev(b)
    want = _oracle(layout, a, b)
    for policy in (3, 4):
        f.set_policy(policy, 128, split_k)
        try:
            got1 = _host(_gpu_fn(f, layout)(da, db))
            assert f.last_path()["split_k"] > 1 and f.last_path()["path"] == policy - 1
            got2 = _host(_gpu_fn(f, layout)(da, db))
        finally:
            f.set_policy(0, 0, 0)
        assert np.array_equal(got1, got2), "split-K reduction must not depend on CTA arrival order"
        check_tf32_parity(got1, want, k, a, b)


@pytest.mark.parametrize("layout", [NN, NT, TN])
@pytest.mark.parametrize("k,split_k", [(2052, 3), (1000, 1), (288, 1), (8192, 5)])
def test_pair_kernel_two_k_blocks_per_stage(gpu, layout, k, split_k):
    """256 x 256 CTA-pair tiles take two 32-deep k-blocks per pipeline stage once a unit has at
    least eight of them; odd block counts and split boundaries leave a half-filled stage."""
    f = gpu
    m, n = 520, 512
    rng = np.random.default_rng(k + split_k + layout)
    sa, sb = _shapes(layout, m, n, k, 0)
    a = rng.standard_normal(sa, dtype=np.float32)
    b = rng.standard_normal(sb, dtype=np.float32)
    f.set_policy(4, 256, split_k)
    try:
        got = _host(_gpu_fn(f, layout)(_dev(a), _dev(b)))
    finally:
        f.set_policy(0, 0, 0)
    lp = f.last_path()
    assert lp["path"] == 3 and lp["block_n"] == 256 and lp["split_k"] == split_k
    check_tf32_parity(got, _oracle(layout, a, b), k, a, b)


def test_skinny_output_takes_split_k_automatically(gpu):
    f = gpu
    rng = np.random.default_rng(9)
    k, m, n = 8192, 256, 256            # dW = X^T . dY of the transformer config
    x = rng.standard_normal((k, m), dtype=np.float32)
    dy = (rng.standard_normal((k, n)) * 1e-3).astype(np.float32)
    got = f.matmul_tn(_dev(x), _dev(dy))
    assert f.last_path()["split_k"] > 1
    check_tf32_parity(_host(got), oracle.matmul_tn(x, dy), k, x, dy)


# ------------------------------------------------------------ buffers and the general entry ---

def test_output_is_fully_overwritten_and_nothing_else_is_touched(gpu):
    """Recycled (dirty) output buffers are legal inputs; rows beyond C must stay untouched."""
    import torch
    f = gpu
    rng = np.random.default_rng(4)
    for layout in (NN, NT, TN):
        for (m, n, k) in ((130, 72, 40), (3, 5, 4)):
            sa, sb = _shapes(layout, m, n, k, 0)
            a = rng.standard_normal(sa, dtype=np.float32)
            b = rng.standard_normal(sb, dtype=np.float32)
            guard = 64
            buf = torch.full((m * n + 2 * guard,), float("nan"), device="cuda")
            out = buf[guard:guard + m * n].view(m, n)   # 256-byte offset keeps 16-byte alignment
            _gpu_fn(f, layout)(_dev(a), _dev(b), out=out)
            h = _host(buf)
            assert np.isnan(h[:guard]).all() and np.isnan(h[-guard:]).all()
            check_tf32_parity(h[guard:-guard].reshape(m, n), _oracle(layout, a, b), k, a, b)


@pytest.mark.parametrize("layout", [NN, NT, TN])
@pytest.mark.parametrize("aligned", [True, False])
def test_general_entry_alpha_beta_strides(gpu, layout, aligned):
    """fastnn_b200_gemm_ex with padded leading dimensions, batch strides, alpha and beta."""
    import torch
    f = gpu
    m, n, k, batch = (72, 40, 36, 3) if aligned else (71, 39, 35, 3)
    pad = 4 if aligned else 3
    rng = np.random.default_rng(12 + layout)
    ra, ca = (k, m) if layout == TN else (m, k)
    rb, cb = (n, k) if layout == NT else (k, n)
    A = rng.standard_normal((batch, ra, ca + pad), dtype=np.float32)
    B = rng.standard_normal((batch, rb, cb + pad), dtype=np.float32)
    C0 = rng.standard_normal((batch, m, n + pad), dtype=np.float32)
    alpha, beta = 0.75, -1.5
    dA, dB, dC = _dev(A), _dev(B), _dev(C0)
    f.gemm_ex(layout, dA.data_ptr(), dB.data_ptr(), dC.data_ptr(), m, n, k, batch,
              ca + pad, cb + pad, n + pad, ra * (ca + pad), rb * (cb + pad), m * (n + pad),
              alpha, beta)
    torch.cuda.synchronize()
    assert f.last_path()["path"] in ((2, 3) if aligned else (1,))
    got = _host(dC)
    a, b = np.ascontiguousarray(A[..., :ca]), np.ascontiguousarray(B[..., :cb])
    prod = _oracle(layout, a, b)
    want = alpha * prod.astype(np.float64) + beta * C0[..., :n].astype(np.float64)
    assert np.array_equal(got[..., n:], C0[..., n:]), "padding columns of C were written"
    err = np.abs(got[..., :n] - want)
    assert err.max() <= 1e-2 * np.sqrt(k) * np.abs(a).max() * np.abs(b).max()
    assert np.linalg.norm(err) / np.linalg.norm(want) <= 5e-3


def test_beta_with_nan_in_c_is_ignored_when_beta_is_zero(gpu):
    import torch
    f = gpu
    rng = np.random.default_rng(8)
    a = rng.standard_normal((64, 32), dtype=np.float32)
    b = rng.standard_normal((32, 48), dtype=np.float32)
    out = torch.full((64, 48), float("nan"), device="cuda")
    f.cuda_matmul(_dev(a), _dev(b), 64, 48, 32, out=out, alpha=1.0, beta=0.0)
    assert np.isfinite(_host(out)).all()


def test_k_zero_and_empty(gpu):
    import torch
    f = gpu
    a = torch.empty((5, 0), device="cuda")
    b = torch.empty((0, 8), device="cuda")
    out = torch.full((5, 8), 3.0, device="cuda")
    f.cuda_matmul(a, b, 5, 8, 0, out=out)
    assert (_host(out) == 0).all()
    e = f.matmul(torch.empty((0, 4), device="cuda"), torch.empty((4, 8), device="cuda"))
    assert tuple(e.shape) == (0, 8)


def test_uninitialised_device_and_bad_arguments_return_errors(gpu):
    f = gpu
    lib = f.lib()
    p = ctypes.c_void_p(256)
    assert lib.fastnn_cuda_matmul(p, p, p, 4, 4, 4, 3, 4, 4, 1.0, 0.0) == -1       # lda < k
    assert lib.fastnn_b200_gemm_ex(3, p, p, p, 4, 4, 4, 1, 4, 4, 4, 16, 16, 16, 1.0, 0.0, None, 0,
                                   None) == -1
    assert lib.fastnn_cuda_matmul(None, p, p, 4, 4, 4, 4, 4, 4, 1.0, 0.0) == -1    # null operand
    f.set_policy(2, 0, 0)
    try:   # tensor-core-only policy refuses operands TMA cannot address instead of falling back
        assert lib.fastnn_cuda_matmul_nt(p, p, p, 3, 5, 3) == -1
    finally:
        f.set_policy(0, 0, 0)


# ----------------------------------------------------------------------- fused Linear ---

@pytest.mark.parametrize("act", [0, 1, 2])
@pytest.mark.parametrize("layout", [NT, NN])
@pytest.mark.parametrize("shape", [(512, 784, 256), (37, 20, 12), (33, 19, 7), (200, 2048, 132)])
def test_fused_linear_matches_linear_forward(gpu, layout, act, shape):
    """Linear::forward (+relu/gelu) = transpose + matmul + expand + add (+act) in the reference;
    one launch here.  Includes a split-K case (bias/activation applied by the reduce pass)."""
    f = gpu
    rows, in_f, out_f = shape
    rng = np.random.default_rng(rows + act)
    x = rng.random((rows, in_f), dtype=np.float32)                       # U(0,1), pixel-like
    bound = np.sqrt(6.0 / in_f)
    w = rng.uniform(-bound, bound, (out_f, in_f)).astype(np.float32)     # kaiming_uniform
    bias = rng.uniform(-1 / np.sqrt(in_f), 1 / np.sqrt(in_f), out_f).astype(np.float32)
    want = oracle.linear(x, w, bias, act)
    wd = _dev(w) if layout == NT else _dev(np.ascontiguousarray(w.T))
    got = f.linear_forward(_dev(x), wd, _dev(bias), act=act, layout=layout)
    pre = oracle.linear(x, w, bias, 0)
    # activation is 1-Lipschitz, so the pre-activation bound carries over
    err = np.abs(_host(got) - want)
    assert err.max() <= 1e-2 * np.sqrt(in_f) * np.abs(x).max() * np.abs(w).max()
    assert np.linalg.norm(err) / max(np.linalg.norm(pre), 1e-30) <= 5e-3
    nobias = f.linear_forward(_dev(x), wd, None, act=0, layout=layout)
    check_tf32_parity(_host(nobias), oracle.linear(x, w, None, 0), in_f, x, w)


# ------------------------------------------------------------------ configured shapes ---

def test_config_mnist_mlp_layer1(gpu):
    f = gpu
    rng = np.random.default_rng(0)
    a = rng.random((512, 784), dtype=np.float32)
    bound = np.sqrt(6.0 / 784)
    b = rng.uniform(-bound, bound, (784, 256)).astype(np.float32)
    bias = rng.uniform(-1 / 28, 1 / 28, 256).astype(np.float32)
    got = f.linear_forward(_dev(a), _dev(b), _dev(bias), act=0, layout=NN)
    want = oracle.bias_act(oracle.matmul(a, b), bias, 0)
    check_tf32_parity(_host(got), want, 784, a, b)


@pytest.mark.parametrize("kn", [(256, 768), (256, 256), (256, 1024), (1024, 256)])
def test_config_char_lm_forward_and_backward_gemms(gpu, kn):
    f = gpu
    k, n = kn
    m = 8192
    t = oracle.host_threads()
    rng = np.random.default_rng(2000 + k + n)
    x = rng.standard_normal((m, k), dtype=np.float32)
    w = (rng.standard_normal((k, n)) * 0.02).astype(np.float32)
    dy = (rng.standard_normal((m, n)) * 1e-3).astype(np.float32)
    dx, dw_, ddy = _dev(x), _dev(w), _dev(dy)
    check_tf32_parity(_host(f.matmul(dx, dw_)), oracle.matmul(x, w, threads=t), k, x, w, "fwd NN")
    wt = oracle.transpose(w)
    check_tf32_parity(_host(f.matmul_nt(ddy, dw_)), oracle.matmul(dy, wt, threads=t), n, dy, w,
                      "dX = dY.W^T")
    xt = oracle.transpose(x)
    check_tf32_parity(_host(f.matmul_tn(dx, ddy)), oracle.matmul(xt, dy, threads=t), m, x, dy,
                      "dW = X^T.dY")


def test_config_batched_attention_matmuls(gpu):
    f = gpu
    bh, t, d = 512, 128, 32
    rng = np.random.default_rng(3000)
    q = rng.standard_normal((bh, t, d), dtype=np.float32)
    kk = rng.standard_normal((bh, t, d), dtype=np.float32)
    v = rng.standard_normal((bh, t, d), dtype=np.float32)
    s_want = oracle.matmul_nt(q, kk)
    s_got = f.matmul_nt(_dev(q), _dev(kk))
    check_tf32_parity(_host(s_got), s_want, d, q, kk, "S = Q.K^T")
    p = oracle.causal_softmax(s_want, 1.0 / np.sqrt(d))
    o_got = f.matmul(_dev(p), _dev(v))
    check_tf32_parity(_host(o_got), oracle.matmul(p, v), t, p, v, "O = P.V")
