"""GPU: the fused epilogue's activation, isolated from TF32 rounding.

Operands are small integers times powers of two, so every product and every partial sum is exact
in TF32 x TF32 -> FP32: the GEMM result equals the oracle's bit for bit and whatever differs
afterwards is the bias add and the activation alone.  ReLU must then be bit-exact and erf-GELU
within 1e-6 * max(1, |x|) of the oracle's (libm erff against the device's erff: a few ulp), on each
of the three epilogues an activation can run in: the by-column drain of the persistent kernels,
the split-K reduce pass, and the in-cluster reduction."""
import numpy as np
import pytest

import oracle

pytestmark = pytest.mark.gpu

NN = 0
ACT_NONE, ACT_RELU, ACT_GELU = 0, 1, 2


def _exact_operands(m, n, k, seed):
    rng = np.random.default_rng(seed)
    a = (rng.integers(-8, 9, size=(m, k)).astype(np.float32)) * np.float32(0.125)
    b = (rng.integers(-8, 9, size=(k, n)).astype(np.float32)) * np.float32(0.0625)
    bias = (rng.integers(-16, 17, size=n).astype(np.float32)) * np.float32(0.25)
    return a, b, bias


# (policy, block_n, split_k, expected path): which epilogue applies the activation
PATHS = {
    "by_column_single_cta": (3, 0, 1, 2),
    "by_column_cta_pair": (4, 0, 1, 3),
    "splitk_reduce_pass": (3, 128, 4, 2),
    "cluster_reduction": (5, 64, 4, 6),
}


@pytest.mark.parametrize("path", sorted(PATHS))
@pytest.mark.parametrize("act", [ACT_NONE, ACT_RELU, ACT_GELU])
def test_activation_is_exact_on_every_epilogue(gpu, path, act):
    import torch
    f = gpu
    policy, block_n, split_k, want_path = PATHS[path]
    m, n, k = 512, 256, 1024
    a, b, bias = _exact_operands(m, n, k, 17)
    pre = oracle.matmul(a, b)
    # the premise: the pre-activation is exact (integers / 128, |sum| < 2^24 / 128)
    assert np.array_equal(pre.astype(np.float64), a.astype(np.float64) @ b.astype(np.float64))
    want = oracle.bias_act(pre, bias, act)
    f.set_policy(policy, block_n, split_k)
    try:
        got = f.linear_forward(torch.from_numpy(a).cuda(), torch.from_numpy(b).cuda(),
                               torch.from_numpy(bias).cuda(), act=act, layout=NN)
    finally:
        f.set_policy(0, 0, 0)
    lp = f.last_path()
    assert lp["path"] == want_path and lp["split_k"] == split_k, (path, lp)
    got = got.cpu().numpy()
    if act != ACT_GELU:
        assert np.array_equal(got, want), f"{path}: act {act} must be bit-exact on exact operands"
    else:
        x = pre + bias
        tol = 1e-6 * np.maximum(1.0, np.abs(x))
        bad = np.abs(got.astype(np.float64) - want) > tol
        assert not bad.any(), (path, float(np.abs(got - want).max()))
    assert f.device_status() == 0


def test_gelu_is_the_same_function_on_every_epilogue(gpu):
    """One erf-GELU behind act = 2, whichever kernel the planner picks: identical bits."""
    import torch
    f = gpu
    a, b, bias = _exact_operands(512, 256, 1024, 23)
    da, db, dbias = (torch.from_numpy(t).cuda() for t in (a, b, bias))
    outs = {}
    for path, (policy, block_n, split_k, _) in PATHS.items():
        f.set_policy(policy, block_n, split_k)
        try:
            outs[path] = f.linear_forward(da, db, dbias, act=ACT_GELU, layout=NN).cpu().numpy()
        finally:
            f.set_policy(0, 0, 0)
    first = outs["by_column_single_cta"]
    for path, got in outs.items():
        assert np.array_equal(got, first), path


def test_gelu_derivative_matches_the_oracle_on_exact_operands(gpu):
    """linear_backward_input's epilogue: (dy . W) * gelu'(pre) with an exact product."""
    import torch
    f = gpu
    rows, out_f, in_f = 256, 128, 192
    rng = np.random.default_rng(29)
    dy = rng.integers(-8, 9, size=(rows, out_f)).astype(np.float32) * np.float32(0.125)
    w = rng.integers(-8, 9, size=(out_f, in_f)).astype(np.float32) * np.float32(0.0625)
    pre = (rng.standard_normal((rows, in_f)) * 2.0).astype(np.float32)
    want_dx, want_db = oracle.linear_backward_input(dy, w, pre, ACT_GELU)
    dx, db = f.linear_backward_input(torch.from_numpy(dy).cuda(), torch.from_numpy(w).cuda(),
                                     torch.from_numpy(pre).cuda(), act=ACT_GELU, bias_grad=True)
    g = oracle.matmul(dy, w)
    tol = 2e-6 * np.maximum(1.0, np.abs(g))                 # derivative in [-0.13, 1.13], few ulp off
    assert (np.abs(dx.cpu().numpy().astype(np.float64) - want_dx) <= tol).all()
    assert np.abs(db.cpu().numpy() - want_db).max() <= 1e-4 * rows
