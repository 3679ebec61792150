"""GPU parity tests for the cluster form of split-K: the K slices of one output tile run as the
CTAs of a thread-block cluster and add their partial tiles through distributed shared memory
(no workspace, no reduce launch).  Policy 5 forces it with split_k as the cluster size; the
checker is the CPU oracle on identical inputs, at the TF32 tolerance of the other GEMM tests,
and the workspace form of the same split (policy 3) as a second comparator.
"""
import ctypes

import numpy as np
import pytest

import oracle
from helpers import check_tf32_parity

pytestmark = pytest.mark.gpu

NN, NT, TN = 0, 1, 2
CLUSTER_PATH = 6


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


@pytest.mark.parametrize("cluster", [2, 4, 8, 16])
@pytest.mark.parametrize("layout", [NN, NT, TN])
@pytest.mark.parametrize("shape", [(512, 256, 784, 0, 64), (256, 264, 2052, 2, 128), (100, 60, 1028, 0, 32),
                                   (132, 260, 516, 3, 96), (384, 512, 4096, 0, 256)])
def test_cluster_split_k_matches_oracle_and_is_deterministic(gpu, layout, cluster, shape):
    f = gpu
    m, n, k, batch, block_n = shape
    rng = np.random.default_rng(cluster * 100 + layout * 10 + m)
    sa, sb = _shapes(layout, m, n, k, batch)
    a = rng.standard_normal(sa, dtype=np.float32)
    b = rng.standard_normal(sb, dtype=np.float32)
    da, db = _dev(a), _dev(b)
    f.set_policy(5, block_n, cluster)
    try:
        got1 = _host(_gpu_fn(f, layout)(da, db))
        lp = f.last_path()
        got2 = _host(_gpu_fn(f, layout)(da, db))
    finally:
        f.set_policy(0, 0, 0)
    if cluster == 16 and lp["path"] == 2:
        pytest.skip("this device places no clusters of 16 CTAs (beyond the portable size of 8)")
    assert lp["path"] == CLUSTER_PATH and lp["split_k"] == cluster and lp["block_n"] == block_n
    assert lp["num_ctas"] % cluster == 0
    assert np.array_equal(got1, got2), "the cluster reduction adds slices in a fixed order"
    check_tf32_parity(got1, _oracle(layout, a, b), k, a, b)
    assert f.device_status() == 0


def test_cluster_split_k_against_the_workspace_form(gpu):
    """Same split, same slice boundaries (K a multiple of 32 * split), same order of additions:
    the two forms of split-K give the same bits."""
    f = gpu
    m, n, k, split = 256, 384, 4096, 4
    rng = np.random.default_rng(77)
    a = rng.standard_normal((m, k), dtype=np.float32)
    b = rng.standard_normal((k, n), dtype=np.float32)
    da, db = _dev(a), _dev(b)
    try:
        f.set_policy(5, 128, split)
        c_cluster = _host(f.matmul(da, db))
        assert f.last_path()["path"] == CLUSTER_PATH
        f.set_policy(3, 128, split)
        c_workspace = _host(f.matmul(da, db))
        assert f.last_path()["path"] == 2 and f.last_path()["split_k"] == split
    finally:
        f.set_policy(0, 0, 0)
    assert np.array_equal(c_cluster, c_workspace)


@pytest.mark.parametrize("act", [0, 1, 2])
@pytest.mark.parametrize("layout", [NT, NN])
@pytest.mark.parametrize("shape", [(512, 784, 256), (200, 2048, 132), (37, 260, 13)])
def test_cluster_split_k_carries_the_linear_epilogue(gpu, layout, act, shape):
    """Linear::forward (src/nn/linear.rs:55-88) + ReLU / erf-GELU with the bias and activation
    applied by the cluster's reduction; n = 13 takes the scalar stores."""
    f = gpu
    rows, in_f, out_f = shape
    rng = np.random.default_rng(rows + act)
    x = rng.random((rows, in_f), dtype=np.float32)
    bound = np.sqrt(6.0 / in_f)
    w = rng.uniform(-bound, bound, (out_f, in_f)).astype(np.float32)
    bias = rng.uniform(-1 / np.sqrt(in_f), 1 / np.sqrt(in_f), out_f).astype(np.float32)
    want = oracle.linear(x, w, bias, act)
    pre = oracle.linear(x, w, bias, 0)
    if layout == NN and out_f % 4 != 0:
        pytest.skip("row stride of W [in, out] not a multiple of 4 floats: SIMT path")
    wd = _dev(w) if layout == NT else _dev(np.ascontiguousarray(w.T))
    f.set_policy(5, 0, 4)
    try:
        got = f.linear_forward(_dev(x), wd, _dev(bias), act=act, layout=layout)
        assert f.last_path()["path"] == CLUSTER_PATH
    finally:
        f.set_policy(0, 0, 0)
    err = np.abs(_host(got) - want)
    assert err.max() <= 1e-2 * np.sqrt(in_f) * np.abs(x).max() * np.abs(w).max()
    assert np.linalg.norm(err) / max(np.linalg.norm(pre), 1e-30) <= 5e-3


def test_cluster_split_k_alpha_beta_and_strided_c(gpu):
    """C = alpha * A.B + beta * C into a strided, dirty C through the general entry."""
    import torch
    f = gpu
    m, n, k, ldc = 200, 136, 1024, 160
    rng = np.random.default_rng(5)
    a = rng.standard_normal((m, k), dtype=np.float32)
    b = rng.standard_normal((k, n), dtype=np.float32)
    c0 = rng.standard_normal((m, ldc), dtype=np.float32)
    da, db, dc = _dev(a), _dev(b), _dev(c0)
    f.set_policy(5, 64, 8)
    try:
        f.gemm_ex(NN, da.data_ptr(), db.data_ptr(), dc.data_ptr(), m, n, k, 1, k, n, ldc, 0, 0, 0,
                  alpha=0.5, beta=-2.0)
        assert f.last_path()["path"] == CLUSTER_PATH
    finally:
        f.set_policy(0, 0, 0)
    torch.cuda.synchronize()
    got = _host(dc)
    want = 0.5 * oracle.matmul(a, b) - 2.0 * c0[:, :n]
    assert np.array_equal(got[:, n:], c0[:, n:]), "columns past n must stay untouched"
    err = np.abs(got[:, :n] - want)
    assert err.max() <= 0.5 * 1e-2 * np.sqrt(k) * np.abs(a).max() * np.abs(b).max()


def test_cluster_split_k_falls_back_when_k_is_too_short(gpu):
    """Fewer 32-deep k-blocks than CTAs in the cluster: the workspace form of the split runs."""
    f = gpu
    rng = np.random.default_rng(6)
    a = rng.standard_normal((128, 96), dtype=np.float32)
    b = rng.standard_normal((96, 128), dtype=np.float32)
    f.set_policy(5, 128, 8)
    try:
        got = _host(f.matmul(_dev(a), _dev(b)))
        assert f.last_path()["path"] == 2
    finally:
        f.set_policy(0, 0, 0)
    check_tf32_parity(got, oracle.matmul(a, b), 96, a, b)


def test_mnist_layer_takes_the_cluster_form_by_default(gpu):
    """MNIST-MLP layer 1 (512 x 784 . 784 x 256 + bias): 8 output tiles of 128 x 128 for 148 SMs,
    so the planner cuts K; the cut is a cluster, not a workspace plus a second launch."""
    f = gpu
    rng = np.random.default_rng(0)
    a = rng.random((512, 784), dtype=np.float32)
    bound = np.sqrt(6.0 / 784)
    b = rng.uniform(-bound, bound, (784, 256)).astype(np.float32)
    bias = rng.uniform(-1 / 28, 1 / 28, 256).astype(np.float32)
    before = f.launch_count()
    got = f.linear_forward(_dev(a), _dev(b), _dev(bias), act=0, layout=NN)
    lp = f.last_path()
    assert lp["path"] == CLUSTER_PATH and f.launch_count() - before == 1, lp
    check_tf32_parity(_host(got), oracle.bias_act(oracle.matmul(a, b), bias, 0), 784, a, b)
