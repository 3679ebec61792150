"""GPU: the fused backward epilogue -- dx = (dy . W) * act'(pre) and its sum over rows -- against
the CPU composition FastNN's tape runs (matmul_nt -> ReluBackward / GeluBackward -> row sum behind
the bias expand; src/autograd/backward_ops.rs:136-160, 194-218, src/nn/linear.rs:78-82).

Tolerance: the GEMM bar on dx (relative Frobenius <= 5e-3, max-abs <= 1e-2 sqrt(K) max|dy| max|W|;
|act'| <= 1.13 so the mask does not widen it).  The bias gradient adds `rows` such values per
column: relative Frobenius <= 5e-3 against its own norm, max-abs <= rows x the element bound."""
import ctypes

import numpy as np
import pytest

import oracle

pytestmark = pytest.mark.gpu

ACTS = {"none": 0, "relu": 1, "gelu": 2}


def _inputs(rows, out_f, in_f, seed):
    rng = np.random.default_rng(seed)
    dy = rng.standard_normal((rows, out_f), dtype=np.float32)
    w = (rng.standard_normal((out_f, in_f), dtype=np.float32) * 0.5).astype(np.float32)
    pre = rng.standard_normal((rows, in_f), dtype=np.float32)
    return dy, w, pre


def _check(dx, db, want_dx, want_db, dy, w, k, rows, what):
    bound = 1e-2 * np.sqrt(max(k, 1)) * np.abs(dy).max() * np.abs(w).max() * 1.13
    err = dx.astype(np.float64) - want_dx
    assert np.isfinite(dx).all(), what
    if np.linalg.norm(want_dx) > 0:
        assert np.linalg.norm(err) / np.linalg.norm(want_dx) <= 5e-3, what
    assert np.abs(err).max() <= bound, what
    if db is not None:
        e2 = db.astype(np.float64) - want_db
        assert np.isfinite(db).all(), what
        if np.linalg.norm(want_db) > 0:
            assert np.linalg.norm(e2) / np.linalg.norm(want_db) <= 5e-3, what + " bias_grad"
        assert np.abs(e2).max() <= rows * bound, what + " bias_grad"


@pytest.mark.parametrize("act", ["none", "relu", "gelu"])
@pytest.mark.parametrize("shape", [
    (256, 128, 256),        # whole tiles
    (1000, 96, 200),        # ragged rows and columns (TMA clipping, partial slabs)
    (33, 64, 32),           # two slabs, the second with one row
    (8192, 1024, 256),      # ff2 backward of the configured transformer block
    (640, 36, 260),         # several tile columns, short K
])
def test_backward_input_matches_the_tape_composition(gpu, shape, act):
    import torch
    f = gpu
    rows, out_f, in_f = shape
    dy, w, pre = _inputs(rows, out_f, in_f, rows + out_f + in_f + ACTS[act])
    want_dx, want_db = oracle.linear_backward_input(dy, w, pre if act != "none" else None, ACTS[act])
    dx, db = f.linear_backward_input(torch.from_numpy(dy).cuda(), torch.from_numpy(w).cuda(),
                                     torch.from_numpy(pre).cuda(), act=ACTS[act], bias_grad=True)
    torch.cuda.synchronize()
    assert f.last_path()["path"] in (2, 3) and f.last_path()["split_k"] == 1
    _check(dx.cpu().numpy(), db.cpu().numpy(), want_dx, want_db, dy, w, out_f, rows, f"{shape} {act}")
    assert f.device_status() == 0


def test_backward_input_nt_layout_and_no_bias_grad(gpu):
    """NT takes the transposed weight copy [in,out]; without bias_grad nothing but dx is written."""
    import torch
    f = gpu
    dy, w, pre = _inputs(512, 192, 320, 77)
    want_dx, _ = oracle.linear_backward_input(dy, w, pre, 2)
    wt = torch.from_numpy(np.ascontiguousarray(w.T)).cuda()
    dx = f.linear_backward_input(torch.from_numpy(dy).cuda(), wt, torch.from_numpy(pre).cuda(),
                                 act=2, layout=f.NT)
    _check(dx.cpu().numpy(), None, want_dx, None, dy, w, 192, 512, "NT gelu")


def test_backward_input_is_deterministic_and_ignores_dirty_outputs(gpu):
    import torch
    f = gpu
    dy, w, pre = _inputs(2048, 256, 512, 5)
    a = [torch.from_numpy(x).cuda() for x in (dy, w, pre)]
    out = torch.full((2048, 512), float("nan"), device="cuda")
    dx1, db1 = f.linear_backward_input(a[0], a[1], a[2], act=1, bias_grad=True, out=out)
    dx1, db1 = dx1.clone(), db1.clone()
    dx2, db2 = f.linear_backward_input(a[0], a[1], a[2], act=1, bias_grad=True)
    assert torch.equal(dx1, dx2) and torch.equal(db1, db2)
    # ReLU mask is exact: zero wherever pre <= 0
    assert (dx1[a[2] <= 0] == 0).all()


def test_backward_input_on_both_tensor_core_kernels_and_the_simt_fallback(gpu):
    import torch
    f = gpu
    dy, w, pre = _inputs(1024, 512, 512, 9)
    want_dx, want_db = oracle.linear_backward_input(dy, w, pre, 2)
    t = [torch.from_numpy(x).cuda() for x in (dy, w, pre)]
    try:
        for policy, path in ((3, 2), (4, 3), (1, 1)):
            f.set_policy(policy, 0, 0)
            dx, db = f.linear_backward_input(t[0], t[1], t[2], act=2, bias_grad=True)
            assert f.last_path()["path"] == path
            _check(dx.cpu().numpy(), db.cpu().numpy(), want_dx, want_db, dy, w, 512, 1024, f"policy {policy}")
    finally:
        f.set_policy(0, 0, 0)
    # operands TMA cannot address (odd leading dimension) take the SIMT kernel + two small passes
    dy, w, pre = _inputs(70, 33, 45, 11)
    want_dx, want_db = oracle.linear_backward_input(dy, w, pre, 1)
    dx, db = f.linear_backward_input(torch.from_numpy(dy).cuda(), torch.from_numpy(w).cuda(),
                                     torch.from_numpy(pre).cuda(), act=1, bias_grad=True)
    assert f.last_path()["path"] == 1
    _check(dx.cpu().numpy(), db.cpu().numpy(), want_dx, want_db, dy, w, 33, 70, "simt")


def test_backward_input_argument_errors_and_empty_shapes(gpu):
    import torch
    f = gpu
    lib = f.lib()
    t = torch.zeros(64 * 64, device="cuda")
    p, null = ctypes.c_void_p(t.data_ptr()), ctypes.c_void_p(0)
    assert lib.fastnn_b200_linear_backward_input(2, p, p, p, 8, 8, 8, 0, null, null, None) == -1   # TN
    assert lib.fastnn_b200_linear_backward_input(0, p, p, p, 8, 8, 8, 3, p, null, None) == -1      # act
    assert lib.fastnn_b200_linear_backward_input(0, p, p, p, 8, 8, 8, 2, null, null, None) == -1   # no pre
    assert lib.fastnn_b200_linear_backward_input(0, p, p, p, -1, 8, 8, 0, null, null, None) == -1
    db = torch.full((8,), 7.0, device="cuda")
    assert lib.fastnn_b200_linear_backward_input(0, p, p, p, 0, 8, 8, 0, null,
                                                 ctypes.c_void_p(db.data_ptr()), None) == 0
    torch.cuda.synchronize()
    assert (db == 0).all()                       # no rows: the bias gradient is zero
