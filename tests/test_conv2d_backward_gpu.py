"""GPU: gradients of Conv2d against the CPU loops of Conv2dBackward
(src/autograd/backward_ops.rs:753-770).

Tolerance: the GEMM bar with the contraction length of each product: grad_input sums
Cout*KH*KW terms, grad_weight sums N*OH*OW terms; relative Frobenius <= 5e-3,
max-abs <= 1e-2 sqrt(K) max|a| max|b|."""
import ctypes

import numpy as np
import pytest

import oracle

pytestmark = pytest.mark.gpu


def _case(n, ci, co, h, w, kh, kw, stride, padding, seed):
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((n, ci, h, w), dtype=np.float32)
    wt = (rng.standard_normal((co, ci, kh, kw), dtype=np.float32) * 0.2).astype(np.float32)
    oh = (h + 2 * padding[0] - kh) // stride[0] + 1
    ow = (w + 2 * padding[1] - kw) // stride[1] + 1
    go = rng.standard_normal((n, co, oh, ow), dtype=np.float32)
    return x, wt, go


def _check(got, want, k, a, b, what):
    assert got.shape == want.shape, what
    assert np.isfinite(got).all(), what
    err = got.astype(np.float64) - want
    assert np.linalg.norm(err) / np.linalg.norm(want) <= 5e-3, what
    assert np.abs(err).max() <= 1e-2 * np.sqrt(k) * np.abs(a).max() * np.abs(b).max(), what


@pytest.mark.parametrize("cfg", [
    # n, ci, co, h, w, kh, kw, padding  (stride 1: both gradients)
    (2, 8, 16, 16, 16, 3, 3, (1, 1)),
    (3, 3, 12, 20, 18, 5, 3, (2, 0)),        # RGB input, rectangular kernel, uneven padding
    (4, 16, 32, 14, 14, 1, 1, (0, 0)),       # pointwise
    (2, 32, 24, 28, 28, 3, 3, (0, 0)),       # no padding: grad_input pads by kernel - 1
    (1, 4, 6, 9, 11, 3, 3, (2, 2)),          # padding = kernel - 1, the largest covered
])
def test_conv2d_gradients_match_the_cpu_loops(gpu, cfg):
    import torch
    f = gpu
    n, ci, co, h, w, kh, kw, padding = cfg
    x, wt, go = _case(n, ci, co, h, w, kh, kw, (1, 1), padding, sum(cfg[:7]))
    want_gi, want_gw = oracle.conv2d_backward(x, wt, go, (1, 1), padding)
    gi, gw = f.conv2d_backward(torch.from_numpy(x).cuda(), torch.from_numpy(wt).cuda(),
                               torch.from_numpy(go).cuda(), padding=padding)
    torch.cuda.synchronize()
    _check(gi.cpu().numpy(), want_gi, co * kh * kw, go, wt, f"grad_input {cfg}")
    _check(gw.cpu().numpy(), want_gw, n * go.shape[2] * go.shape[3], go, x, f"grad_weight {cfg}")
    assert f.device_status() == 0


def test_grad_weight_with_stride_and_through_the_reference_symbols(gpu):
    import torch
    f = gpu
    lib = f.lib()
    x, wt, go = _case(3, 6, 10, 15, 17, 3, 3, (2, 2), (1, 1), 77)
    _, want_gw = oracle.conv2d_backward(x, wt, go, (2, 2), (1, 1))
    xd, wd, gd = (torch.from_numpy(t).cuda() for t in (x, wt, go))
    gw = torch.full(wt.shape, float("nan"), device="cuda")
    vp = lambda t: ctypes.c_void_p(t.data_ptr())
    oh, ow = go.shape[2], go.shape[3]
    assert lib.fastnn_cuda_conv2d_backward_weight(vp(xd), vp(gd), vp(gw), 3, 6, 10, 15, 17, oh, ow, 3, 3,
                                                  2, 2, 1, 1) == 0
    torch.cuda.synchronize()
    _check(gw.cpu().numpy(), want_gw, 3 * oh * ow, go, x, "strided grad_weight")
    # grad_input: stride 2 is not covered; stride 1 through FastNN's own symbol is
    gi = torch.empty_like(xd)
    assert lib.fastnn_cuda_conv2d_backward_data(vp(gd), vp(wd), vp(gi), 3, 6, 10, 15, 17, oh, ow, 3, 3,
                                                2, 2, 1, 1) == -1
    x1, w1, g1 = _case(2, 6, 10, 12, 12, 3, 3, (1, 1), (1, 1), 78)
    want_gi, _ = oracle.conv2d_backward(x1, w1, g1, (1, 1), (1, 1))
    g1d, w1d = torch.from_numpy(g1).cuda(), torch.from_numpy(w1).cuda()
    gi1 = torch.full(x1.shape, float("nan"), device="cuda")
    assert lib.fastnn_cuda_conv2d_backward_data(vp(g1d), vp(w1d), vp(gi1), 2, 6, 10, 12, 12, 12, 12, 3, 3,
                                                1, 1, 1, 1) == 0
    torch.cuda.synchronize()
    _check(gi1.cpu().numpy(), want_gi, 90, g1, w1, "grad_input via the reference symbol")


def test_conv2d_gradients_are_deterministic_and_check_their_arguments(gpu):
    import torch
    f = gpu
    x, wt, go = _case(4, 8, 16, 12, 12, 3, 3, (1, 1), (1, 1), 5)
    t = [torch.from_numpy(a).cuda() for a in (x, wt, go)]
    a = f.conv2d_backward(*t, padding=(1, 1))
    b = f.conv2d_backward(*t, padding=(1, 1))
    assert torch.equal(a[0], b[0]) and torch.equal(a[1], b[1])
    lib = f.lib()
    p = ctypes.c_void_p(t[0].data_ptr())
    # output size that does not follow from the other arguments
    assert lib.fastnn_b200_conv2d_backward_weight(p, p, p, 1, 8, 16, 12, 12, 11, 12, 3, 3, 1, 1, 1, 1, None) == -1
    assert lib.fastnn_b200_conv2d_backward_data(p, p, p, 1, 8, 16, 12, 12, 11, 12, 3, 3, 1, 1, 1, 1, None) == -1
    # padding beyond kernel - 1 is outside what grad_input covers
    assert lib.fastnn_b200_conv2d_backward_data(p, p, p, 1, 8, 16, 12, 12, 16, 16, 3, 3, 1, 1, 3, 3, None) == -1
