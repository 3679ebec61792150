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
    # grad_input with stride 2 through FastNN's own symbol (the gather-form kernel)
    want_gi2, _ = oracle.conv2d_backward(x, wt, go, (2, 2), (1, 1))
    gi = torch.full(x.shape, float("nan"), device="cuda")
    assert lib.fastnn_cuda_conv2d_backward_data(vp(gd), vp(wd), vp(gi), 3, 6, 10, 15, 17, oh, ow, 3, 3,
                                                2, 2, 1, 1) == 0
    torch.cuda.synchronize()
    _check(gi.cpu().numpy(), want_gi2, 10 * 9, go, wt, "strided grad_input via the reference symbol")
    x1, w1, g1 = _case(2, 6, 10, 12, 12, 3, 3, (1, 1), (1, 1), 78)
    want_gi, _ = oracle.conv2d_backward(x1, w1, g1, (1, 1), (1, 1))
    g1d, w1d = torch.from_numpy(g1).cuda(), torch.from_numpy(w1).cuda()
    gi1 = torch.full(x1.shape, float("nan"), device="cuda")
    assert lib.fastnn_cuda_conv2d_backward_data(vp(g1d), vp(w1d), vp(gi1), 2, 6, 10, 12, 12, 12, 12, 3, 3,
                                                1, 1, 1, 1) == 0
    torch.cuda.synchronize()
    _check(gi1.cpu().numpy(), want_gi, 90, g1, w1, "grad_input via the reference symbol")


def test_grad_weight_takes_the_implicit_gemm_and_the_explicit_form_by_plane(gpu):
    """out_h * out_w a multiple of 4: implicit GEMM (path 5, K slices > 1 for a long contraction);
    otherwise the explicit column-matrix form (a batched GEMM, path 2).  Same result either way."""
    import torch
    f = gpu
    lib = f.lib()
    vp = lambda t: ctypes.c_void_p(t.data_ptr())
    for (n, ci, co, h, w, pad), want_path in (((8, 16, 40, 28, 28, 1), 5), ((4, 8, 24, 13, 11, 1), 2)):
        x, wt, go = _case(n, ci, co, h, w, 3, 3, (1, 1), (pad, pad), n + ci + co)
        _, want_gw = oracle.conv2d_backward(x, wt, go, (1, 1), (pad, pad))
        xd, gd = torch.from_numpy(x).cuda(), torch.from_numpy(go).cuda()
        gw = torch.full(wt.shape, float("nan"), device="cuda")
        assert lib.fastnn_b200_conv2d_backward_weight(vp(xd), vp(gd), vp(gw), n, ci, co, h, w, h, w, 3, 3, 1, 1,
                                                      pad, pad, None) == 0
        torch.cuda.synchronize()
        lp = f.last_path()
        assert lp["path"] == want_path or (want_path == 5 and lp["path"] == 11) or (want_path == 2 and lp["path"] == 1), lp
        if want_path == 5:
            assert lp["split_k"] > 1, "the contraction over 8 x 784 positions is cut into slices"
        _check(gw.cpu().numpy(), want_gw, n * h * w, go, x, f"grad_weight {(n, ci, co, h, w)}")
    assert f.device_status() == 0


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


@pytest.mark.parametrize("cfg", [
    # n, ci, co, h, w, kh, kw, stride, padding: what the stride-1 implicit-GEMM form does not cover
    (2, 8, 16, 16, 16, 3, 3, (2, 2), (1, 1)),
    (3, 5, 7, 19, 23, 7, 7, (2, 2), (3, 3)),        # 7 x 7, stride 2 (a network's first layer)
    (2, 4, 6, 17, 15, 3, 5, (3, 2), (0, 2)),        # uneven strides, rows the kernel never reaches
    (1, 3, 4, 10, 10, 2, 2, (1, 1), (3, 3)),        # stride 1 with padding beyond kernel - 1
    (2, 6, 5, 12, 12, 1, 1, (2, 2), (0, 0)),        # strided pointwise: three quarters of grad_input are 0
    (2, 4, 6, 20, 20, 2, 2, (3, 3), (1, 1)),        # stride beyond the kernel: whole phases are zero
    (1, 16, 32, 56, 56, 3, 3, (2, 2), (1, 1)),      # a network-sized plane, tiles spanning image rows
])
def test_conv2d_gradients_for_any_stride_and_padding(gpu, cfg):
    """FastNN's own entries accept every stride and padding (col2im, cuda/kernels.cu:862-893):
    so do these, against the CPU loops."""
    import torch
    f = gpu
    n, ci, co, h, w, kh, kw, stride, padding = cfg
    x, wt, go = _case(n, ci, co, h, w, kh, kw, stride, padding, 1000 + sum(cfg[:7]))
    want_gi, want_gw = oracle.conv2d_backward(x, wt, go, stride, padding)
    gi, gw = f.conv2d_backward(torch.from_numpy(x).cuda(), torch.from_numpy(wt).cuda(),
                               torch.from_numpy(go).cuda(), stride=stride, padding=padding)
    torch.cuda.synchronize()
    _check(gi.cpu().numpy(), want_gi, co * kh * kw, go, wt, f"grad_input {cfg}")
    _check(gw.cpu().numpy(), want_gw, n * go.shape[2] * go.shape[3], go, x, f"grad_weight {cfg}")
    assert f.device_status() == 0


def test_conv2d_forward_with_more_taps_than_the_gather_encodes(gpu):
    """An 8 x 8 kernel has 64 taps, one more than the implicit-GEMM gather's mask holds: served by
    the direct kernel (path 7), forward and input gradient."""
    import torch
    f = gpu
    x, wt, go = _case(2, 3, 5, 20, 20, 8, 8, (1, 1), (2, 2), 31)
    b = np.arange(5, dtype=np.float32)
    y = f.conv2d_forward(torch.from_numpy(x).cuda(), torch.from_numpy(wt).cuda(), torch.from_numpy(b).cuda(),
                         padding=(2, 2), act=f.ACT_RELU)
    assert f.last_path()["path"] == 7
    want = np.maximum(oracle.conv2d(x, wt, b, (1, 1), (2, 2)), 0.0)
    assert np.abs(y.cpu().numpy() - want).max() <= 1e-4 * 3 * 64
    want_gi, _ = oracle.conv2d_backward(x, wt, go, (1, 1), (2, 2))
    gi, _ = f.conv2d_backward(torch.from_numpy(x).cuda(), torch.from_numpy(wt).cuda(),
                              torch.from_numpy(go).cuda(), padding=(2, 2))
    assert np.abs(gi.cpu().numpy() - want_gi).max() <= 1e-4 * 5 * 64


@pytest.mark.parametrize("cfg", [
    # n, ci, co, h, w, kh, kw, stride, padding -- shapes the tensor-memory form of the weight gradient takes
    (2, 64, 128, 56, 56, 3, 3, (1, 1), (1, 1)),      # the benchmark layer, two images: 5 tap tiles, the last half full
    (3, 20, 200, 24, 24, 3, 3, (1, 1), (1, 1)),      # two channel tiles (128 + 72), 180 taps
    (2, 7, 9, 16, 20, 5, 5, (1, 1), (2, 2)),         # 25 taps per channel, fewer channels than a warp has lanes
    (2, 16, 24, 32, 32, 3, 3, (2, 2), (1, 1)),       # stride 2: inputs of a k-block two words apart
    (4, 40, 48, 12, 12, 1, 1, (1, 1), (0, 0)),       # pointwise: one channel per tap
    (2, 8, 16, 20, 36, 3, 4, (1, 1), (1, 4)),        # output rows of 41 columns: no 16-byte pitch, another form serves it
    (1, 5, 6, 8, 8, 3, 3, (1, 1), (1, 1)),           # one image, 64 positions: fewer slabs than SMs
    (2, 32, 32, 16, 64, 3, 3, (1, 1), (1, 1)),       # rows of exactly two k-blocks
])
def test_grad_weight_through_tensor_memory(gpu, cfg):
    """grad_weight with taps as the M dimension and the gathered input rows in tensor memory (path 11)."""
    import torch
    f = gpu
    lib = f.lib()
    vp = lambda t: ctypes.c_void_p(t.data_ptr())
    n, ci, co, h, w, kh, kw, stride, padding = cfg
    x, wt, go = _case(n, ci, co, h, w, kh, kw, stride, padding, 300 + sum(cfg[:7]))
    oh, ow = go.shape[2], go.shape[3]
    _, want_gw = oracle.conv2d_backward(x, wt, go, stride, padding)
    xd, gd = torch.from_numpy(x).cuda(), torch.from_numpy(go).cuda()
    gw = torch.full(wt.shape, float("nan"), device="cuda")
    assert lib.fastnn_b200_conv2d_backward_weight(vp(xd), vp(gd), vp(gw), n, ci, co, h, w, oh, ow, kh, kw,
                                                  stride[0], stride[1], padding[0], padding[1], None) == 0
    torch.cuda.synchronize()
    lp = f.last_path()
    if ow % 4 == 0:
        assert lp["path"] == 11, lp
    _check(gw.cpu().numpy(), want_gw, n * oh * ow, go, x, f"grad_weight {cfg}")
    # the same call again: bit-identical (fixed order of the slices and of the two accumulators)
    gw2 = torch.full(wt.shape, float("nan"), device="cuda")
    assert lib.fastnn_b200_conv2d_backward_weight(vp(xd), vp(gd), vp(gw2), n, ci, co, h, w, oh, ow, kh, kw,
                                                  stride[0], stride[1], padding[0], padding[1], None) == 0
    assert torch.equal(gw, gw2)
    assert f.device_status() == 0
