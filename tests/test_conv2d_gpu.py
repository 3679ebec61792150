"""GPU: Conv2d forward as an implicit GEMM against the CPU loops of Conv2d::forward
(src/nn/conv.rs:97-123).

Tolerance: the GEMM bar with K = Cin*KH*KW: relative Frobenius <= 5e-3,
max-abs <= 1e-2 sqrt(K) max|x| max|w|."""
import ctypes

import numpy as np
import pytest

import oracle

pytestmark = pytest.mark.gpu


def _case(n, ci, co, h, w, kh, kw, seed, bias=True):
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((n, ci, h, w), dtype=np.float32)
    wt = (rng.standard_normal((co, ci, kh, kw), dtype=np.float32) * 0.2).astype(np.float32)
    b = rng.standard_normal(co, dtype=np.float32) if bias else None
    return x, wt, b


def _check(got, want, k, x, wt, what):
    assert got.shape == want.shape, what
    assert np.isfinite(got).all(), what
    err = got.astype(np.float64) - want
    assert np.linalg.norm(err) / np.linalg.norm(want) <= 5e-3, what
    assert np.abs(err).max() <= 1e-2 * np.sqrt(k) * np.abs(x).max() * np.abs(wt).max(), what


@pytest.mark.parametrize("cfg", [
    # n, ci, co, h, w, kh, kw, stride, padding
    (2, 3, 16, 32, 32, 3, 3, (1, 1), (1, 1)),        # RGB stem: K = 27, padded weights
    (4, 16, 32, 28, 28, 3, 3, (1, 1), (1, 1)),       # K = 144
    (2, 8, 24, 17, 19, 5, 3, (2, 1), (2, 0)),        # ragged sizes, rectangular kernel, mixed stride / padding
    (3, 32, 64, 14, 14, 1, 1, (1, 1), (0, 0)),       # pointwise
    (1, 4, 300, 9, 9, 3, 3, (2, 2), (0, 0)),         # more channels than one tile is wide
    (8, 64, 128, 16, 16, 3, 3, (1, 1), (1, 1)),      # K = 576, several position tiles per image
    (1, 1, 1, 5, 5, 5, 5, (1, 1), (0, 0)),           # one output element
])
def test_conv2d_matches_the_cpu_loops(gpu, cfg):
    import torch
    f = gpu
    n, ci, co, h, w, kh, kw, stride, padding = cfg
    x, wt, b = _case(n, ci, co, h, w, kh, kw, sum(cfg[:7]))
    want = oracle.conv2d(x, wt, b, stride, padding)
    got = f.conv2d_forward(torch.from_numpy(x).cuda(), torch.from_numpy(wt).cuda(), torch.from_numpy(b).cuda(),
                           stride=stride, padding=padding)
    torch.cuda.synchronize()
    assert f.last_path()["path"] in (5, 9)
    _check(got.cpu().numpy(), want, ci * kh * kw, x, wt, str(cfg))
    assert f.device_status() == 0


def test_conv2d_without_bias_with_relu_and_through_the_reference_symbol(gpu):
    import torch
    f = gpu
    x, wt, b = _case(2, 6, 20, 12, 12, 3, 3, 5)
    xd, wd, bd = (torch.from_numpy(t).cuda() for t in (x, wt, b))
    want = oracle.conv2d(x, wt, None, (1, 1), (1, 1))
    _check(f.conv2d_forward(xd, wd, None, padding=(1, 1)).cpu().numpy(), want, 54, x, wt, "no bias")
    relu = f.conv2d_forward(xd, wd, bd, padding=(1, 1), act=f.ACT_RELU).cpu().numpy()
    want_b = oracle.conv2d(x, wt, b, (1, 1), (1, 1))
    _check(relu, np.maximum(want_b, 0), 54, x, wt, "relu")
    assert (relu >= 0).all()
    # FastNN's own entry point name and argument list
    out = torch.full((2, 20, 12, 12), float("nan"), device="cuda")
    vp = lambda t: ctypes.c_void_p(t.data_ptr())
    assert f.lib().fastnn_cuda_conv2d_forward(vp(xd), vp(wd), vp(bd), vp(out), 2, 6, 20, 12, 12, 3, 3,
                                              1, 1, 1, 1) == 0
    torch.cuda.synchronize()
    _check(out.cpu().numpy(), want_b, 54, x, wt, "reference symbol")


def test_conv2d_is_deterministic_and_rejects_bad_arguments(gpu):
    import torch
    f = gpu
    x, wt, b = _case(4, 16, 48, 20, 20, 3, 3, 9)
    t = [torch.from_numpy(a).cuda() for a in (x, wt, b)]
    a = f.conv2d_forward(*t, padding=(1, 1))
    c = f.conv2d_forward(*t, padding=(1, 1))
    assert torch.equal(a, c)
    lib = f.lib()
    p, null = ctypes.c_void_p(t[0].data_ptr()), ctypes.c_void_p(0)
    assert lib.fastnn_b200_conv2d_forward(p, p, null, p, 1, 0, 4, 8, 8, 3, 3, 1, 1, 0, 0, 0, None) == -1   # channels
    assert lib.fastnn_b200_conv2d_forward(p, p, null, p, 1, 4, 4, 2, 2, 3, 3, 1, 1, 0, 0, 0, None) == -1   # kernel > input
    assert lib.fastnn_b200_conv2d_forward(p, p, null, p, 1, 4, 4, 8, 8, 3, 3, 0, 1, 0, 0, 0, None) == -1   # stride
    assert lib.fastnn_b200_conv2d_forward(p, p, null, p, 1, 4, 4, 8, 8, 3, 3, 1, 1, 0, 0, 2, None) == -1   # act
    assert lib.fastnn_b200_conv2d_forward(p, p, null, p, 0, 4, 4, 8, 8, 3, 3, 1, 1, 0, 0, 0, None) == 0    # empty batch
    # (64 taps or more and images of 2^25 elements or more are served by the direct kernel:
    # tests/test_conv2d_backward_gpu.py::test_conv2d_forward_with_more_taps_than_the_gather_encodes)


def test_conv2d_with_a_seven_by_seven_kernel_and_stride_two(gpu):
    """49 taps (the tap mask's upper half) and a tile that spans images."""
    import torch
    f = gpu
    x, wt, b = _case(3, 3, 64, 37, 41, 7, 7, 13)
    want = oracle.conv2d(x, wt, b, (2, 2), (3, 3))
    got = f.conv2d_forward(torch.from_numpy(x).cuda(), torch.from_numpy(wt).cuda(), torch.from_numpy(b).cuda(),
                           stride=(2, 2), padding=(3, 3))
    _check(got.cpu().numpy(), want, 3 * 49, x, wt, "7x7 stride 2")


@pytest.mark.parametrize("cfg", [
    # n, ci, co, h, w, kh, kw, stride, padding -- shapes whose rows a tensor map can address (w % 4 == 0)
    (2, 64, 128, 56, 56, 3, 3, (1, 1), (1, 1)),      # the benchmark layer, two images: 2 chunks, tiles of 2.3 rows
    (2, 48, 40, 24, 24, 3, 3, (1, 1), (1, 1)),       # second chunk half out of range (48 = 32 + 16 channels)
    (3, 100, 300, 12, 12, 3, 3, (1, 1), (1, 1)),     # four chunks, three channel tiles, 144 positions per image
    (2, 8, 16, 40, 36, 5, 5, (1, 1), (2, 2)),        # 25 taps, padding 2
    (2, 3, 32, 8, 32, 7, 7, (1, 1), (3, 3)),         # 49 taps, padding 3 (three of the four halo columns)
    (2, 16, 24, 20, 16, 3, 3, (2, 1), (0, 1)),       # mixed stride and padding
    (5, 32, 64, 8, 8, 3, 3, (1, 1), (1, 1)),         # 64 positions per image: half of every tile is past the image
    (1, 4, 8, 16, 248, 1, 3, (1, 1), (0, 1)),        # the widest row a slab takes (248 + 8 columns), one-row kernel
    (2, 12, 20, 16, 16, 3, 4, (1, 1), (1, 4)),       # horizontal padding equal to the halo
])
def test_conv2d_from_rows_staged_in_shared_memory(gpu, cfg):
    """The form that brings every tile's input rows into shared memory by TMA (path 9)."""
    import torch
    f = gpu
    n, ci, co, h, w, kh, kw, stride, padding = cfg
    x, wt, b = _case(n, ci, co, h, w, kh, kw, 100 + sum(cfg[:7]))
    want = oracle.conv2d(x, wt, b, stride, padding)
    got = f.conv2d_forward(torch.from_numpy(x).cuda(), torch.from_numpy(wt).cuda(), torch.from_numpy(b).cuda(),
                           stride=stride, padding=padding)
    torch.cuda.synchronize()
    assert f.last_path()["path"] == 9, f.last_path()
    _check(got.cpu().numpy(), want, ci * kh * kw, x, wt, str(cfg))
    assert f.device_status() == 0


@pytest.mark.parametrize("cfg", [
    (2, 8, 16, 16, 16, 3, 3, (1, 1), (5, 5)),        # padding wider than the halo
    (2, 8, 16, 16, 18, 3, 3, (1, 1), (1, 1)),        # row pitch not a multiple of 16 bytes
    (1, 4, 8, 8, 260, 1, 3, (1, 1), (0, 1)),         # row wider than a TMA box
    (2, 3, 32, 32, 32, 7, 7, (2, 2), (3, 3)),        # 21 input rows per tile: two slabs do not fit
])
def test_conv2d_shapes_the_staged_form_leaves_to_the_global_gather(gpu, cfg):
    import torch
    f = gpu
    n, ci, co, h, w, kh, kw, stride, padding = cfg
    x, wt, b = _case(n, ci, co, h, w, kh, kw, 200 + sum(cfg[:7]))
    want = oracle.conv2d(x, wt, b, stride, padding)
    got = f.conv2d_forward(torch.from_numpy(x).cuda(), torch.from_numpy(wt).cuda(), torch.from_numpy(b).cuda(),
                           stride=stride, padding=padding)
    torch.cuda.synchronize()
    assert f.last_path()["path"] == 5, f.last_path()
    _check(got.cpu().numpy(), want, ci * kh * kw, x, wt, str(cfg))
