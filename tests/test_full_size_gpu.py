"""GPU: the full-size configurations, checked through size-independent properties.

At 8192^3 and 32768 x 16384 x 4096 the CPU oracle needs minutes per product, so these cases use
(1) exact integer arithmetic: small-integer operands are exact in TF32 and their dot products are
    exact in FP32, so row/column checksums of C must equal checksums computed from A and B alone
    ("checksum of checksums"), bit for bit;
(2) a contiguous slab of rows plus 64 rows drawn at random, recomputed by the oracle on the
    real-valued inputs (TF32 tolerance); the checked fraction of the output is printed;
(3) agreement of the three layouts on the same logical operands.
"""
import numpy as np
import pytest

import oracle
from helpers import check_tf32_parity

pytestmark = pytest.mark.gpu

NN, NT, TN = 0, 1, 2


def _int_operands(torch, m, n, k, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    a = torch.randint(-3, 4, (m, k), device="cuda", generator=g).float()
    b = torch.randint(-3, 4, (k, n), device="cuda", generator=g).float()
    return a, b


def _slab_and_random_rows(total, slab0, slab_rows, extra, seed):
    """A contiguous slab [slab0, slab0 + slab_rows) and `extra` further rows drawn at random."""
    slab = np.arange(slab0, slab0 + slab_rows)
    rest = np.setdiff1d(np.arange(total), slab)
    return np.sort(np.concatenate([slab, np.random.default_rng(seed).choice(rest, extra, replace=False)]))


def _run(f, layout, a, b):
    if layout == NN:
        return f.matmul(a, b)
    if layout == NT:
        return f.matmul_nt(a, b.t().contiguous())
    return f.matmul_tn(a.t().contiguous(), b)


@pytest.mark.parametrize("layout", [NN, NT, TN])
def test_square_8192_integer_checksums_are_exact(gpu, layout):
    import torch
    f = gpu
    m = n = k = 8192
    a, b = _int_operands(torch, m, n, k, 40 + layout)
    c = _run(f, layout, a, b)
    assert f.last_path()["path"] in (2, 3)
    ad, bd, cd = a.double(), b.double(), c.double()
    ones_n = torch.ones(n, 1, device="cuda", dtype=torch.float64)
    ones_m = torch.ones(1, m, device="cuda", dtype=torch.float64)
    # |entries| <= 9 * 8192 < 2^24: every partial sum is an exact FP32 integer
    assert torch.equal(cd @ ones_n, ad @ (bd @ ones_n)), "row checksums differ"
    assert torch.equal(ones_m @ cd, (ones_m @ ad) @ bd), "column checksums differ"
    # a random +-1 probe catches errors that cancel in plain sums
    g = torch.Generator(device="cuda").manual_seed(7)
    s = (torch.randint(0, 2, (n, 1), device="cuda", generator=g) * 2 - 1).double()
    assert torch.equal(cd @ s, ad @ (bd @ s))


def test_square_8192_real_inputs_row_slab_and_layout_agreement(gpu):
    import torch
    f = gpu
    m = n = k = 8192
    g = torch.Generator(device="cuda").manual_seed(4000)
    a = torch.randn(m, k, device="cuda", generator=g)
    b = torch.randn(k, n, device="cuda", generator=g)
    c_nn, c_nt, c_tn = (_run(f, L, a, b) for L in (NN, NT, TN))
    rows = _slab_and_random_rows(m, 3072, 512, 64, seed=1)
    print(f"8192^3: {len(rows)} of {m} rows checked against the oracle ({100.0 * len(rows) / m:.1f} % of C)")
    ah = a[torch.from_numpy(rows).cuda()].cpu().numpy()
    bh = b.cpu().numpy()
    want = oracle.matmul(ah, bh, threads=oracle.host_threads())
    for name, c in (("NN", c_nn), ("NT", c_nt), ("TN", c_tn)):
        got = c[torch.from_numpy(rows).cuda()].cpu().numpy()
        check_tf32_parity(got, want, k, ah, bh, what=f"8192^3 {name} rows")
    # same logical product through three operand layouts: equal up to summation order
    scale = c_nn.abs().max().item()
    assert (c_nn - c_nt).abs().max().item() <= 1e-4 * scale
    assert (c_nn - c_tn).abs().max().item() <= 1e-4 * scale


def test_scaled_linear_gelu_full_size(gpu):
    """X[32768,4096] . W[4096,16384] + bias, exact-erf GELU; plus the two backward shapes."""
    import torch
    f = gpu
    m, k, n = 32768, 4096, 16384
    g = torch.Generator(device="cuda").manual_seed(5000)
    x = torch.randn(m, k, device="cuda", generator=g)
    bound = float(np.sqrt(6.0 / (k + n)))
    w = (torch.rand(k, n, device="cuda", generator=g) * 2 - 1) * bound
    bias = (torch.rand(n, device="cuda", generator=g) * 2 - 1) * 0.01
    y = f.linear_forward(x, w, bias, act=2, layout=NN)
    assert f.last_path()["path"] in (2, 3)
    rows = _slab_and_random_rows(m, 16384, 128, 64, seed=2)
    print(f"linear+GELU forward: {len(rows)} of {m} rows checked against the oracle")
    ridx = torch.from_numpy(rows).cuda()
    xh, wh, bh = x[ridx].cpu().numpy(), w.cpu().numpy(), bias.cpu().numpy()
    pre = oracle.bias_act(oracle.matmul(xh, wh, threads=oracle.host_threads()), bh, 0)
    want = oracle.bias_act(pre, None, 2)
    got = y[ridx].cpu().numpy()
    err = np.abs(got - want)
    assert err.max() <= 1e-2 * np.sqrt(k) * np.abs(xh).max() * np.abs(wh).max()
    assert np.linalg.norm(err) / np.linalg.norm(pre) <= 5e-3
    del y
    # the two backward products on the configured real-valued inputs (dY ~ N(0, 1e-3)), rows and
    # columns recomputed by the oracle
    dy = torch.randn(m, n, device="cuda", generator=g) * 1e-3
    threads = oracle.host_threads()
    dx = f.matmul_nt(dy, w)                                   # dX = dY . W^T   [m, k], contraction n
    assert f.last_path()["path"] in (2, 3)
    rows = _slab_and_random_rows(m, 8192, 32, 64, seed=3)
    ridx = torch.from_numpy(rows).cuda()
    dyh = dy[ridx].cpu().numpy()
    want = oracle.matmul(dyh, np.ascontiguousarray(wh.T), threads=threads)
    check_tf32_parity(dx[ridx].cpu().numpy(), want, n, dyh, wh, what="dX = dY . W^T rows")
    print(f"dX: {len(rows)} of {m} rows checked against the oracle")
    del dx
    dwt = f.matmul_tn(x, dy)                                  # dW = X^T . dY   [k, n], contraction m
    assert f.last_path()["path"] in (2, 3)
    cols = _slab_and_random_rows(k, 1024, 32, 64, seed=4)     # rows of dW = columns of the stored X
    cidx = torch.from_numpy(cols).cuda()
    xt = np.ascontiguousarray(x[:, cidx].cpu().numpy().T)     # [len(cols), m]
    dy_host = dy.cpu().numpy()
    want = oracle.matmul(xt, dy_host, threads=threads)
    check_tf32_parity(dwt[cidx].cpu().numpy(), want, m, xt, dy_host, what="dW = X^T . dY rows")
    print(f"dW: {len(cols)} of {k} rows checked against the oracle")
    del dwt, dy_host, want
    # and on integer operands: exact row, column and +-1-probe checksums
    dyi = torch.randint(-2, 3, (m, n), device="cuda", generator=g).float()
    wi = torch.randint(-2, 3, (k, n), device="cuda", generator=g).float()
    xi = torch.randint(-2, 3, (m, k), device="cuda", generator=g).float()
    probe = lambda size: (torch.randint(0, 2, (size, 1), device="cuda", generator=g) * 2 - 1).double()
    dx = f.matmul_nt(dyi, wi).double()                        # [m, k]; |entries| <= 4 * 16384 < 2^24
    for s_k in (torch.ones(k, 1, device="cuda", dtype=torch.float64), probe(k)):
        assert torch.equal(dx @ s_k, dyi.double() @ (wi.double().t() @ s_k)), "dX row checksum"
    ones_m = torch.ones(1, m, device="cuda", dtype=torch.float64)
    assert torch.equal(ones_m @ dx, (ones_m @ dyi.double()) @ wi.double().t()), "dX column checksum"
    del dx
    dwt = f.matmul_tn(xi, dyi).double()                       # [k, n]; |entries| <= 4 * 32768 < 2^24
    for s_n in (torch.ones(n, 1, device="cuda", dtype=torch.float64), probe(n)):
        assert torch.equal(dwt @ s_n, xi.double().t() @ (dyi.double() @ s_n)), "dW row checksum"
    ones_k = torch.ones(1, k, device="cuda", dtype=torch.float64)
    assert torch.equal(ones_k @ dwt, (ones_k @ xi.double().t()) @ dyi.double()), "dW column checksum"


def test_run_to_run_determinism(gpu):
    import torch
    f = gpu
    g = torch.Generator(device="cuda").manual_seed(1)
    a = torch.randn(2048, 1024, device="cuda", generator=g)
    b = torch.randn(1024, 3072, device="cuda", generator=g)
    c1 = f.matmul(a, b).clone()
    c2 = f.matmul(a, b)
    assert torch.equal(c1, c2)
