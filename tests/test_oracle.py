"""CPU: the oracle against the golden vectors and against itself (no GPU, no product code)."""
import numpy as np
import pytest

import oracle


def test_splitmix64_known_answer(golden):
    # Published SplitMix64 seed-0 outputs are E220A8397B1DCDAF, 6E789E6AA1B965F4, 06C45D188009454F;
    # the reference's Rng pre-advances once, so its first two draws are the 2nd and 3rd.
    assert golden["splitmix_seed0_reference_stream"][:2] == ["0x6e789e6aa1b965f4", "0x6c45d188009454f"]
    u = oracle.rand_data(2, 0)
    want = [np.float32(np.float32(z >> 40) / np.float32(1 << 24) * np.float32(2) - np.float32(1))
            for z in (0x6E789E6AA1B965F4, 0x06C45D188009454F)]
    assert u.tolist() == [float(w) for w in want]


def test_rand_data_matches_golden(golden):
    for c in golden["cases"]:
        a = oracle.rand_data(c["a"].size, 1).reshape(c["a"].shape)
        b = oracle.rand_data(c["b"].size, 2).reshape(c["b"].shape)
        assert np.array_equal(a.view(np.uint32), c["a"].view(np.uint32)), c["name"]
        assert np.array_equal(b.view(np.uint32), c["b"].view(np.uint32)), c["name"]
        w = oracle.rand_data(c["c"].size, 0xBADC0DE ^ len(c["name"]))
        assert np.array_equal(w.view(np.uint32), c["w"].view(np.uint32).ravel())


def _fwd(op, a, b):
    return {"nn": oracle.matmul, "nt": oracle.matmul_nt, "tn": oracle.matmul_tn}[op](a, b)


def test_forward_bit_exact_against_golden(golden):
    for c in golden["cases"]:
        got = _fwd(c["op"], c["a"], c["b"])
        assert got.shape == c["c"].shape
        assert np.array_equal(got.view(np.uint32), c["c"].view(np.uint32)), c["name"]


def test_backward_identities_bit_exact_against_golden(golden):
    # GradFns of src/autograd/backward_ops.rs:82-134 expressed with the oracle's entry points.
    for c in golden["cases"]:
        a, b, w = c["a"], c["b"], c["w"]
        if c["op"] == "nn":
            ga, gb = oracle.matmul_nt(w, b), oracle.matmul_tn(a, w)
        elif c["op"] == "nt":
            ga, gb = oracle.matmul(w, b), oracle.matmul_tn(w, a)
        else:
            ga, gb = oracle.matmul_nt(b, w), oracle.matmul(a, w)
        assert np.array_equal(ga.view(np.uint32), c["grad_a"].view(np.uint32)), c["name"]
        assert np.array_equal(gb.view(np.uint32), c["grad_b"].view(np.uint32)), c["name"]


def test_integer_known_answers():
    a = np.array([[1, 2, 3], [4, 5, 6]], dtype=np.float32)
    b = np.array([[7, 8], [9, 10], [11, 12]], dtype=np.float32)
    assert oracle.matmul(a, b).tolist() == [[58, 64], [139, 154]]
    assert oracle.matmul_nt(a, b.T.copy()).tolist() == [[58, 64], [139, 154]]
    assert oracle.matmul_tn(a.T.copy(), b).tolist() == [[58, 64], [139, 154]]


def test_summation_order_is_p_ascending_unfused():
    # 2^24 + 1 - 2^24: ascending order loses the 1 (rounds to 2^24, then 0); FMA or another
    # order would give a different bit pattern.
    a = np.array([[2.0 ** 24, 1.0, -(2.0 ** 24)]], dtype=np.float32)
    b = np.ones((3, 1), dtype=np.float32)
    assert oracle.matmul(a, b)[0, 0] == 0.0
    # unfused multiply: (1+2^-12)^2 rounds to 1+2^-11 before the add
    x = np.float32(1 + 2.0 ** -12)
    a = np.array([[x, -1.0]], dtype=np.float32)
    b = np.array([[x], [np.float32(1 + 2.0 ** -11)]], dtype=np.float32)
    assert oracle.matmul(a, b)[0, 0] == 0.0


@pytest.mark.parametrize("shape", [(17, 9, 33), (64, 64, 64), (1, 7, 5), (130, 3, 1)])
def test_against_float64(shape):
    m, n, k = shape
    rng = np.random.default_rng(7)
    a = rng.standard_normal((m, k), dtype=np.float32)
    b = rng.standard_normal((k, n), dtype=np.float32)
    want = a.astype(np.float64) @ b.astype(np.float64)
    for got in (oracle.matmul(a, b), oracle.matmul_nt(a, b.T.copy()), oracle.matmul_tn(a.T.copy(), b)):
        assert np.abs(got - want).max() <= 1e-6 * k * np.abs(a).max() * np.abs(b).max()


def test_layout_variants_bit_identical():
    rng = np.random.default_rng(3)
    a = rng.standard_normal((4, 37, 29), dtype=np.float32)
    b = rng.standard_normal((4, 29, 31), dtype=np.float32)
    c = oracle.matmul(a, b)
    assert np.array_equal(c, oracle.matmul_nt(a, oracle.transpose(b)))
    assert np.array_equal(c, oracle.matmul_tn(oracle.transpose(a), b))
    # batch-1 broadcast of the CPU arm (src/tensor/ops.rs:401-411)
    c1 = oracle.matmul(a[:1], b)
    assert np.array_equal(c1[2], oracle.matmul(a[0], b[2]))


def test_row_parallel_twin_is_bit_identical():
    rng = np.random.default_rng(5)
    a = rng.standard_normal((203, 77), dtype=np.float32)
    b = rng.standard_normal((77, 65), dtype=np.float32)
    c = oracle.matmul(a, b)
    for t in (2, 3, 8):
        assert np.array_equal(c, oracle.matmul(a, b, threads=t))
    assert np.array_equal(c[50:120], oracle.matmul_rows(a, b, 50, 120, threads=4))


def test_empty_and_degenerate_shapes():
    z = np.zeros((0, 4), dtype=np.float32)
    b = np.ones((4, 3), dtype=np.float32)
    assert oracle.matmul(z, b).shape == (0, 3)
    a = np.ones((2, 0), dtype=np.float32)
    assert oracle.matmul(a, np.ones((0, 3), dtype=np.float32)).tolist() == [[0, 0, 0], [0, 0, 0]]


def test_linear_bias_relu_gelu():
    rng = np.random.default_rng(11)
    x = rng.standard_normal((9, 6), dtype=np.float32)
    w = rng.standard_normal((5, 6), dtype=np.float32)
    bias = rng.standard_normal(5, dtype=np.float32)
    y = oracle.linear(x, w, bias)
    assert np.array_equal(y, oracle.matmul(x, oracle.transpose(w)) + bias[None, :])
    assert np.array_equal(oracle.linear(x, w, bias, oracle.ACT_RELU), np.maximum(y, 0))
    from math import erf, sqrt
    g = oracle.linear(x, w, bias, oracle.ACT_GELU)
    want = np.array([[0.5 * v * (1 + erf(v / sqrt(2))) for v in row] for row in y.astype(np.float64)])
    assert np.abs(g - want).max() < 1e-6


def test_linear_backward_input_follows_the_tape():
    """dx = matmul(dy, W) * act'(pre); the GELU derivative is the analytic one (checked against a
    float64 finite difference of the forward GELU); the bias gradient is the sum over rows."""
    from math import erf, sqrt
    rng = np.random.default_rng(21)
    dy = rng.standard_normal((7, 5), dtype=np.float32)
    w = rng.standard_normal((5, 6), dtype=np.float32)
    pre = rng.standard_normal((7, 6), dtype=np.float32)
    base = oracle.matmul(dy, w)
    dx, db = oracle.linear_backward_input(dy, w, None, oracle.ACT_NONE)
    assert np.array_equal(dx, base)
    assert np.allclose(db, base.astype(np.float64).sum(0), atol=1e-5)
    dx, db = oracle.linear_backward_input(dy, w, pre, oracle.ACT_RELU)
    assert np.array_equal(dx, base * (pre > 0))
    dx, db = oracle.linear_backward_input(dy, w, pre, oracle.ACT_GELU)
    gelu = lambda v: 0.5 * v * (1 + erf(v / sqrt(2)))
    h = 1e-6
    fd = np.array([[(gelu(v + h) - gelu(v - h)) / (2 * h) for v in row] for row in pre.astype(np.float64)])
    assert np.abs(dx - base * fd).max() < 1e-4
    assert np.allclose(db, dx.astype(np.float64).sum(0), atol=1e-5)


def test_rnn_gates_are_the_two_products_plus_both_biases():
    rng = np.random.default_rng(31)
    x = rng.standard_normal((5, 7), dtype=np.float32)
    h = rng.standard_normal((5, 3), dtype=np.float32)
    w_ih = rng.standard_normal((12, 7), dtype=np.float32)
    w_hh = rng.standard_normal((12, 3), dtype=np.float32)
    b1 = rng.standard_normal(12, dtype=np.float32)
    b2 = rng.standard_normal(12, dtype=np.float32)
    g = oracle.rnn_gates(x, h, w_ih, w_hh, b1, b2)
    want = x.astype(np.float64) @ w_ih.T.astype(np.float64) + h.astype(np.float64) @ w_hh.T + b1 + b2
    assert g.dtype == np.float32 and np.abs(g - want).max() < 1e-5
    assert np.array_equal(oracle.rnn_gates(x, h, w_ih, w_hh, None, None),
                          oracle.matmul_nt(x, w_ih) + oracle.matmul_nt(h, w_hh))


def test_conv2d_loops_against_a_direct_float64_sum():
    rng = np.random.default_rng(41)
    x = rng.standard_normal((2, 3, 7, 6), dtype=np.float32)
    w = rng.standard_normal((4, 3, 3, 2), dtype=np.float32)
    b = rng.standard_normal(4, dtype=np.float32)
    got = oracle.conv2d(x, w, b, (2, 1), (1, 0))
    xp = np.pad(x.astype(np.float64), ((0, 0), (0, 0), (1, 1), (0, 0)))
    oh, ow = (7 + 2 - 3) // 2 + 1, (6 - 2) // 1 + 1
    assert got.shape == (2, 4, oh, ow)
    want = np.zeros((2, 4, oh, ow))
    for i in range(oh):
        for j in range(ow):
            patch = xp[:, :, 2 * i:2 * i + 3, j:j + 2]
            want[:, :, i, j] = np.einsum("nchw,ochw->no", patch, w.astype(np.float64)) + b
    assert np.abs(got - want).max() < 1e-5
    # a 1x1 kernel is a matmul over channels
    w1 = rng.standard_normal((5, 3, 1, 1), dtype=np.float32)
    y = oracle.conv2d(x, w1, None)
    ref = np.einsum("nchw,oc->nohw", x.astype(np.float64), w1[:, :, 0, 0].astype(np.float64))
    assert np.abs(y - ref).max() < 1e-5


def test_conv2d_backward_is_the_adjoint_of_the_forward_loops():
    """<grad_input, x'> = <go, conv(x', w)> and <grad_weight, w'> = <go, conv(x, w')> for any x', w'."""
    rng = np.random.default_rng(43)
    x = rng.standard_normal((2, 3, 8, 7), dtype=np.float32)
    w = rng.standard_normal((4, 3, 3, 2), dtype=np.float32)
    stride, padding = (2, 1), (1, 0)
    go = rng.standard_normal(oracle.conv2d(x, w, None, stride, padding).shape, dtype=np.float32)
    gi, gw = oracle.conv2d_backward(x, w, go, stride, padding)
    x2 = rng.standard_normal(x.shape, dtype=np.float32)
    w2 = rng.standard_normal(w.shape, dtype=np.float32)
    lhs_i = float((gi.astype(np.float64) * x2).sum())
    rhs_i = float((go.astype(np.float64) * oracle.conv2d(x2, w, None, stride, padding)).sum())
    lhs_w = float((gw.astype(np.float64) * w2).sum())
    rhs_w = float((go.astype(np.float64) * oracle.conv2d(x, w2, None, stride, padding)).sum())
    assert abs(lhs_i - rhs_i) <= 1e-3 * max(1.0, abs(rhs_i))
    assert abs(lhs_w - rhs_w) <= 1e-3 * max(1.0, abs(rhs_w))


def test_causal_softmax_rows():
    rng = np.random.default_rng(2)
    s = rng.standard_normal((3, 8, 8), dtype=np.float32)
    p = oracle.causal_softmax(s, 1.0 / np.sqrt(32.0))
    assert np.allclose(p.sum(-1), 1.0, atol=1e-6)
    assert np.all(np.triu(p, 1) == 0.0)


def test_gru_restatement_matches_a_float64_evaluation():
    """oracle.gru_gates / gru_step (src/nn/rnn.rs:164-180) against the same formulas in float64."""
    rng = np.random.default_rng(11)
    batch, inp, hid = 5, 7, 6
    x = rng.standard_normal((batch, inp)).astype(np.float32)
    h = rng.standard_normal((batch, hid)).astype(np.float32)
    w_ih = rng.standard_normal((3 * hid, inp)).astype(np.float32)
    w_hh = rng.standard_normal((3 * hid, hid)).astype(np.float32)
    b_ih = rng.standard_normal(3 * hid).astype(np.float32)
    b_hh = rng.standard_normal(3 * hid).astype(np.float32)
    gi, gh = oracle.gru_gates(x, h, w_ih, w_hh, b_ih, b_hh)
    gi64 = x.astype(np.float64) @ w_ih.astype(np.float64).T + b_ih
    gh64 = h.astype(np.float64) @ w_hh.astype(np.float64).T + b_hh
    assert np.allclose(gi, gi64, rtol=1e-5, atol=1e-5) and np.allclose(gh, gh64, rtol=1e-5, atol=1e-5)
    sig = lambda v: 1.0 / (1.0 + np.exp(-v))
    r = sig(gi64[:, :hid] + gh64[:, :hid])
    z = sig(gi64[:, hid:2 * hid] + gh64[:, hid:2 * hid])
    n = np.tanh(gi64[:, 2 * hid:] + r * gh64[:, 2 * hid:])
    want = (1 - z) * n + z * h
    got = oracle.gru_step(gi, gh, h)
    assert got.dtype == np.float32 and np.allclose(got, want, rtol=1e-4, atol=1e-5)
