"""GPU: gate pre-activations of a recurrent step, x_t . W_ih^T + h . W_hh^T + b_ih + b_hh in one
launch, against the CPU composition of LSTM::forward (src/nn/rnn.rs:72-77).

Tolerance: the GEMM bar with K = input + hidden (both products share one accumulator):
relative Frobenius <= 5e-3, max-abs <= 1e-2 sqrt(K) max|operand| max|weight|."""
import ctypes

import numpy as np
import pytest

import oracle

pytestmark = pytest.mark.gpu


def _data(batch, inp, hid, g_rows, seed, seq=1):
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((batch, seq, inp), dtype=np.float32)
    h = rng.standard_normal((batch, hid), dtype=np.float32)
    w_ih = (rng.standard_normal((g_rows, inp), dtype=np.float32) * 0.3).astype(np.float32)
    w_hh = (rng.standard_normal((g_rows, hid), dtype=np.float32) * 0.3).astype(np.float32)
    b_ih = rng.standard_normal(g_rows, dtype=np.float32)
    b_hh = rng.standard_normal(g_rows, dtype=np.float32)
    return x, h, w_ih, w_hh, b_ih, b_hh


def _check(got, want, k, amax, wmax, what):
    assert np.isfinite(got).all(), what
    err = got.astype(np.float64) - want
    assert np.linalg.norm(err) / np.linalg.norm(want) <= 5e-3, what
    assert np.abs(err).max() <= 1e-2 * np.sqrt(k) * amax * wmax, what


@pytest.mark.parametrize("shape", [
    (64, 128, 256, 1024),      # LSTM: 4 * hidden gate rows
    (256, 64, 64, 256),
    (40, 36, 100, 400),        # ragged batch, K ranges that end inside a 32-deep block
    (512, 256, 512, 2048),
    (8, 32, 32, 32),           # plain RNN cell: gate_rows = hidden
])
def test_gates_match_the_lstm_composition(gpu, shape):
    import torch
    f = gpu
    batch, inp, hid, g_rows = shape
    x, h, w_ih, w_hh, b_ih, b_hh = _data(batch, inp, hid, g_rows, sum(shape))
    want = oracle.rnn_gates(x[:, 0, :], h, w_ih, w_hh, b_ih, b_hh)
    t = [torch.from_numpy(np.ascontiguousarray(a)).cuda() for a in (x[:, 0, :], h, w_ih, w_hh, b_ih, b_hh)]
    got = f.rnn_gates_forward(*t)
    torch.cuda.synchronize()
    assert f.last_path()["path"] in (2, 6) and f.launch_count() > 0   # single CTAs, or a K-split cluster
    amax = max(np.abs(x).max(), np.abs(h).max())
    wmax = max(np.abs(w_ih).max(), np.abs(w_hh).max())
    _check(got.cpu().numpy(), want, inp + hid, amax, wmax, str(shape))
    assert f.device_status() == 0


def test_gates_take_one_launch_and_a_strided_time_slice(gpu):
    """x_t = x[:, t, :] of x[batch, seq, input] is passed as a view (row stride seq * input)."""
    import torch
    f = gpu
    batch, seq, inp, hid = 96, 5, 64, 128
    x, h, w_ih, w_hh, b_ih, b_hh = _data(batch, inp, hid, 4 * hid, 17, seq=seq)
    xd = torch.from_numpy(x).cuda()
    rest = [torch.from_numpy(a).cuda() for a in (h, w_ih, w_hh, b_ih, b_hh)]
    for t in (0, 3):
        n0 = f.launch_count()
        got = f.rnn_gates_forward(xd[:, t, :], *rest)
        # one GEMM launch for both products, plus the reduce when the planner split K through the
        # workspace (path 2); a K-split cluster (path 6) reduces inside the launch
        lp = f.last_path()
        assert lp["path"] in (2, 6)
        assert f.launch_count() - n0 == (2 if lp["split_k"] > 1 and lp["path"] == 2 else 1)
        want = oracle.rnn_gates(x[:, t, :], h, w_ih, w_hh, b_ih, b_hh)
        _check(got.cpu().numpy(), want, inp + hid, 5.0, 2.0, f"t={t}")


def test_gates_without_biases_and_with_one(gpu):
    import torch
    f = gpu
    x, h, w_ih, w_hh, b_ih, b_hh = _data(128, 96, 160, 640, 23)
    t = [torch.from_numpy(np.ascontiguousarray(a)).cuda() for a in (x[:, 0, :], h, w_ih, w_hh)]
    bi, bh = torch.from_numpy(b_ih).cuda(), torch.from_numpy(b_hh).cuda()
    for a, b, wa, wb in ((None, None, None, None), (bi, None, b_ih, None), (None, bh, None, b_hh)):
        got = f.rnn_gates_forward(*t, a, b)
        want = oracle.rnn_gates(x[:, 0, :], h, w_ih, w_hh, wa, wb)
        _check(got.cpu().numpy(), want, 256, 5.0, 2.0, "bias variants")


def test_gates_fall_back_to_two_launches_when_tma_cannot_address_an_operand(gpu):
    import torch
    f = gpu
    x, h, w_ih, w_hh, b_ih, b_hh = _data(20, 30, 45, 90, 29)          # odd leading dimensions
    t = [torch.from_numpy(np.ascontiguousarray(a)).cuda() for a in (x[:, 0, :], h, w_ih, w_hh, b_ih, b_hh)]
    n0 = f.launch_count()
    got = f.rnn_gates_forward(*t)
    assert f.launch_count() - n0 == 2 and f.last_path()["path"] == 1
    want = oracle.rnn_gates(x[:, 0, :], h, w_ih, w_hh, b_ih, b_hh)
    _check(got.cpu().numpy(), want, 75, 5.0, 2.0, "fallback")


def test_gates_argument_errors_and_empty_shapes(gpu):
    import torch
    f = gpu
    lib = f.lib()
    buf = torch.zeros(4096, device="cuda")
    p, null = ctypes.c_void_p(buf.data_ptr()), ctypes.c_void_p(0)
    assert lib.fastnn_b200_rnn_gates_forward(p, 16, p, p, p, null, null, p, -1, 16, 16, 64, None) == -1
    assert lib.fastnn_b200_rnn_gates_forward(p, 8, p, p, p, null, null, p, 4, 16, 16, 64, None) == -1   # ld_x
    assert lib.fastnn_b200_rnn_gates_forward(p, 16, null, p, p, null, null, p, 4, 16, 16, 64, None) == -1
    assert lib.fastnn_b200_rnn_gates_forward(p, 16, p, p, p, null, null, p, 0, 16, 16, 64, None) == 0


@pytest.mark.parametrize("shape", [(64, 96, 128), (37, 52, 64), (256, 512, 256)])
def test_gru_step_in_one_launch_with_packed_weights(gpu, shape):
    """GRU::forward_seq (src/nn/rnn.rs:164-180) needs gi_n and gh_n apart; with the parameters
    repacked once (zero blocks opposite the n gate's rows) one gates launch per step returns
    [r and z pre-activations | gi_n | gh_n], and the step computed from it matches the oracle's."""
    import torch
    f = gpu
    batch, inp, hid = shape
    rng = np.random.default_rng(sum(shape))
    x = rng.standard_normal((batch, inp), dtype=np.float32)
    h = rng.standard_normal((batch, hid), dtype=np.float32)
    bound = 1.0 / np.sqrt(hid)
    w_ih = rng.uniform(-bound, bound, (3 * hid, inp)).astype(np.float32)
    w_hh = rng.uniform(-bound, bound, (3 * hid, hid)).astype(np.float32)
    b_ih = rng.uniform(-bound, bound, 3 * hid).astype(np.float32)
    b_hh = rng.uniform(-bound, bound, 3 * hid).astype(np.float32)
    gi, gh = oracle.gru_gates(x, h, w_ih, w_hh, b_ih, b_hh)
    dev = lambda a: torch.from_numpy(a).cuda()
    packed = f.gru_pack_weights(dev(w_ih), dev(w_hh), dev(b_ih), dev(b_hh))
    n0 = f.launch_count()
    gates = f.rnn_gates_forward(dev(x), dev(h), *packed)
    lp = f.last_path()
    assert lp["path"] in (2, 6)
    assert f.launch_count() - n0 == (2 if lp["split_k"] > 1 and lp["path"] == 2 else 1)
    got = gates.cpu().numpy()
    assert got.shape == (batch, 4 * hid)
    amax = max(np.abs(x).max(), np.abs(h).max())
    wmax = max(np.abs(w_ih).max(), np.abs(w_hh).max())
    _check(got[:, :2 * hid], gi[:, :2 * hid] + gh[:, :2 * hid], inp + hid, amax, wmax, "r, z")
    _check(got[:, 2 * hid:3 * hid], gi[:, 2 * hid:], inp, amax, wmax, "gi_n")
    _check(got[:, 3 * hid:], gh[:, 2 * hid:], hid, amax, wmax, "gh_n")
    # the step itself, from the launch's output: 1-Lipschitz gates keep the pre-activation bound
    gi_dev = np.concatenate([got[:, :2 * hid], got[:, 2 * hid:3 * hid]], axis=1)
    gh_dev = np.concatenate([np.zeros((batch, 2 * hid), np.float32), got[:, 3 * hid:]], axis=1)
    h_new = oracle.gru_step(gi_dev, gh_dev, h)
    want = oracle.gru_step(gi, gh, h)
    assert np.abs(h_new - want).max() <= 2e-2 * np.sqrt(inp + hid) * amax * wmax
    assert f.device_status() == 0
