"""GPU: the GEMM whose epilogue also stores every tile to other GPUs' copies of C
(fastnn_b200_gemm_gather_ex).

On one device the "peers" are further buffers of the same GPU: the kernel path (extra tensor maps,
one bulk group of stores per staging tile) is the one the multi-GPU runs take, only the
destination memory differs.  Every destination must equal, bit for bit, what fastnn_b200_gemm_ex
writes for the same arguments; rows outside the shard must stay untouched.  The two-GPU form
over symmetric memory is tested in test_sharding_gpu.py."""
import numpy as np
import pytest

import oracle
from helpers import check_tf32_parity

pytestmark = pytest.mark.gpu

NN, NT, TN = 0, 1, 2


def _operands(layout, m, n, k, batch, seed):
    import torch
    rng = np.random.default_rng(seed)
    sa = (k, m) if layout == TN else (m, k)
    sb = (n, k) if layout == NT else (k, n)
    if batch > 1:
        sa, sb = (batch,) + sa, (batch,) + sb
    a = rng.standard_normal(sa, dtype=np.float32)
    b = rng.standard_normal(sb, dtype=np.float32)
    return a, b, torch.from_numpy(a).cuda(), torch.from_numpy(b).cuda()


def _call(f, layout, da, db, c_ptr, m, n, k, batch, peers, bias=None, act=0):
    lda = m if layout == TN else k
    ldb = k if layout == NT else n
    f.gemm_gather_ex(layout, da.data_ptr(), db.data_ptr(), c_ptr, m, n, k, batch, lda, ldb, n,
                     m * k, k * n, m * n, peers, bias_ptr=bias.data_ptr() if bias is not None else 0, act=act)


@pytest.mark.parametrize("policy", [3, 4])          # single-CTA and CTA-pair kernels
@pytest.mark.parametrize("layout", [NN, NT, TN])
@pytest.mark.parametrize("shape", [(384, 256, 160, 1, 3), (252, 72, 64, 1, 2), (128, 128, 32, 5, 7),
                                   (1024, 512, 512, 1, 1)])
def test_gather_epilogue_writes_every_destination(gpu, layout, shape, policy):
    import torch
    f = gpu
    m, n, k, batch, n_peers = shape
    a, b, da, db = _operands(layout, m, n, k, batch, 11 * m + n + k + layout)
    # every destination is a larger buffer [pad rows | the shard | pad rows]; the shard is written
    # at a row offset, as a rank's rows lie inside the full C
    pad = 3 * n
    bufs = [torch.full((pad + batch * m * n + pad,), float("nan"), device="cuda") for _ in range(n_peers + 1)]
    want = torch.empty(batch * m * n, device="cuda")
    lda = m if layout == TN else k
    ldb = k if layout == NT else n
    f.set_policy(policy, 0, 0)
    try:
        f.gemm_ex(layout, da.data_ptr(), db.data_ptr(), want.data_ptr(), m, n, k, batch, lda, ldb, n,
                  m * k, k * n, m * n)
        plain_path = f.last_path()
        _call(f, layout, da, db, bufs[0].data_ptr() + 4 * pad, m, n, k, batch,
              [bf.data_ptr() + 4 * pad for bf in bufs[1:]])
    finally:
        f.set_policy(0, 0, 0)
    assert f.last_path()["path"] == policy - 1
    assert f.last_path()["split_k"] == 1, "a gathered tile holds the whole K range"
    torch.cuda.synchronize()
    for i, bf in enumerate(bufs):
        assert torch.isnan(bf[:pad]).all() and torch.isnan(bf[-pad:]).all(), f"destination {i}: wrote outside"
        if plain_path["split_k"] == 1:
            assert torch.equal(bf[pad:-pad], want), f"destination {i} differs from the plain GEMM"
        else:       # the plain call split K: same product, other summation order
            assert torch.allclose(bf[pad:-pad], want, rtol=1e-4, atol=1e-3)
        assert torch.equal(bf[pad:-pad], bufs[0][pad:-pad])
    ref = [oracle.matmul, oracle.matmul_nt, oracle.matmul_tn][layout](a, b)
    check_tf32_parity(bufs[-1][pad:-pad].cpu().numpy().reshape(ref.shape), ref, k, a, b, what=f"gather {shape}")
    assert f.device_status() == 0


@pytest.mark.parametrize("act", [0, 1, 2])
def test_gather_with_bias_and_activation(gpu, act):
    """The by-column epilogue (bias, ReLU, erf-GELU) stores to the peers too."""
    import torch
    f = gpu
    m, n, k = 640, 384, 256
    a, b, da, db = _operands(NN, m, n, k, 1, 99)
    bias_h = np.random.default_rng(5).standard_normal(n).astype(np.float32)
    bias = torch.from_numpy(bias_h).cuda()
    bufs = [torch.full((m * n,), float("nan"), device="cuda") for _ in range(8)]      # 7 peers: the maximum
    _call(f, NN, da, db, bufs[0].data_ptr(), m, n, k, 1, [bf.data_ptr() for bf in bufs[1:]], bias=bias, act=act)
    f.set_policy(6, 0, 1)           # no K split: the summation order of a gathered tile
    try:
        want = f.linear_forward(da, db, bias, act=act, layout=f.NN)
    finally:
        f.set_policy(0, 0, 0)
    torch.cuda.synchronize()
    for bf in bufs:
        assert torch.equal(bf.view(m, n), want)
    ref = oracle.bias_act(oracle.matmul(a, b), bias_h, act)
    assert np.abs(want.cpu().numpy() - ref).max() <= 1e-2 * np.sqrt(k) * np.abs(a).max() * np.abs(b).max()


@pytest.mark.parametrize("layout", [NN, TN])
def test_gather_of_shapes_tma_cannot_address_goes_by_copies(gpu, layout):
    """Row lengths that are not multiples of four floats, a destination that is only 4-byte
    aligned: the ordinary GEMM (SIMT kernel here) plus one strided copy per destination."""
    import torch
    f = gpu
    m, n, k = 250, 70, 45
    a, b, da, db = _operands(layout, m, n, k, 1, 61)
    bufs = [torch.full((m * n + 8,), float("nan"), device="cuda") for _ in range(3)]
    _call(f, layout, da, db, bufs[0].data_ptr(), m, n, k, 1, [bufs[1].data_ptr(), bufs[2].data_ptr() + 4])
    torch.cuda.synchronize()
    ref = [oracle.matmul, oracle.matmul_nt, oracle.matmul_tn][layout](a, b)
    for bf, off in ((bufs[0], 0), (bufs[1], 0), (bufs[2], 1)):
        got = bf[off: off + m * n].cpu().numpy().reshape(m, n)
        check_tf32_parity(got, ref, k, a, b, what="gather by copies")
        assert torch.isnan(bf[off + m * n:]).all()
    assert f.device_status() == 0


def test_gather_argument_errors(gpu):
    import torch
    f = gpu
    a, b, da, db = _operands(NN, 128, 128, 32, 1, 3)
    c = torch.empty(128 * 128 + 1, device="cuda")
    good = torch.empty(128 * 128, device="cuda")
    with pytest.raises(f.CudaError):        # more than seven peers
        _call(f, NN, da, db, good.data_ptr(), 128, 128, 32, 1, [good.data_ptr()] * 8)
    with pytest.raises(f.CudaError):        # null peer
        _call(f, NN, da, db, good.data_ptr(), 128, 128, 32, 1, [0])
    assert f.device_status() == 0
