"""GPU: the fused attention core against the CPU composition FastNN runs
(matmul -> scale -> additive causal mask -> softmax -> matmul; src/nn/transformer.rs:87-115).

Tolerance: both products are TF32 and the scores pass through exp, so the bar is the GEMM one
applied to the output with K = t_k and the softmax weights (<= 1) as the left operand:
relative Frobenius <= 5e-3, max-abs <= 1e-2 * sqrt(t_k) * max|V|."""
import ctypes

import numpy as np
import pytest

import oracle

pytestmark = pytest.mark.gpu


def _run(f, q, k, v, scale, causal):
    import torch
    out = f.attention_forward(torch.from_numpy(q).cuda(), torch.from_numpy(k).cuda(),
                              torch.from_numpy(v).cuda(), scale=scale, causal=causal)
    torch.cuda.synchronize()
    return out.cpu().numpy()


def _check(got, want, tk, v, what):
    assert np.isfinite(got).all(), what
    err = got.astype(np.float64) - want
    rel = np.linalg.norm(err) / np.linalg.norm(want)
    assert rel <= 5e-3, f"{what}: relative Frobenius {rel:.2e}"
    assert np.abs(err).max() <= 1e-2 * np.sqrt(tk) * np.abs(v).max(), what


@pytest.mark.parametrize("causal", [True, False])
@pytest.mark.parametrize("shape", [
    (6, 128, 128, 32),      # the configured attention shape (few heads)
    (3, 64, 64, 32),        # tile tails: fewer queries and keys than a tile
    (2, 200, 136, 32),      # t_q over two tiles, ragged t_k
    (2, 128, 192, 32),      # long key range: single-buffered operands
    (2, 96, 64, 64),        # two 32-wide head-dim blocks
    (1, 40, 8, 32),         # t_k smaller than one block
    (5, 130, 96, 96),
    (2, 128, 256, 64),      # longest key range: one score tile fills half of TMEM
    (300, 128, 128, 32),    # more units than SMs: the per-CTA pipeline runs several deep
])
def test_fused_attention_matches_reference_composition(gpu, shape, causal):
    f = gpu
    heads, tq, tk, d = shape
    rng = np.random.default_rng(heads * 1000 + tq + tk + d + int(causal))
    q = rng.standard_normal((heads, tq, d), dtype=np.float32)
    k = rng.standard_normal((heads, tk, d), dtype=np.float32)
    v = rng.standard_normal((heads, tk, d), dtype=np.float32)
    scale = 1.0 / np.sqrt(d)
    got = _run(f, q, k, v, scale, causal)
    want = oracle.attention(q, k, v, scale, causal)
    _check(got, want, tk, v, f"{shape} causal={causal}")
    assert f.last_path()["path"] == 4
    assert f.device_status() == 0


def test_fused_attention_full_config_and_determinism(gpu):
    """512 heads, T = 128, head_dim 32, causal: the configured batched-attention case."""
    import torch
    f = gpu
    rng = np.random.default_rng(3000)
    q = rng.standard_normal((512, 128, 32), dtype=np.float32)
    k = rng.standard_normal((512, 128, 32), dtype=np.float32)
    v = rng.standard_normal((512, 128, 32), dtype=np.float32)
    scale = 1.0 / np.sqrt(32.0)
    got = _run(f, q, k, v, scale, True)
    _check(got, oracle.attention(q, k, v, scale, True), 128, v, "512x128x128x32")
    assert np.array_equal(got, _run(f, q, k, v, scale, True))
    # causal: output row 0 of every head is exactly v[0] (one visible key, weight 1)
    assert np.allclose(got[:, 0, :], v[:, 0, :], rtol=2e-3, atol=1e-6)


def test_fused_attention_agrees_with_the_unfused_gpu_path(gpu):
    """Same result, within TF32 tolerance, as composing it from the GEMM entries on the GPU."""
    import torch
    f = gpu
    g = torch.Generator(device="cuda").manual_seed(5)
    q = torch.randn(16, 128, 32, device="cuda", generator=g)
    k = torch.randn(16, 128, 32, device="cuda", generator=g)
    v = torch.randn(16, 128, 32, device="cuda", generator=g)
    scale = 1.0 / np.sqrt(32.0)
    s = f.matmul_nt(q, k) * scale
    mask = torch.triu(torch.full((128, 128), -1e9, device="cuda"), diagonal=1)
    p = torch.softmax(s + mask, dim=-1)
    want = f.matmul(p, v).cpu().numpy().astype(np.float64)
    got = f.attention_forward(q, k, v, scale=scale, causal=True).cpu().numpy()
    _check(got, want, 128, v.cpu().numpy(), "fused vs unfused GPU")


def _operands(heads, tq, tk, d, seed):
    rng = np.random.default_rng(seed)
    return (rng.standard_normal((heads, tq, d), dtype=np.float32),
            rng.standard_normal((heads, tk, d), dtype=np.float32),
            rng.standard_normal((heads, tk, d), dtype=np.float32))


@pytest.mark.parametrize("causal", [True, False])
@pytest.mark.parametrize("shape", [(6, 128, 128, 32), (3, 200, 136, 64), (2, 64, 40, 32)])
def test_fused_attention_with_an_additive_mask(gpu, shape, causal):
    """A general additive [t_q, t_k] mask (the form of FastNN's cached mask tensor,
    src/nn/transformer.rs:15-30, 99-105) inside the fused kernel: finite biases and -1e9 entries,
    one row hidden completely except one key."""
    import torch
    f = gpu
    heads, tq, tk, d = shape
    q, k, v = _operands(heads, tq, tk, d, sum(shape) + int(causal))
    rng = np.random.default_rng(77)
    mask = rng.standard_normal((tq, tk)).astype(np.float32)
    mask[rng.random((tq, tk)) < 0.2] = -1e9
    mask[:, 0] = 0.0                                    # every query keeps one visible key
    mask[5, 1:] = -1e9
    scale = 1.0 / np.sqrt(d)
    got = f.attention_forward(torch.from_numpy(q).cuda(), torch.from_numpy(k).cuda(), torch.from_numpy(v).cuda(),
                              scale=scale, causal=causal, mask=torch.from_numpy(mask).cuda())
    assert f.last_path()["path"] == 4
    want = oracle.attention(q, k, v, scale, causal, mask=mask)
    _check(got.cpu().numpy(), want, tk, v, f"masked {shape} causal={causal}")
    assert np.allclose(got.cpu().numpy()[:, 5, :], v[:, 0, :], rtol=2e-3, atol=1e-6)
    assert f.device_status() == 0


@pytest.mark.parametrize("shape", [
    (2, 300, 300, 32),      # more keys than the fused kernel's 256
    (3, 128, 1024, 64),     # long key range
    (2, 50, 70, 48),        # head_dim not a multiple of 32
    (2, 33, 17, 20),        # nothing aligned for TMA: both GEMMs on the SIMT kernel
    (4, 128, 128, 160),     # head_dim above 128
])
def test_attention_outside_the_fused_kernel_is_composed_from_the_gemms(gpu, shape):
    """What the fused kernel does not cover runs FastNN's own composition (batched scale * Q.K^T,
    masked row softmax, batched P.V) on this library's kernels -- no shape is refused."""
    import torch
    f = gpu
    heads, tq, tk, d = shape
    q, k, v = _operands(heads, tq, tk, d, sum(shape))
    scale = 1.0 / np.sqrt(d)
    for causal, use_mask in ((True, False), (False, True), (False, False)):
        mask = None
        if use_mask:
            mask = np.random.default_rng(5).standard_normal((tq, tk)).astype(np.float32)
        got = f.attention_forward(torch.from_numpy(q).cuda(), torch.from_numpy(k).cuda(),
                                  torch.from_numpy(v).cuda(), scale=scale, causal=causal,
                                  mask=None if mask is None else torch.from_numpy(mask).cuda())
        assert f.last_path()["path"] == 8
        want = oracle.attention(q, k, v, scale, causal, mask=mask)
        _check(got.cpu().numpy(), want, tk, v, f"composed {shape} causal={causal} mask={use_mask}")
    assert f.device_status() == 0


def test_reference_symbol_returns_output_and_probabilities(gpu):
    """fastnn_cuda_scaled_dot_product_attention with FastNN's argument list: output and
    attn_weights, with a causal flag and a mask that take effect (FastNN's entry ignores both)."""
    import torch
    f = gpu
    lib = f.lib()
    batch, nheads, tq, tk, d = 2, 3, 96, 96, 32
    q, k, v = _operands(batch * nheads, tq, tk, d, 41)
    mask = np.random.default_rng(6).standard_normal((tq, tk)).astype(np.float32)
    scale = 1.0 / np.sqrt(d)
    dq, dk, dv, dm = (torch.from_numpy(t).cuda() for t in (q, k, v, mask))
    vp = lambda t: ctypes.c_void_p(t.data_ptr() if t is not None else 0)
    for causal, m, dmask in ((1, None, None), (0, mask, dm), (1, mask, dm)):
        o = torch.full((batch * nheads, tq, d), float("nan"), device="cuda")
        w = torch.full((batch * nheads, tq, tk), float("nan"), device="cuda")
        assert lib.fastnn_cuda_scaled_dot_product_attention(vp(dq), vp(dk), vp(dv), vp(o), vp(w), vp(dmask), batch,
                                                            nheads, tq, tk, d, scale, causal) == 0
        torch.cuda.synchronize()
        want_o, want_w = oracle.attention(q, k, v, scale, bool(causal), mask=m, return_weights=True)
        _check(o.cpu().numpy(), want_o, tk, v, f"reference symbol causal={causal}")
        wg = w.cpu().numpy()
        assert np.abs(wg - want_w).max() <= 2e-3              # probabilities from TF32 scores
        assert np.abs(wg.sum(-1) - 1.0).max() <= 1e-5
        if causal:
            iu = np.triu_indices(tq, 1)
            assert (wg[:, iu[0], iu[1]] == 0.0).all()
    # without attn_weights the same symbol takes the fused kernel
    o = torch.empty((batch * nheads, tq, d), device="cuda")
    assert lib.fastnn_cuda_scaled_dot_product_attention(vp(dq), vp(dk), vp(dv), vp(o), None, None, batch, nheads,
                                                        tq, tk, d, scale, 1) == 0
    assert f.last_path()["path"] == 4
    _check(o.cpu().numpy(), oracle.attention(q, k, v, scale, True), tk, v, "reference symbol, fused")
    assert f.device_status() == 0


def test_attention_checks_its_arguments(gpu):
    import torch
    f = gpu
    lib = f.lib()
    t = torch.zeros(1024, device="cuda")
    p = ctypes.c_void_p(t.data_ptr())
    assert lib.fastnn_b200_attention_forward(p, p, p, p, 1, 16, 0, 32, 1.0, 0, None) == -1    # no keys
    assert lib.fastnn_b200_attention_forward(p, p, p, p, 1, 16, 16, 0, 1.0, 0, None) == -1    # head_dim
    assert lib.fastnn_b200_attention_forward(p, p, p, None, 1, 16, 16, 32, 1.0, 0, None) == -1  # null output
    assert lib.fastnn_b200_attention_forward(p, p, p, p, 0, 16, 16, 32, 1.0, 0, None) == 0    # empty
