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


def test_fused_attention_rejects_what_it_does_not_cover(gpu):
    import torch
    f = gpu
    lib = f.lib()
    t = torch.zeros(4 * 300 * 48, device="cuda")
    p = ctypes.c_void_p(t.data_ptr())
    assert lib.fastnn_b200_attention_forward(p, p, p, p, 1, 16, 16, 48, 1.0, 0, None) == -1   # head_dim
    assert lib.fastnn_b200_attention_forward(p, p, p, p, 1, 16, 300, 32, 1.0, 0, None) == -1  # t_k
    assert lib.fastnn_b200_attention_forward(p, p, p, p, 1, 16, 256, 128, 1.0, 0, None) == -1  # smem
    assert lib.fastnn_b200_attention_forward(p, p, p, p, 1, 16, 16, 32, 0.0, 0, None) == -1   # scale
    assert lib.fastnn_b200_attention_forward(p, p, p, p, 0, 16, 16, 32, 1.0, 0, None) == 0    # empty
