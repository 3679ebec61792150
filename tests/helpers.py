"""Shared parity criteria for the GEMM tests."""
import numpy as np

# BASELINE tolerance for TF32 multiply / FP32 accumulate against the FP32 CPU oracle.
REL_FRO_TOL = 5e-3


def maxabs_bound(k, a, b):
    """1e-2 * sqrt(K) * max|A| * max|B|."""
    return 1e-2 * np.sqrt(max(k, 1)) * float(np.abs(a).max()) * float(np.abs(b).max())


def check_tf32_parity(got, want, k, a, b, what=""):
    got = np.asarray(got, dtype=np.float64)
    want = np.asarray(want, dtype=np.float64)
    assert got.shape == want.shape, f"{what}: shape {got.shape} vs {want.shape}"
    assert np.isfinite(got).all(), f"{what}: non-finite output"
    err = got - want
    denom = np.linalg.norm(want.ravel())
    rel = np.linalg.norm(err.ravel()) / denom if denom > 0 else np.linalg.norm(err.ravel())
    mx = float(np.abs(err).max()) if err.size else 0.0
    bound = maxabs_bound(k, a, b)
    assert rel <= REL_FRO_TOL, f"{what}: relative Frobenius error {rel:.3e} > {REL_FRO_TOL}"
    assert mx <= bound, f"{what}: max-abs error {mx:.3e} > bound {bound:.3e}"
    return rel, mx


def reference_assert_close(cpu, gpu, rtol=2e-2, atol=2e-3, what=""):
    """The element rule of FastNN's tests/cuda_parity.rs:50-58 (TF32_RTOL, ATOL :109-111)."""
    cpu = np.asarray(cpu, dtype=np.float32).ravel()
    gpu = np.asarray(gpu, dtype=np.float32).ravel()
    assert cpu.shape == gpu.shape, f"{what}: length mismatch"
    diff = np.abs(cpu - gpu)
    denom = np.maximum(np.maximum(np.abs(cpu), np.abs(gpu)), 1.0)
    bad = ~((diff <= atol) | (diff / denom <= rtol))
    assert not bad.any(), f"{what}: mismatch at {np.flatnonzero(bad)[:5]}"
