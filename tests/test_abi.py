"""CPU: the C-ABI library builds, loads and exports exactly what include/*.h declares."""
import ctypes
import glob
import os
import re
import subprocess

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_functions():
    names = []
    for hdr in glob.glob(os.path.join(ROOT, "include", "*.h")):
        text = open(hdr).read()
        text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
        names += re.findall(r"FASTNN_B200_API\s+[\w\s\*]+?\b(fastnn_\w+)\s*\(", text)
    return sorted(set(names))


def test_header_declares_the_reference_gemm_family():
    names = _declared_functions()
    for sym in ["fastnn_cuda_init", "fastnn_cuda_device_count", "fastnn_cuda_synchronize",
                "fastnn_cuda_get_memory_info", "fastnn_cuda_malloc", "fastnn_cuda_free",
                "fastnn_cuda_memcpy_h2d", "fastnn_cuda_memcpy_d2h", "fastnn_cuda_memcpy_d2d",
                "fastnn_cuda_memset", "fastnn_cuda_matmul", "fastnn_cuda_matmul_batched",
                "fastnn_cuda_matmul_nt", "fastnn_cuda_matmul_tn", "fastnn_cuda_matmul_batched_nt",
                "fastnn_cuda_matmul_batched_tn"]:
        assert sym in names, sym


def test_library_exports_every_declared_symbol(built_library):
    handle = ctypes.CDLL(built_library)
    for name in _declared_functions():
        assert getattr(handle, name) is not None, name


def test_library_exports_nothing_else(built_library):
    out = subprocess.check_output(["nm", "-D", "--defined-only", built_library], text=True)
    exported = sorted(line.split()[-1] for line in out.splitlines()
                      if " T " in line and not line.split()[-1].startswith("_"))
    assert exported == _declared_functions()


def test_library_does_not_link_cublas_or_the_oracle(built_library):
    out = subprocess.check_output(["ldd", built_library], text=True)
    for banned in ("cublas", "cudnn", "liboracle", "libfastnn_ref"):
        assert banned not in out, banned


def test_python_bindings_cover_every_symbol(built_library):
    from fastnn_b200._lib import SIGNATURES
    assert sorted(SIGNATURES) == _declared_functions()


def test_compute_entries_fail_loudly_without_a_device(built_library):
    import torch
    if torch.cuda.is_available():
        return  # covered by the GPU tests
    import fastnn_b200 as f
    lib = f.lib()
    assert lib.fastnn_cuda_device_count() == 0
    assert lib.fastnn_cuda_init(0) == -1
    # uninitialised context: every GEMM entry reports failure instead of falling back
    null = ctypes.c_void_p(0)
    dummy = ctypes.c_void_p(16)
    assert lib.fastnn_cuda_matmul(dummy, dummy, dummy, 4, 4, 4, 4, 4, 4, 1.0, 0.0) == -1
    assert lib.fastnn_cuda_matmul_nt(dummy, dummy, dummy, 4, 4, 4) == -1
    assert lib.fastnn_cuda_matmul_tn(dummy, dummy, dummy, 4, 4, 4) == -1
    assert lib.fastnn_cuda_matmul_batched(dummy, dummy, dummy, 4, 4, 4, 2, 1.0, 0.0) == -1
    assert lib.fastnn_b200_linear_forward(1, dummy, dummy, null, dummy, 4, 4, 4, 0) == -1


def test_argument_validation(built_library):
    import fastnn_b200 as f
    lib = f.lib()
    dummy = ctypes.c_void_p(16)
    # bad layout / negative sizes / short leading dimension are rejected before any launch
    assert lib.fastnn_b200_gemm_ex(7, dummy, dummy, dummy, 4, 4, 4, 1, 4, 4, 4, 16, 16, 16,
                                   1.0, 0.0, None, 0, None) == -1
    assert lib.fastnn_cuda_matmul(dummy, dummy, dummy, -1, 4, 4, 4, 4, 4, 1.0, 0.0) == -1
    assert lib.fastnn_cuda_matmul(dummy, dummy, dummy, 4, 4, 4, 2, 4, 4, 1.0, 0.0) == -1
    assert lib.fastnn_b200_set_policy(7, 0, 0) == -1
    assert lib.fastnn_b200_set_policy(5, 0, 4) == 0 and lib.fastnn_b200_set_policy(0, 0, 0) == 0
    assert lib.fastnn_b200_set_policy(0, 48, 0) == -1
    assert lib.fastnn_b200_set_policy(0, 0, 0) == 0
    # empty outputs succeed without touching the device
    assert lib.fastnn_cuda_matmul(dummy, dummy, dummy, 0, 4, 4, 4, 4, 4, 1.0, 0.0) == 0


def test_product_sources_never_touch_the_oracle():
    pkg = os.path.join(ROOT, "fastnn_b200")
    for dirpath, _, files in os.walk(pkg):
        for fn in files:
            if fn.endswith((".py", ".cu", ".cuh", ".cpp", ".h")):
                text = open(os.path.join(dirpath, fn), errors="ignore").read()
                assert "oracle" not in text.lower(), os.path.join(dirpath, fn)
