"""ctypes loader for libfastnn_b200.so.  Fails loudly when the library is absent."""
from __future__ import annotations

import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
_PATH = os.path.join(_HERE, "libfastnn_b200.so")
_lib = None

c_fp = ctypes.POINTER(ctypes.c_float)
_i, _f, _ll, _vp = ctypes.c_int, ctypes.c_float, ctypes.c_longlong, ctypes.c_void_p


class LibraryMissing(RuntimeError):
    pass


def library_path() -> str:
    return _PATH


# name -> (restype, argtypes); pointers to device memory are passed as void* integers
SIGNATURES = {
    "fastnn_cuda_init": (_i, [_i]),
    "fastnn_cuda_device_count": (_i, []),
    "fastnn_cuda_synchronize": (_i, []),
    "fastnn_cuda_get_memory_info": (None, [ctypes.POINTER(ctypes.c_size_t)] * 2),
    "fastnn_cuda_malloc": (_i, [ctypes.POINTER(_vp), ctypes.c_size_t]),
    "fastnn_cuda_free": (_i, [_vp]),
    "fastnn_cuda_memcpy_h2d": (_i, [_vp, _vp, ctypes.c_size_t]),
    "fastnn_cuda_memcpy_d2h": (_i, [_vp, _vp, ctypes.c_size_t]),
    "fastnn_cuda_memcpy_d2d": (_i, [_vp, _vp, ctypes.c_size_t]),
    "fastnn_cuda_memset": (_i, [_vp, _i, ctypes.c_size_t]),
    "fastnn_cuda_matmul": (_i, [_vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _f, _f]),
    "fastnn_cuda_matmul_batched": (_i, [_vp, _vp, _vp, _i, _i, _i, _i, _f, _f]),
    "fastnn_cuda_matmul_nt": (_i, [_vp, _vp, _vp, _i, _i, _i]),
    "fastnn_cuda_matmul_tn": (_i, [_vp, _vp, _vp, _i, _i, _i]),
    "fastnn_cuda_matmul_batched_nt": (_i, [_vp, _vp, _vp, _i, _i, _i, _i]),
    "fastnn_cuda_matmul_batched_tn": (_i, [_vp, _vp, _vp, _i, _i, _i, _i]),
    "fastnn_b200_gemm_ex": (_i, [_i, _vp, _vp, _vp, _i, _i, _i, _i, _ll, _ll, _ll, _ll, _ll, _ll,
                                 _f, _f, _vp, _i, _vp]),
    "fastnn_b200_linear_forward": (_i, [_i, _vp, _vp, _vp, _vp, _i, _i, _i, _i]),
    "fastnn_b200_linear_backward_input": (_i, [_i, _vp, _vp, _vp, _i, _i, _i, _i, _vp, _vp, _vp]),
    "fastnn_b200_rnn_gates_forward": (_i, [_vp, _ll, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _vp]),
    "fastnn_b200_memcpy_h2d_async": (_i, [_vp, _vp, ctypes.c_size_t, _vp]),
    "fastnn_b200_memcpy_d2h_async": (_i, [_vp, _vp, ctypes.c_size_t, _vp]),
    "fastnn_b200_memcpy_d2d_async": (_i, [_vp, _vp, ctypes.c_size_t, _vp]),
    "fastnn_cuda_conv2d_forward": (_i, [_vp, _vp, _vp, _vp] + [_i] * 11),
    "fastnn_b200_conv2d_forward": (_i, [_vp, _vp, _vp, _vp] + [_i] * 12 + [_vp]),
    "fastnn_cuda_conv2d_backward_data": (_i, [_vp, _vp, _vp] + [_i] * 13),
    "fastnn_b200_conv2d_backward_data": (_i, [_vp, _vp, _vp] + [_i] * 13 + [_vp]),
    "fastnn_cuda_conv2d_backward_weight": (_i, [_vp, _vp, _vp] + [_i] * 13),
    "fastnn_b200_conv2d_backward_weight": (_i, [_vp, _vp, _vp] + [_i] * 13 + [_vp]),
    "fastnn_b200_gemm_splitk_static": (_i, [_i, _vp, _vp, _vp, _i, _i, _i, _i, _vp]),
    "fastnn_b200_attention_forward": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _f, _i, _vp]),
    "fastnn_b200_attention_forward_ex": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _f, _i, _vp]),
    "fastnn_cuda_scaled_dot_product_attention": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _f, _i]),
    "fastnn_b200_gemm_gather_ex": (_i, [_i, _vp, _vp, _vp, _i, _i, _i, _i, _ll, _ll, _ll, _ll, _ll, _ll,
                                        _f, _vp, _i, ctypes.POINTER(_vp), _i, _vp]),
    "fastnn_b200_gemm_gather_mc_ex": (_i, [_i, _vp, _vp, _vp, _i, _i, _i, _i, _ll, _ll, _ll, _ll, _ll, _ll,
                                           _f, _vp, _i, _vp, _vp]),
    "fastnn_b200_selftest_bounded_wait": (_i, [ctypes.c_uint, ctypes.POINTER(ctypes.c_uint)]),
    "fastnn_b200_reduce_partials": (_i, [_vp, _vp, _i, _i, _i, _ll, _f, _f, _vp, _i, _vp]),
    "fastnn_b200_set_policy": (_i, [_i, _i, _i]),
    "fastnn_b200_last_path": (_i, [ctypes.POINTER(_i)] * 3),
    "fastnn_b200_plan_query": (_i, [_i] * 5 + [ctypes.POINTER(_i)] * 4),
    "fastnn_b200_device_status": (_i, [ctypes.POINTER(ctypes.c_uint)]),
    "fastnn_b200_launch_count": (ctypes.c_ulonglong, []),
    "fastnn_b200_version": (ctypes.c_char_p, []),
}


def lib() -> ctypes.CDLL:
    """The loaded library.  Raises LibraryMissing if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(_PATH):
            raise LibraryMissing(
                f"{_PATH} not found: build it with `python -m fastnn_b200.build` "
                "(there is no CPU or library fallback for the GEMM path)")
        handle = ctypes.CDLL(_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)      # AttributeError here = ABI drift, by design
            fn.restype = res
            fn.argtypes = args
        _lib = handle
    return _lib
