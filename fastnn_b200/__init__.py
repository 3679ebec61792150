"""fastnn_b200 -- FastNN's matrix-multiply path on B200 (sm_100a).

The product is ``libfastnn_b200.so`` (C ABI in ``include/fastnn_b200_kernels.h``).  This
package loads it and offers the thin host wrappers FastNN's ``cuda_backend`` module has
(``cuda_matmul``, ``cuda_matmul_nt`` ...), operating on torch CUDA tensors.  There is no
CPU fallback: importing works anywhere, computing needs the library and a B200.
"""
from ._lib import LibraryMissing, lib, library_path  # noqa: F401
from .cuda_backend import (  # noqa: F401
    ACT_GELU, ACT_NONE, ACT_RELU, NN, NT, TN, CudaError, attention_forward, conv2d_backward, conv2d_forward, cuda_init, cuda_matmul, cuda_matmul_batched,
    cuda_matmul_batched_nt, cuda_matmul_batched_tn, cuda_matmul_nt, cuda_matmul_tn, device_status,
    current_stream_ptr, gemm_ex, gemm_gather_ex, gemm_gather_mc_ex, gemm_splitk_static, selftest_bounded_wait, gru_pack_weights, last_path, reduce_partials, launch_count, linear_backward_input, linear_forward, matmul, matmul_nt, matmul_tn, plan_query, rnn_gates_forward, set_policy,
    synchronize,
)

__all__ = [n for n in dir() if not n.startswith("_")]
