"""numpy-facing wrapper over ``liboracle.so`` (TEST INFRASTRUCTURE ONLY).

Each function mirrors one CPU arm of FastNN's ``Tensor`` API; the C source cites
the reference lines.  Inputs are C-contiguous float32 numpy arrays.
"""
from __future__ import annotations

import ctypes
import os

import numpy as np

from . import build_oracle as _b

__all__ = [
    "rand_data", "matmul", "matmul_nt", "matmul_tn", "matmul_rows", "transpose",
    "bias_act", "linear", "linear_backward_input", "rnn_gates", "gru_gates", "gru_step", "conv2d", "conv2d_backward", "causal_softmax", "attention", "host_threads", "ACT_NONE", "ACT_RELU",
    "ACT_GELU", "ref_gpu_library_path",
]

ACT_NONE, ACT_RELU, ACT_GELU = 0, 1, 2

_lib = None
_fp = ctypes.POINTER(ctypes.c_float)
_sz = ctypes.c_size_t


def _load():
    global _lib
    if _lib is None:
        path = _b.build_oracle()
        lib = ctypes.CDLL(path)
        lib.oracle_rand_data.argtypes = [_fp, _sz, ctypes.c_uint64]
        lib.oracle_rand_data.restype = None
        lib.oracle_matmul_nn.argtypes = [_fp, _fp, _fp, _sz, _sz, _sz]
        lib.oracle_matmul_nn.restype = None
        lib.oracle_matmul_nn_rows.argtypes = [_fp, _fp, _fp, _sz, _sz, _sz, _sz]
        lib.oracle_matmul_nn_rows.restype = None
        lib.oracle_matmul_nn_rows_par.argtypes = [_fp, _fp, _fp, _sz, _sz, _sz, _sz, ctypes.c_int]
        lib.oracle_matmul_nn_rows_par.restype = ctypes.c_int
        lib.oracle_transpose.argtypes = [_fp, _fp, _sz, _sz, _sz]
        lib.oracle_transpose.restype = None
        lib.oracle_matmul_batched.argtypes = [_fp, _fp, _fp, _sz, _sz, _sz, _sz, _sz]
        lib.oracle_matmul_batched.restype = None
        lib.oracle_matmul_nt.argtypes = [_fp, _fp, _fp, _sz, _sz, _sz, _sz]
        lib.oracle_matmul_nt.restype = ctypes.c_int
        lib.oracle_matmul_tn.argtypes = [_fp, _fp, _fp, _sz, _sz, _sz, _sz]
        lib.oracle_matmul_tn.restype = ctypes.c_int
        lib.oracle_bias_act.argtypes = [_fp, _fp, _sz, _sz, ctypes.c_int]
        lib.oracle_bias_act.restype = None
        lib.oracle_linear.argtypes = [_fp, _fp, _fp, _fp, _sz, _sz, _sz, ctypes.c_int]
        lib.oracle_linear.restype = ctypes.c_int
        lib.oracle_causal_softmax.argtypes = [_fp, _sz, _sz, ctypes.c_float]
        lib.oracle_causal_softmax.restype = None
        _lib = lib
    return _lib


def _p(a: np.ndarray):
    assert a.dtype == np.float32 and a.flags["C_CONTIGUOUS"], "oracle wants contiguous float32"
    return a.ctypes.data_as(_fp)


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


def host_threads() -> int:
    """Threads available to this process (what the row-parallel twin uses)."""
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:  # pragma: no cover
        return max(1, os.cpu_count() or 1)


def rand_data(n: int, seed: int) -> np.ndarray:
    """SplitMix64 uniform [-1,1) fixture generator of the reference's tests."""
    out = np.empty(int(n), dtype=np.float32)
    _load().oracle_rand_data(_p(out), int(n), ctypes.c_uint64(seed & 0xFFFFFFFFFFFFFFFF))
    return out


def transpose(a: np.ndarray) -> np.ndarray:
    a = _f32(a)
    rows, cols = a.shape[-2:]
    outer = int(np.prod(a.shape[:-2], dtype=np.int64)) if a.ndim > 2 else 1
    out = np.empty(a.shape[:-2] + (cols, rows), dtype=np.float32)
    _load().oracle_transpose(_p(a), _p(out), outer, rows, cols)
    return out


def matmul(a: np.ndarray, b: np.ndarray, threads: int = 1) -> np.ndarray:
    """``Tensor::matmul`` on CPU tensors: 2-D, or batched with batch-1 broadcast."""
    a, b = _f32(a), _f32(b)
    lib = _load()
    if a.ndim == 2 and b.ndim == 2:
        m, k = a.shape
        k2, n = b.shape
        assert k == k2, f"Matmul shape mismatch: {a.shape} x {b.shape}"
        c = np.empty((m, n), dtype=np.float32)
        if threads > 1:
            rc = lib.oracle_matmul_nn_rows_par(_p(a), _p(b), _p(c), n, k, 0, m, threads)
            assert rc == 0
        else:
            lib.oracle_matmul_nn(_p(a), _p(b), _p(c), m, n, k)
        return c
    m, k = a.shape[-2:]
    k2, n = b.shape[-2:]
    assert k == k2, "Matmul shape mismatch"
    ab = int(np.prod(a.shape[:-2], dtype=np.int64))
    bb = int(np.prod(b.shape[:-2], dtype=np.int64))
    assert ab == bb or ab == 1 or bb == 1, "Batch dimensions must match or be broadcastable"
    c = np.empty(a.shape[:-2] + (m, n), dtype=np.float32) if ab >= bb else \
        np.empty(b.shape[:-2] + (m, n), dtype=np.float32)
    lib.oracle_matmul_batched(_p(a), _p(b), _p(c), m, n, k, ab, bb)
    return c


def matmul_rows(a: np.ndarray, b: np.ndarray, row0: int, row1: int, threads: int = 1) -> np.ndarray:
    """Rows [row0,row1) of the 2-D NN product (bounded CPU sample of a large GEMM)."""
    a, b = _f32(a), _f32(b)
    m, k = a.shape
    n = b.shape[1]
    assert 0 <= row0 <= row1 <= m
    c = np.empty((m, n), dtype=np.float32) if False else np.empty((row1 - row0, n), dtype=np.float32)
    # the C routine indexes C by absolute row, so hand it a pointer shifted back by row0 rows
    base = c.ctypes.data - row0 * n * 4
    cptr = ctypes.cast(ctypes.c_void_p(base), _fp)
    lib = _load()
    if threads > 1:
        rc = lib.oracle_matmul_nn_rows_par(_p(a), _p(b), cptr, n, k, row0, row1, threads)
        assert rc == 0
    else:
        lib.oracle_matmul_nn_rows(_p(a), _p(b), cptr, n, k, row0, row1)
    return c


def matmul_nt(a: np.ndarray, b: np.ndarray) -> np.ndarray:
    """``Tensor::matmul_nt`` CPU arm: a[..,m,k] . transpose(b[..,n,k])."""
    a, b = _f32(a), _f32(b)
    m, k = a.shape[-2:]
    n, k2 = b.shape[-2:]
    assert k == k2
    batch = int(np.prod(a.shape[:-2], dtype=np.int64)) if a.ndim > 2 else 1
    c = np.empty(a.shape[:-2] + (m, n), dtype=np.float32)
    assert _load().oracle_matmul_nt(_p(a), _p(b), _p(c), m, n, k, batch) == 0
    return c


def matmul_tn(a: np.ndarray, b: np.ndarray) -> np.ndarray:
    """``Tensor::matmul_tn`` CPU arm: transpose(a[..,k,m]) . b[..,k,n]."""
    a, b = _f32(a), _f32(b)
    k, m = a.shape[-2:]
    k2, n = b.shape[-2:]
    assert k == k2
    batch = int(np.prod(a.shape[:-2], dtype=np.int64)) if a.ndim > 2 else 1
    c = np.empty(a.shape[:-2] + (m, n), dtype=np.float32)
    assert _load().oracle_matmul_tn(_p(a), _p(b), _p(c), m, n, k, batch) == 0
    return c


def bias_act(c: np.ndarray, bias, act: int = ACT_NONE) -> np.ndarray:
    """Row-broadcast bias add followed by none/ReLU/erf-GELU (returns a new array)."""
    out = _f32(c).copy()
    n = out.shape[-1]
    rows = out.size // n if n else 0
    bp = _p(_f32(bias)) if bias is not None else ctypes.cast(None, _fp)
    _load().oracle_bias_act(_p(out), bp, rows, n, act)
    return out


def linear(x: np.ndarray, w: np.ndarray, bias, act: int = ACT_NONE) -> np.ndarray:
    """``Linear::forward`` (+ optional activation): x[batch,in] . W[out,in]^T + bias."""
    x, w = _f32(x), _f32(w)
    batch, in_f = x.shape
    out_f, in2 = w.shape
    assert in_f == in2
    y = np.empty((batch, out_f), dtype=np.float32)
    bp = _p(_f32(bias)) if bias is not None else ctypes.cast(None, _fp)
    assert _load().oracle_linear(_p(x), _p(w), bp, _p(y), batch, in_f, out_f, act) == 0
    return y


def linear_backward_input(dy: np.ndarray, w: np.ndarray, pre, act: int = ACT_NONE):
    """Gradient flowing into the previous layer's pre-activation, as FastNN's tape computes it
    on CPU tensors: MatmulBackward's grad_a = matmul_nt(dy, W^T) for y = x . W^T
    (i.e. dy[rows,out] . W[out,in]), then ReluBackward / GeluBackward against the saved
    pre-activation ``pre[rows,in]``, then the row sum that is that layer's bias gradient.
    Returns (dx[rows,in], colsum[in])."""
    dy, w = _f32(dy), _f32(w)
    dx = matmul(dy, w).copy()
    rows, n = dx.shape
    colsum = np.empty(n, dtype=np.float32)
    lib = _load()
    lib.oracle_act_backward_colsum.argtypes = [_fp, _fp, _fp, _sz, _sz, ctypes.c_int]
    lib.oracle_act_backward_colsum.restype = None
    pre32 = _f32(pre) if pre is not None else None        # kept alive across the call
    xp = _p(pre32) if pre32 is not None else ctypes.cast(None, _fp)
    lib.oracle_act_backward_colsum(_p(dx), xp, _p(colsum), rows, n, act if pre is not None else 0)
    return dx, colsum


def conv2d(x: np.ndarray, w: np.ndarray, bias, stride=(1, 1), padding=(0, 0)) -> np.ndarray:
    """``Conv2d::forward`` on CPU tensors (src/nn/conv.rs:97-123): x [N,Cin,H,W], w [Cout,Cin,KH,KW]."""
    x, w = _f32(x), _f32(w)
    n, ci, h, wd = x.shape
    co, ci2, kh, kw = w.shape
    assert ci == ci2
    (sh, sw), (ph, pw) = stride, padding
    oh, ow = (h + 2 * ph - kh) // sh + 1, (wd + 2 * pw - kw) // sw + 1
    out = np.empty((n, co, oh, ow), dtype=np.float32)
    b32 = _f32(bias) if bias is not None else None
    bp = _p(b32) if b32 is not None else ctypes.cast(None, _fp)
    lib = _load()
    lib.oracle_conv2d_forward.argtypes = [_fp, _fp, _fp, _fp] + [_sz] * 11
    lib.oracle_conv2d_forward.restype = None
    lib.oracle_conv2d_forward(_p(x), _p(w), bp, _p(out), n, ci, co, h, wd, kh, kw, sh, sw, ph, pw)
    return out


def conv2d_backward(x: np.ndarray, w: np.ndarray, go: np.ndarray, stride=(1, 1), padding=(0, 0)):
    """``Conv2dBackward`` on CPU tensors (src/autograd/backward_ops.rs:753-770): (grad_input, grad_weight)."""
    x, w, go = _f32(x), _f32(w), _f32(go)
    n, ci, h, wd = x.shape
    co, _, kh, kw = w.shape
    (sh, sw), (ph, pw) = stride, padding
    gi, gw = np.empty_like(x), np.empty_like(w)
    lib = _load()
    lib.oracle_conv2d_backward.argtypes = [_fp] * 5 + [_sz] * 11
    lib.oracle_conv2d_backward.restype = None
    lib.oracle_conv2d_backward(_p(x), _p(w), _p(go), _p(gi), _p(gw), n, ci, co, h, wd, kh, kw, sh, sw, ph, pw)
    return gi, gw


def rnn_gates(x_t: np.ndarray, h: np.ndarray, w_ih: np.ndarray, w_hh: np.ndarray, b_ih, b_hh) -> np.ndarray:
    """Gate pre-activations of one recurrent step as LSTM::forward forms them on CPU tensors
    (src/nn/rnn.rs:72-77): x_t.matmul(W_ih^T), h.matmul(W_hh^T), then three f32 adds in the order
    gates_i + gates_h + bias_ih + bias_hh."""
    gi = matmul(_f32(x_t), transpose(_f32(w_ih)))
    gh = matmul(_f32(h), transpose(_f32(w_hh)))
    g = gi + gh
    if b_ih is not None:
        g = g + _f32(b_ih)[None, :]
    if b_hh is not None:
        g = g + _f32(b_hh)[None, :]
    return g.astype(np.float32)


def gru_gates(x_t: np.ndarray, h: np.ndarray, w_ih: np.ndarray, w_hh: np.ndarray, b_ih, b_hh):
    """The two biased products of one GRU step as GRU::forward_seq forms them on CPU tensors
    (src/nn/rnn.rs:164-170): gi = x_t.matmul(W_ih^T) + b_ih and gh = h.matmul(W_hh^T) + b_hh, each
    [batch, 3H] with gate order r, z, n."""
    gi = matmul(_f32(x_t), transpose(_f32(w_ih)))
    gh = matmul(_f32(h), transpose(_f32(w_hh)))
    if b_ih is not None:
        gi = gi + _f32(b_ih)[None, :]
    if b_hh is not None:
        gh = gh + _f32(b_hh)[None, :]
    return gi.astype(np.float32), gh.astype(np.float32)


def gru_step(gi: np.ndarray, gh: np.ndarray, h: np.ndarray) -> np.ndarray:
    """h' of one GRU step from the two products (src/nn/rnn.rs:172-180): r = sigmoid(gi_r + gh_r),
    z = sigmoid(gi_z + gh_z), n = tanh(gi_n + r * gh_n), h' = (1 - z) * n + z * h, all in f32."""
    gi, gh, h = _f32(gi), _f32(gh), _f32(h)
    hs = h.shape[1]
    one = np.float32(1.0)
    sig = lambda v: (one / (one + np.exp(-v, dtype=np.float32))).astype(np.float32)
    r = sig(gi[:, :hs] + gh[:, :hs])
    z = sig(gi[:, hs:2 * hs] + gh[:, hs:2 * hs])
    n = np.tanh(gi[:, 2 * hs:] + r * gh[:, 2 * hs:], dtype=np.float32)
    return ((one - z) * n + z * h).astype(np.float32)


def causal_softmax(scores: np.ndarray, scale: float) -> np.ndarray:
    """softmax(scores*scale + causal mask) over the last dim of [batch,t,t]."""
    s = _f32(scores).copy()
    batch, t, t2 = s.shape
    assert t == t2
    _load().oracle_causal_softmax(_p(s), batch, t, ctypes.c_float(scale))
    return s


def attention(q: np.ndarray, k: np.ndarray, v: np.ndarray, scale: float, causal: bool, mask=None,
              return_weights: bool = False):
    """The attention core of MultiHeadAttention::forward_attn on CPU tensors
    (src/nn/transformer.rs:87-115): matmul(q, k^T) * scale (+ mask) -> softmax -> matmul(., v).
    q [heads, t_q, d], k and v [heads, t_k, d]; ``mask`` an additive [t_q, t_k] array shared by
    all heads, or None.  With ``return_weights`` also returns the probabilities."""
    q, k, v = _f32(q), _f32(k), _f32(v)
    s = matmul(q, transpose(k))                 # forward uses the NN entry on a materialised K^T
    heads, tq, tk = s.shape
    lib = _load()
    lib.oracle_masked_softmax_add.argtypes = [_fp, _sz, _sz, _sz, ctypes.c_float, ctypes.c_int, _fp]
    lib.oracle_masked_softmax_add.restype = None
    m32 = _f32(mask) if mask is not None else None
    mp = _p(m32) if m32 is not None else ctypes.cast(None, _fp)
    lib.oracle_masked_softmax_add(_p(s), heads, tq, tk, ctypes.c_float(scale), 1 if causal else 0, mp)
    o = matmul(s, v)
    return (o, s) if return_weights else o


def ref_gpu_library_path():
    """Path of the reference's own GPU library (cuBLAS TF32) if it has been built."""
    return _b.REF_SO if os.path.exists(_b.REF_SO) else None
