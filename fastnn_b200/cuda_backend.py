"""Host wrappers over the C ABI, named after FastNN's ``src/tensor/cuda_backend.rs``.

Each ``cuda_matmul*`` wrapper does what its Rust namesake does (cuda_backend.rs:121-147,
175-204): allocate the output buffer, call the FFI entry with ``lda=k, ldb=n, ldc=n,
alpha=1, beta=0``, and turn a non-zero status into an error.  ``matmul`` / ``matmul_nt`` /
``matmul_tn`` add the 2-D-versus-batched dispatch and shape checks of ``Tensor::matmul*``
(src/tensor/ops.rs:341-518).  Tensors are torch CUDA float32, used for device memory only.
"""
from __future__ import annotations

import ctypes

import torch

from ._lib import lib

NN, NT, TN = 0, 1, 2
ACT_NONE, ACT_RELU, ACT_GELU = 0, 1, 2


class CudaError(RuntimeError):
    """A C-ABI entry returned non-zero (FastNN maps this to Err(String))."""


_initialised = set()


def cuda_init(device: int = 0) -> None:
    """CudaContext::new (src/cuda/context.rs:19-29): once per device."""
    if device in _initialised:
        return
    if lib().fastnn_cuda_init(int(device)) != 0:
        raise CudaError(f"Failed to initialize CUDA device {device}")
    _initialised.add(device)


def synchronize() -> None:
    if lib().fastnn_cuda_synchronize() != 0:
        raise CudaError("CUDA synchronize failed")


def _check(t: torch.Tensor, name: str) -> None:
    if not (t.is_cuda and t.dtype == torch.float32 and t.is_contiguous()):
        raise ValueError(f"{name}: expected a contiguous float32 CUDA tensor")


def _ptr(t):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else ctypes.c_void_p(0)


def _ensure_ctx(t: torch.Tensor) -> None:
    dev = t.device.index if t.device.index is not None else torch.cuda.current_device()
    if torch.cuda.current_device() != dev:
        raise ValueError("tensor is not on the current CUDA device")
    cuda_init(dev)


def _out(shape, like, out):
    if out is None:
        return torch.empty(shape, dtype=torch.float32, device=like.device)
    _check(out, "out")
    if tuple(out.shape) != tuple(shape):
        raise ValueError("out has the wrong shape")
    return out


# ---- FFI-level wrappers (names of cuda_backend.rs) -----------------------------------

def cuda_matmul(a, b, m, n, k, out=None, alpha=1.0, beta=0.0):
    _ensure_ctx(a)
    c = _out((m, n), a, out)
    if lib().fastnn_cuda_matmul(_ptr(a), _ptr(b), _ptr(c), m, n, k, k, n, n, alpha, beta) != 0:
        raise CudaError("CUDA matmul failed")
    return c


def cuda_matmul_batched(a, b, m, n, k, batch, out=None, alpha=1.0, beta=0.0):
    _ensure_ctx(a)
    c = _out((batch, m, n), a, out)
    if lib().fastnn_cuda_matmul_batched(_ptr(a), _ptr(b), _ptr(c), m, n, k, batch, alpha, beta) != 0:
        raise CudaError("CUDA batched matmul failed")
    return c


def cuda_matmul_nt(a, b, m, n, k, out=None):
    _ensure_ctx(a)
    c = _out((m, n), a, out)
    if lib().fastnn_cuda_matmul_nt(_ptr(a), _ptr(b), _ptr(c), m, n, k) != 0:
        raise CudaError("CUDA matmul_nt failed")
    return c


def cuda_matmul_tn(a, b, m, n, k, out=None):
    _ensure_ctx(a)
    c = _out((m, n), a, out)
    if lib().fastnn_cuda_matmul_tn(_ptr(a), _ptr(b), _ptr(c), m, n, k) != 0:
        raise CudaError("CUDA matmul_tn failed")
    return c


def cuda_matmul_batched_nt(a, b, m, n, k, batch, out=None):
    _ensure_ctx(a)
    c = _out((batch, m, n), a, out)
    if lib().fastnn_cuda_matmul_batched_nt(_ptr(a), _ptr(b), _ptr(c), m, n, k, batch) != 0:
        raise CudaError("CUDA matmul_batched_nt failed")
    return c


def cuda_matmul_batched_tn(a, b, m, n, k, batch, out=None):
    _ensure_ctx(a)
    c = _out((batch, m, n), a, out)
    if lib().fastnn_cuda_matmul_batched_tn(_ptr(a), _ptr(b), _ptr(c), m, n, k, batch) != 0:
        raise CudaError("CUDA matmul_batched_tn failed")
    return c


# ---- Tensor-level dispatch (src/tensor/ops.rs) ------------------------------------------

def _batch_of(t):
    n = 1
    for s in t.shape[:-2]:
        n *= int(s)
    return n


def matmul(a: torch.Tensor, b: torch.Tensor, out=None) -> torch.Tensor:
    """Tensor::matmul (ops.rs:341-438) for CUDA tensors: 2-D, or batched over leading dims.

    The batched C ABI has no broadcast (dense strides m*k and k*n), so a batch-1 operand is
    rejected here rather than read out of bounds."""
    _check(a, "a"); _check(b, "b")
    if a.dim() < 2 or b.dim() < 2:
        raise ValueError("matmul requires at least 2D tensors")
    m, k = int(a.shape[-2]), int(a.shape[-1])
    k2, n = int(b.shape[-2]), int(b.shape[-1])
    if k != k2:
        raise ValueError(f"Matmul shape mismatch: {tuple(a.shape)} x {tuple(b.shape)}")
    if a.dim() == 2 and b.dim() == 2:
        return cuda_matmul(a, b, m, n, k, out)
    ab, bb = _batch_of(a), _batch_of(b)
    if ab != bb:
        raise ValueError("Batch dimensions must match on CUDA tensors")
    c = cuda_matmul_batched(a, b, m, n, k, ab,
                            None if out is None else out.view(ab, m, n))
    return c.view(*a.shape[:-2], m, n) if out is None else out


def matmul_nt(a: torch.Tensor, b: torch.Tensor, out=None) -> torch.Tensor:
    """Tensor::matmul_nt (ops.rs:441-478): a[..,m,k] . b[..,n,k]^T."""
    _check(a, "a"); _check(b, "b")
    m, k = int(a.shape[-2]), int(a.shape[-1])
    n, k2 = int(b.shape[-2]), int(b.shape[-1])
    if k != k2:
        raise ValueError("matmul_nt shape mismatch")
    if a.dim() == 2 and b.dim() == 2:
        return cuda_matmul_nt(a, b, m, n, k, out)
    batch = _batch_of(a)
    if batch != _batch_of(b):
        raise ValueError("Batch dimensions must match")
    c = cuda_matmul_batched_nt(a, b, m, n, k, batch,
                               None if out is None else out.view(batch, m, n))
    return c.view(*a.shape[:-2], m, n) if out is None else out


def matmul_tn(a: torch.Tensor, b: torch.Tensor, out=None) -> torch.Tensor:
    """Tensor::matmul_tn (ops.rs:481-518): a[..,k,m]^T . b[..,k,n]."""
    _check(a, "a"); _check(b, "b")
    k, m = int(a.shape[-2]), int(a.shape[-1])
    k2, n = int(b.shape[-2]), int(b.shape[-1])
    if k != k2:
        raise ValueError("matmul_tn shape mismatch")
    if a.dim() == 2 and b.dim() == 2:
        return cuda_matmul_tn(a, b, m, n, k, out)
    batch = _batch_of(a)
    if batch != _batch_of(b):
        raise ValueError("Batch dimensions must match")
    c = cuda_matmul_batched_tn(a, b, m, n, k, batch,
                               None if out is None else out.view(batch, m, n))
    return c.view(*a.shape[:-2], m, n) if out is None else out


# ---- additions ------------------------------------------------------------------------------

def linear_forward(x, w, bias=None, act=ACT_NONE, layout=NT, out=None):
    """Linear::forward (src/nn/linear.rs:55-88) + optional ReLU/GELU in one launch.
    layout NT: w is [out,in] as FastNN stores it; NN: w is [in,out]."""
    _check(x, "x"); _check(w, "w")
    _ensure_ctx(x)
    x2 = x.reshape(-1, x.shape[-1])
    rows, in_f = int(x2.shape[0]), int(x2.shape[1])
    out_f = int(w.shape[0] if layout == NT else w.shape[1])
    if int(w.shape[1] if layout == NT else w.shape[0]) != in_f:
        raise ValueError(f"Expected input features {in_f}")
    if bias is not None:
        _check(bias, "bias")
    y = _out((rows, out_f), x, out)
    if lib().fastnn_b200_linear_forward(layout, _ptr(x2), _ptr(w), _ptr(bias), _ptr(y), rows, in_f,
                                        out_f, act) != 0:
        raise CudaError("CUDA linear_forward failed")
    return y.view(*x.shape[:-1], out_f)


def linear_backward_input(dy, w, pre=None, act=ACT_NONE, layout=NN, bias_grad=False, out=None,
                          stream=0):
    """dx = (dy . W) * act'(pre) and, when ``bias_grad`` is true, its sum over rows (the bias
    gradient of the layer that produced ``pre``), in one GEMM launch: what FastNN's tape does
    with matmul_nt + ReluBackward/GeluBackward (src/autograd/backward_ops.rs:136-160, 194-218)
    + the row sum behind Linear's bias expand (src/nn/linear.rs:78-82).
    layout NN: w is [out,in] as Linear stores it; NT: w is the transposed copy [in,out].
    Returns dx, or (dx, bias_grad)."""
    _check(dy, "dy"); _check(w, "w")
    _ensure_ctx(dy)
    dy2 = dy.reshape(-1, dy.shape[-1])
    rows, out_f = int(dy2.shape[0]), int(dy2.shape[1])
    in_f = int(w.shape[1] if layout == NN else w.shape[0])
    if int(w.shape[0] if layout == NN else w.shape[1]) != out_f:
        raise ValueError(f"Expected weight with {out_f} output features")
    if act != ACT_NONE:
        if pre is None:
            raise ValueError("an activation derivative needs the saved pre-activation")
        _check(pre, "pre")
        if pre.numel() != rows * in_f:
            raise ValueError("pre must be [rows, in_features]")
    dx = _out((rows, in_f), dy, out)
    db = torch.empty(in_f, dtype=torch.float32, device=dy.device) if bias_grad else None
    if lib().fastnn_b200_linear_backward_input(layout, _ptr(dy2), _ptr(w), _ptr(dx), rows, out_f, in_f,
                                               act, _ptr(pre if act != ACT_NONE else None), _ptr(db),
                                               stream) != 0:
        raise CudaError("CUDA linear_backward_input failed")
    dx = dx.view(*dy.shape[:-1], in_f)
    return (dx, db) if bias_grad else dx


def conv2d_forward(x, weight, bias=None, stride=(1, 1), padding=(0, 0), act=ACT_NONE, out=None, stream=0):
    """Conv2d::forward (src/nn/conv.rs:80-125) on NCHW tensors as one implicit-GEMM launch:
    x [N,Cin,H,W], weight [Cout,Cin,KH,KW], bias [Cout] or None; zero padding; act 0 none, 1 ReLU."""
    _check(x, "x"); _check(weight, "weight")
    _ensure_ctx(x)
    if x.dim() != 4 or weight.dim() != 4 or int(weight.shape[1]) != int(x.shape[1]):
        raise ValueError("Conv2d expects 4D input [N, C, H, W] and weight [Cout, C, KH, KW]")
    n, ci, h, w = (int(v) for v in x.shape)
    co, _, kh, kw = (int(v) for v in weight.shape)
    (sh, sw), (ph, pw) = stride, padding
    if h + 2 * ph < kh or w + 2 * pw < kw:
        raise ValueError("kernel larger than the padded input")
    oh, ow = (h + 2 * ph - kh) // sh + 1, (w + 2 * pw - kw) // sw + 1
    if bias is not None:
        _check(bias, "bias")
    y = _out((n, co, oh, ow), x, out)
    if lib().fastnn_b200_conv2d_forward(_ptr(x), _ptr(weight), _ptr(bias), _ptr(y), n, ci, co, h, w, kh, kw,
                                        sh, sw, ph, pw, act, stream) != 0:
        raise CudaError("CUDA conv2d_forward failed")
    return y


def conv2d_backward(x, weight, grad_output, stride=(1, 1), padding=(0, 0), stream=0):
    """Conv2dBackward (src/autograd/backward_ops.rs:753-770): returns (grad_input, grad_weight) for
    x [N,Cin,H,W], weight [Cout,Cin,KH,KW], grad_output [N,Cout,OH,OW]; any stride and padding."""
    _check(x, "x"); _check(weight, "weight"); _check(grad_output, "grad_output")
    _ensure_ctx(x)
    n, ci, h, w = (int(v) for v in x.shape)
    co, _, kh, kw = (int(v) for v in weight.shape)
    (sh, sw), (ph, pw) = stride, padding
    oh, ow = (h + 2 * ph - kh) // sh + 1, (w + 2 * pw - kw) // sw + 1
    if tuple(grad_output.shape) != (n, co, oh, ow):
        raise ValueError("grad_output must be [N, Cout, OH, OW]")
    gi = torch.empty_like(x)
    gw = torch.empty_like(weight)
    args = (n, ci, co, h, w, oh, ow, kh, kw, sh, sw, ph, pw, stream)
    if lib().fastnn_b200_conv2d_backward_data(_ptr(grad_output), _ptr(weight), _ptr(gi), *args) != 0:
        raise CudaError("CUDA conv2d_backward_data failed")
    if lib().fastnn_b200_conv2d_backward_weight(_ptr(x), _ptr(grad_output), _ptr(gw), *args) != 0:
        raise CudaError("CUDA conv2d_backward_weight failed")
    return gi, gw


def rnn_gates_forward(x_t, h, w_ih, w_hh, b_ih=None, b_hh=None, out=None, stream=0):
    """gates = x_t . W_ih^T + h . W_hh^T + b_ih + b_hh in one launch: the gate pre-activations of
    LSTM::forward (src/nn/rnn.rs:72-77) and of the plain RNN cell.  x_t [batch,input] may be a
    strided view x[:, t, :] of x[batch,seq,input]; h [batch,hidden]; W_ih [G,input]; W_hh [G,hidden]."""
    for name, t in (("h", h), ("w_ih", w_ih), ("w_hh", w_hh)):
        _check(t, name)
    if x_t.dtype != torch.float32 or not x_t.is_cuda or x_t.dim() != 2 or x_t.stride(1) != 1:
        raise ValueError("x_t must be a float32 CUDA matrix with contiguous rows")
    _ensure_ctx(h)
    batch, in_f = int(x_t.shape[0]), int(x_t.shape[1])
    hid = int(h.shape[1])
    g_rows = int(w_ih.shape[0])
    if tuple(w_ih.shape) != (g_rows, in_f) or tuple(w_hh.shape) != (g_rows, hid) or int(h.shape[0]) != batch:
        raise ValueError("rnn_gates_forward shape mismatch")
    for b in (b_ih, b_hh):
        if b is not None:
            _check(b, "bias")
    gates = _out((batch, g_rows), h, out)
    ld_x = int(x_t.stride(0)) if batch > 1 else max(in_f, 1)
    if lib().fastnn_b200_rnn_gates_forward(_ptr(x_t), ld_x, _ptr(h), _ptr(w_ih), _ptr(w_hh), _ptr(b_ih),
                                           _ptr(b_hh), _ptr(gates), batch, in_f, hid, g_rows, stream) != 0:
        raise CudaError("CUDA rnn_gates_forward failed")
    return gates


def gru_pack_weights(w_ih, w_hh, b_ih=None, b_hh=None):
    """One-time repacking of GRU parameters (W_ih [3H,input], W_hh [3H,hidden], biases [3H]; gate
    order r, z, n as in src/nn/rnn.rs:135-146) so that ONE rnn_gates_forward launch per time step
    yields everything GRU::forward_seq (src/nn/rnn.rs:164-180) needs:
        gates[:, 0:2H]  = gi + gh of the r and z gates (biases included)
        gates[:, 2H:3H] = gi_n = x_t . W_ih[2H:3H]^T + b_ih[2H:3H]
        gates[:, 3H:4H] = gh_n = h . W_hh[2H:3H]^T + b_hh[2H:3H]   (multiplied by r before the tanh)
    The n gate's two products must stay apart, so its rows of each matrix face a zero block of the
    other: W_ih' = [W_ih[0:3H]; 0], W_hh' = [W_hh[0:2H]; 0; W_hh[2H:3H]] (4H rows each)."""
    _check(w_ih, "w_ih"); _check(w_hh, "w_hh")
    h3 = int(w_ih.shape[0])
    if h3 % 3 != 0 or int(w_hh.shape[0]) != h3:
        raise ValueError("GRU weights have 3 * hidden rows")
    hs = h3 // 3
    wi = torch.zeros(4 * hs, w_ih.shape[1], dtype=torch.float32, device=w_ih.device)
    wh = torch.zeros(4 * hs, w_hh.shape[1], dtype=torch.float32, device=w_hh.device)
    wi[:3 * hs] = w_ih
    wh[:2 * hs] = w_hh[:2 * hs]
    wh[3 * hs:] = w_hh[2 * hs:]
    bi = bh = None
    if b_ih is not None:
        bi = torch.zeros(4 * hs, dtype=torch.float32, device=w_ih.device)
        bi[:3 * hs] = b_ih
    if b_hh is not None:
        bh = torch.zeros(4 * hs, dtype=torch.float32, device=w_hh.device)
        bh[:2 * hs] = b_hh[:2 * hs]
        bh[3 * hs:] = b_hh[2 * hs:]
    return wi, wh, bi, bh


def gemm_ex(layout, a_ptr, b_ptr, c_ptr, m, n, k, batch, lda, ldb, ldc, sa, sb, sc,
            alpha=1.0, beta=0.0, bias_ptr=0, act=ACT_NONE, stream=0) -> None:
    """Raw general entry (pointers as integers, strides in elements)."""
    rc = lib().fastnn_b200_gemm_ex(layout, ctypes.c_void_p(a_ptr), ctypes.c_void_p(b_ptr),
                                   ctypes.c_void_p(c_ptr), m, n, k, batch, lda, ldb, ldc, sa, sb, sc,
                                   alpha, beta, ctypes.c_void_p(bias_ptr), act,
                                   ctypes.c_void_p(stream))
    if rc != 0:
        raise CudaError("fastnn_b200_gemm_ex failed")


def _same_device(*tensors) -> None:
    """All tensors on the current CUDA device; does not initialise the library's context."""
    cur = torch.cuda.current_device()
    for t in tensors:
        if t is not None and t.device.index != cur:
            raise ValueError("tensor is not on the current CUDA device")


def gemm_splitk_static(layout, a, b, m, n, k, split_k, out=None, stream=0):
    """C = op(A).op(B) through the entry point that allocates nothing: split-K partial sums go
    to the 16 MiB array built into the library.  Returns the output tensor; raises CudaError
    with ``too_large=True`` in its args when m*n*split_k floats exceed that array.  Needs no
    ``cuda_init`` (and does not call it); pass ``out`` to keep torch's allocator out of it too."""
    _check(a, "a"); _check(b, "b")
    if layout not in (NN, NT, TN):
        raise ValueError("bad layout")
    want_a = (k, m) if layout == TN else (m, k)
    want_b = (n, k) if layout == NT else (k, n)
    if tuple(a.shape) != want_a or tuple(b.shape) != want_b:
        raise ValueError(f"operand shapes {tuple(a.shape)}, {tuple(b.shape)} do not match "
                         f"layout {layout} with m={m}, n={n}, k={k}")
    c = _out((m, n), a, out)
    _same_device(a, b, c)
    rc = lib().fastnn_b200_gemm_splitk_static(layout, _ptr(a), _ptr(b), _ptr(c), m, n, k, split_k,
                                              ctypes.c_void_p(stream))
    if rc != 0:
        raise CudaError("fastnn_b200_gemm_splitk_static failed", rc == -2)
    return c


def gemm_gather_ex(layout, a_ptr, b_ptr, c_ptr, m, n, k, batch, lda, ldb, ldc, sa, sb, sc, peer_ptrs,
                   alpha=1.0, bias_ptr=0, act=ACT_NONE, stream=0) -> None:
    """fastnn_b200_gemm_ex with the all-gather of C fused into the epilogue: every finished tile is
    also stored to ``peer_ptrs`` (the same rows of C in the other GPUs' buffers, peer-mapped)."""
    arr = (ctypes.c_void_p * max(1, len(peer_ptrs)))(*[ctypes.c_void_p(int(p)) for p in peer_ptrs])
    rc = lib().fastnn_b200_gemm_gather_ex(layout, ctypes.c_void_p(a_ptr), ctypes.c_void_p(b_ptr),
                                          ctypes.c_void_p(c_ptr), m, n, k, batch, lda, ldb, ldc, sa, sb, sc,
                                          alpha, ctypes.c_void_p(bias_ptr), act, arr, len(peer_ptrs),
                                          ctypes.c_void_p(stream))
    if rc != 0:
        raise CudaError("fastnn_b200_gemm_gather_ex failed")


def gemm_gather_mc_ex(layout, a_ptr, b_ptr, c_ptr, m, n, k, batch, lda, ldb, ldc, sa, sb, sc, mc_ptr,
                      alpha=1.0, bias_ptr=0, act=ACT_NONE, stream=0) -> None:
    """The gather through the switch: every finished tile goes once, with multimem.st, to the NVLink
    multicast address ``mc_ptr`` of these rows of C and arrives in every GPU's buffer."""
    rc = lib().fastnn_b200_gemm_gather_mc_ex(layout, ctypes.c_void_p(a_ptr), ctypes.c_void_p(b_ptr),
                                             ctypes.c_void_p(c_ptr), m, n, k, batch, lda, ldb, ldc, sa, sb, sc,
                                             alpha, ctypes.c_void_p(bias_ptr), act, ctypes.c_void_p(mc_ptr),
                                             ctypes.c_void_p(stream))
    if rc != 0:
        raise CudaError("fastnn_b200_gemm_gather_mc_ex failed")


def selftest_bounded_wait(budget_us: int = 1000) -> int:
    """Runs the one-warp kernel whose bounded wait must run out; returns how long it waited (us).
    Afterwards ``device_status()`` returns 0x1F0 once and then 0 again."""
    waited = ctypes.c_uint()
    if lib().fastnn_b200_selftest_bounded_wait(int(budget_us), ctypes.byref(waited)) != 0:
        raise CudaError("bounded-wait self-test failed: the wait did not give up")
    return waited.value


def current_stream_ptr() -> int:
    """torch's current stream as an integer for the ``stream`` arguments of this module.  The
    entries without a stream argument use the legacy default stream, as FastNN's do."""
    return int(torch.cuda.current_stream().cuda_stream)


def attention_forward(q, k, v, scale=None, causal=False, out=None, stream=0, mask=None,
                      return_weights=False):
    """softmax(scale * q.k^T + mask) . v for q [.., t_q, d], k, v [.., t_k, d]: the core of
    MultiHeadAttention::forward_attn (src/nn/transformer.rs:87-115).  ``causal`` hides key j from
    query i when j > i; ``mask`` is an additive [t_q, t_k] tensor shared by all heads.  One fused
    launch when the shape allows it and the probabilities are not wanted, FastNN's composition on
    this library's GEMMs otherwise.  With ``return_weights`` returns (o, probabilities)."""
    _check(q, "q"); _check(k, "k"); _check(v, "v")
    _ensure_ctx(q)
    tq, d = int(q.shape[-2]), int(q.shape[-1])
    tk = int(k.shape[-2])
    heads = _batch_of(q)
    if tuple(k.shape) != tuple(v.shape) or int(k.shape[-1]) != d or _batch_of(k) != heads:
        raise ValueError("attention shape mismatch")
    if mask is not None:
        _check(mask, "mask")
        if tuple(mask.shape) != (tq, tk):
            raise ValueError("mask must be [t_q, t_k]")
    if scale is None:
        scale = 1.0 / (d ** 0.5)
    o = _out(tuple(q.shape), q, out)
    w = torch.empty(tuple(q.shape[:-1]) + (tk,), dtype=torch.float32, device=q.device) if return_weights else None
    rc = lib().fastnn_b200_attention_forward_ex(_ptr(q), _ptr(k), _ptr(v), _ptr(o), _ptr(w), _ptr(mask), heads,
                                                tq, tk, d, float(scale), 1 if causal else 0,
                                                ctypes.c_void_p(stream))
    if rc != 0:
        raise CudaError("CUDA attention_forward failed")
    return (o, w) if return_weights else o


def reduce_partials(partials_ptr, c_ptr, m, n, count, ldc=None, alpha=1.0, beta=0.0, bias_ptr=0,
                    act=ACT_NONE, stream=0) -> None:
    """c = act(alpha * sum_i partials[i] + beta * c + bias), partials = count dense [m,n] blocks."""
    rc = lib().fastnn_b200_reduce_partials(ctypes.c_void_p(partials_ptr), ctypes.c_void_p(c_ptr), m, n,
                                           count, n if ldc is None else ldc, alpha, beta,
                                           ctypes.c_void_p(bias_ptr), act, ctypes.c_void_p(stream))
    if rc != 0:
        raise CudaError("fastnn_b200_reduce_partials failed")


def set_policy(policy: int = 0, block_n: int = 0, split_k: int = 0) -> None:
    if lib().fastnn_b200_set_policy(policy, block_n, split_k) != 0:
        raise ValueError("bad policy")


def last_path():
    bn, sk, nc = ctypes.c_int(), ctypes.c_int(), ctypes.c_int()
    path = lib().fastnn_b200_last_path(ctypes.byref(bn), ctypes.byref(sk), ctypes.byref(nc))
    return {"path": path, "block_n": bn.value, "split_k": sk.value, "num_ctas": nc.value}


def plan_query(layout, m, n, k, batch=1):
    """The planner's choice for a GEMM, without a launch (answers without a GPU too)."""
    out = [ctypes.c_int() for _ in range(4)]
    if lib().fastnn_b200_plan_query(layout, m, n, k, batch, *[ctypes.byref(o) for o in out]) != 0:
        raise ValueError("bad GEMM shape")
    return {"block_n": out[0].value, "split_k": out[1].value, "cta_pair": bool(out[2].value),
            "cluster_k": bool(out[3].value)}


def device_status() -> int:
    v = ctypes.c_uint()
    if lib().fastnn_b200_device_status(ctypes.byref(v)) != 0:
        raise CudaError("device_status failed")
    return v.value


def launch_count() -> int:
    return int(lib().fastnn_b200_launch_count())
