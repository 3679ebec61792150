/*
 * C ABI of libfastnn_b200.so: the matrix-multiply path of FastNN's CUDA backend,
 * implemented with hand-written sm_100a kernels (tcgen05 kind::tf32, TMA, TMEM).
 *
 * Section 1 re-declares, with identical names, argument order and meaning, the entry
 * points FastNN's Rust side binds for this path (FastNN: cuda/include/kernels.h;
 * callers in src/tensor/cuda_backend.rs, src/cuda/memory.rs, src/cuda/context.rs), so
 * the library can be linked in place of FastNN's own kernels for these symbols.
 * Section 2 adds entry points FastNN does not have (fused Linear epilogue, explicit
 * leading dimensions and stream, diagnostics); their names carry the fastnn_b200_ prefix.
 *
 * Conventions (same as FastNN): all matrices are dense row-major float32 in device
 * memory; every function returns 0 on success and -1 on failure; work is enqueued on
 * the legacy default stream unless a stream is passed explicitly; the caller owns all
 * buffers and the callee writes every element of the output (an output buffer may be
 * recycled and dirty).  There is no CPU fallback: without a CUDA device every compute
 * entry returns -1.
 */
#ifndef FASTNN_B200_KERNELS_H
#define FASTNN_B200_KERNELS_H

#include <stddef.h>
#include <stdint.h>

/* Every entry point below has default ELF visibility; nothing else is exported. */
#if defined(__GNUC__)
#define FASTNN_B200_API __attribute__((visibility("default")))
#else
#define FASTNN_B200_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

/* ------------------------------------------------------------------------ */
/* 1. FastNN drop-in symbols                                                */
/* ------------------------------------------------------------------------ */

/* Device management -- FastNN cuda/include/kernels.h:13-16, cuda/kernels.cu:35-64.
 * fastnn_cuda_init must be called (per process, per device used) before any GEMM. */
FASTNN_B200_API int fastnn_cuda_init(int device_id);
FASTNN_B200_API int fastnn_cuda_device_count(void);
FASTNN_B200_API int fastnn_cuda_synchronize(void);
FASTNN_B200_API void fastnn_cuda_get_memory_info(size_t* free_mem, size_t* total_mem);

/* Memory -- FastNN cuda/include/kernels.h:21-26, cuda/kernels.cu:69-97.  Sizes in BYTES;
 * copies are synchronous. */
FASTNN_B200_API int fastnn_cuda_malloc(float** ptr, size_t size);
FASTNN_B200_API int fastnn_cuda_free(float* ptr);
FASTNN_B200_API int fastnn_cuda_memcpy_h2d(float* dst, const float* src, size_t size);
FASTNN_B200_API int fastnn_cuda_memcpy_d2h(float* dst, const float* src, size_t size);
FASTNN_B200_API int fastnn_cuda_memcpy_d2d(float* dst, const float* src, size_t size);
FASTNN_B200_API int fastnn_cuda_memset(float* ptr, int value, size_t size);

/* C[m,n] = alpha * A[m,k] . B[k,n] + beta * C, leading dimensions in elements.
 * FastNN cuda/include/kernels.h:71-74, cuda/kernels.cu:431-445. */
FASTNN_B200_API int fastnn_cuda_matmul(const float* a, const float* b, float* c,
                       int m, int n, int k,
                       int lda, int ldb, int ldc,
                       float alpha, float beta);
/* Per batch C[m,n] = alpha * A[m,k] . B[k,n] + beta * C, dense strides m*k, k*n, m*n.
 * FastNN cuda/include/kernels.h:75-77, cuda/kernels.cu:509-526. */
FASTNN_B200_API int fastnn_cuda_matmul_batched(const float* a, const float* b, float* c,
                               int m, int n, int k, int batch_size,
                               float alpha, float beta);
/* C[m,n] = A[m,k] . B^T, B stored [n,k].  FastNN kernels.h:78, kernels.cu:452-461. */
FASTNN_B200_API int fastnn_cuda_matmul_nt(const float* a, const float* b, float* c, int m, int n, int k);
/* C[m,n] = A^T . B[k,n], A stored [k,m].  FastNN kernels.h:79, kernels.cu:464-473. */
FASTNN_B200_API int fastnn_cuda_matmul_tn(const float* a, const float* b, float* c, int m, int n, int k);
/* Batched forms, dense strides.  FastNN kernels.h:80-81, kernels.cu:476-507. */
FASTNN_B200_API int fastnn_cuda_matmul_batched_nt(const float* a, const float* b, float* c,
                                  int m, int n, int k, int batch_size);
FASTNN_B200_API int fastnn_cuda_matmul_batched_tn(const float* a, const float* b, float* c,
                                  int m, int n, int k, int batch_size);

/* ------------------------------------------------------------------------ */
/* 2. Additions (no FastNN symbol of these names)                            */
/* ------------------------------------------------------------------------ */

/* layout of the two operands */
#define FASTNN_B200_NN 0   /* A[m,k], B[k,n] */
#define FASTNN_B200_NT 1   /* A[m,k], B[n,k] */
#define FASTNN_B200_TN 2   /* A[k,m], B[k,n] */

/* epilogue activation */
#define FASTNN_B200_ACT_NONE 0
#define FASTNN_B200_ACT_RELU 1   /* max(x, 0)                   -- FastNN src/tensor/ops.rs:191-198 */
#define FASTNN_B200_ACT_GELU 2   /* 0.5 x (1 + erf(x / sqrt 2)) -- FastNN src/tensor/ops.rs:220-230 */

/* General form behind every GEMM entry:
 *   C[b] = act( alpha * op(A[b]) . op(B[b]) + beta * C[b] + bias )      b in [0, batch)
 * lda/ldb/ldc are row strides in elements, stride_a/b/c are batch strides in elements,
 * bias is [n] or NULL, stream is a cudaStream_t (NULL = legacy default stream).
 * Replaces, in one launch, the transpose + matmul + expand + add (+ gelu/relu) sequence of
 * FastNN's Linear::forward (src/nn/linear.rs:71-87). */
FASTNN_B200_API int fastnn_b200_gemm_ex(int layout, const float* a, const float* b, float* c,
                        int m, int n, int k, int batch,
                        long long lda, long long ldb, long long ldc,
                        long long stride_a, long long stride_b, long long stride_c,
                        float alpha, float beta,
                        const float* bias, int act, void* stream);

/* y[rows,out] = act( x[rows,in] . W + bias[out] ) with dense operands.
 * layout NT takes W as FastNN stores it, [out,in] (Linear's weight); layout NN takes W
 * already as [in,out].  Semantics of Linear::forward (+ Tensor::relu / Tensor::gelu). */
FASTNN_B200_API int fastnn_b200_linear_forward(int layout, const float* x, const float* w, const float* bias,
                               float* y, int rows, int in_features, int out_features, int act);

/* Backward of y = act(pre) . W2^T seen from the layer that produced `pre`, in one GEMM launch
 * (plus one small reduce when bias_grad is wanted):
 *   dx[rows,in] = ( dy[rows,out] . W ) * act'( pre[rows,in] )
 *   bias_grad[in] = sum over rows of dx          (optional; pass NULL to skip)
 * layout NN takes W as Linear stores it, [out,in]; layout NT takes the transposed copy [in,out]
 * that Linear::forward materialises (src/nn/linear.rs:74) and MatmulBackward hands to matmul_nt.
 * act: 0 none (pre may be NULL), 1 ReLU, 2 GELU(erf); the derivative is the one ReluBackward /
 * GeluBackward apply (src/autograd/backward_ops.rs:136-160, 194-218; cuda/kernels.cu:244-252).
 * Replaces matmul_nt + relu/gelu_backward + the sum over rows behind the bias expand
 * (src/nn/linear.rs:78-82; FastNN's sum_axis allocates per call, cuda/kernels.cu:701-714).
 * Rows are added in a fixed order, so bias_grad is deterministic. */
FASTNN_B200_API int fastnn_b200_linear_backward_input(int layout, const float* dy, const float* w,
                                                      float* dx, int rows, int out_features,
                                                      int in_features, int act, const float* pre,
                                                      float* bias_grad, void* stream);

/* Gate pre-activations of one recurrent step in one launch:
 *   gates[batch, gate_rows] = x_t[batch,input] . W_ih[gate_rows,input]^T
 *                           + h[batch,hidden]  . W_hh[gate_rows,hidden]^T + b_ih + b_hh
 * i.e. FastNN's  x_t.matmul(W_ih^T) + h.matmul(W_hh^T) + bias + bias2  of LSTM::forward
 * (src/nn/rnn.rs:72-77; gate_rows = 4 * hidden) and of the plain RNN cell (gate_rows = hidden):
 * two transposes, two GEMMs and three elementwise adds there.  Both products accumulate in the
 * same tensor-memory tile (the K loop runs over input, then hidden).  x_t may be a strided
 * view: row b of x_t starts at x_t + b * ld_x (ld_x = seq_len * input for x[batch,seq,input]).
 * Either bias may be NULL.  Operands TMA cannot address are served by two dependent launches. */
FASTNN_B200_API int fastnn_b200_rnn_gates_forward(const float* x_t, long long ld_x, const float* h,
                                                  const float* w_ih, const float* w_hh,
                                                  const float* b_ih, const float* b_hh, float* gates,
                                                  int batch, int input_size, int hidden_size,
                                                  int gate_rows, void* stream);

/* Conv2d forward, NCHW, as an implicit GEMM (no im2col matrix in memory):
 *   output[n, co, oh, ow] = bias[co] + sum over (ci, ki, kj) of
 *       weight[co, ci, ki, kj] * input[n, ci, oh*stride_h + ki - pad_h, ow*stride_w + kj - pad_w]
 * with out_h = (input_h + 2 pad_h - kernel_h) / stride_h + 1 (likewise out_w), zero padding, no
 * dilation or groups: Conv2d::forward (src/nn/conv.rs:80-125).  fastnn_cuda_conv2d_forward has
 * the signature of FastNN's own CUDA entry (cuda/kernels.cu:896-946: im2col + cuBLAS per image,
 * bias added one channel at a time through host copies) and replaces it; the _b200_ form adds a
 * fused activation (0 none, 1 ReLU) and a stream.  bias may be NULL.  All images go in one
 * launch (plus a small weight-padding launch when in_channels*kernel_h*kernel_w is not a
 * multiple of 4). */
FASTNN_B200_API int fastnn_cuda_conv2d_forward(const float* input, const float* weight, const float* bias,
                                               float* output, int batch_size, int in_channels,
                                               int out_channels, int input_h, int input_w,
                                               int kernel_h, int kernel_w, int stride_h, int stride_w,
                                               int pad_h, int pad_w);
FASTNN_B200_API int fastnn_b200_conv2d_forward(const float* input, const float* weight, const float* bias,
                                               float* output, int batch_size, int in_channels,
                                               int out_channels, int input_h, int input_w,
                                               int kernel_h, int kernel_w, int stride_h, int stride_w,
                                               int pad_h, int pad_w, int act, void* stream);

/* Gradients of that convolution, Conv2dBackward (src/autograd/backward_ops.rs:753-770):
 *   grad_input[n, ci, ih, iw]  += grad_output[n, co, oh, ow] * weight[co, ci, ki, kj]
 *   grad_weight[co, ci, ki, kj] += grad_output[n, co, oh, ow] * input[n, ci, ih, iw]
 * over all (n, co, oh, ow, ci, ki, kj) with ih = oh*stride_h + ki - pad_h inside the image
 * (likewise iw); both outputs are overwritten, not accumulated into.  The fastnn_cuda_ names keep
 * FastNN's argument lists (cuda/kernels.cu:949-987 and 989-1026: col2im / im2col + cuBLAS per
 * image); the _b200_ forms add a stream.
 * backward_data: for stride 1 with pad <= kernel - 1, the implicit-GEMM forward kernel run on
 * grad_output with the kernel reversed and channels swapped; for every other stride and padding a
 * gather-form kernel in which each grad_input element adds its (co, ki, kj) terms (the sums
 * FastNN's GEMM + col2im forms, cuda/kernels.cu:862-893) -- no column matrix, no atomics.
 * backward_weight, any stride: an implicit GEMM over all positions of all images -- grad_output
 * tiles by TMA, the input values under every kernel tap gathered straight into the tensor core's
 * operand stages, no column matrix -- cut into slices that are added in a fixed order
 * (deterministic).  Outputs whose out_h * out_w is not a multiple of 4 take the explicit form: one
 * im2col launch for all images (tap-major, as FastNN's kernel_im2col lays it out), one batched NT
 * GEMM into per-image partials, one fixed-order sum. */
FASTNN_B200_API int fastnn_cuda_conv2d_backward_data(const float* grad_output, const float* weight,
                                                     float* grad_input, int batch_size, int in_channels,
                                                     int out_channels, int input_h, int input_w,
                                                     int output_h, int output_w, int kernel_h,
                                                     int kernel_w, int stride_h, int stride_w,
                                                     int pad_h, int pad_w);
FASTNN_B200_API int fastnn_b200_conv2d_backward_data(const float* grad_output, const float* weight,
                                                     float* grad_input, int batch_size, int in_channels,
                                                     int out_channels, int input_h, int input_w,
                                                     int output_h, int output_w, int kernel_h,
                                                     int kernel_w, int stride_h, int stride_w,
                                                     int pad_h, int pad_w, void* stream);
FASTNN_B200_API int fastnn_cuda_conv2d_backward_weight(const float* input, const float* grad_output,
                                                       float* grad_weight, int batch_size,
                                                       int in_channels, int out_channels, int input_h,
                                                       int input_w, int output_h, int output_w,
                                                       int kernel_h, int kernel_w, int stride_h,
                                                       int stride_w, int pad_h, int pad_w);
FASTNN_B200_API int fastnn_b200_conv2d_backward_weight(const float* input, const float* grad_output,
                                                       float* grad_weight, int batch_size,
                                                       int in_channels, int out_channels, int input_h,
                                                       int input_w, int output_h, int output_w,
                                                       int kernel_h, int kernel_w, int stride_h,
                                                       int stride_w, int pad_h, int pad_w, void* stream);

/* Attention core, per head h in [0, batch_heads):
 *   O[h] = softmax( scale * Q[h] . K[h]^T + mask ) . V[h]
 * q [batch_heads, t_q, head_dim], k and v [batch_heads, t_k, head_dim], o like q, all dense.
 * With causal != 0, key j is hidden from query i when j > i (FastNN adds -1e9 there,
 * src/nn/transformer.rs:22-27); `mask` (the _ex form and FastNN's symbol; may be NULL) is an
 * additive [t_q, t_k] matrix shared by all heads, the form FastNN's cached mask has
 * (src/nn/transformer.rs:15-30, 99-105); softmax over keys as src/tensor/ops.rs:273-284.
 * attn_weights (may be NULL) receives the probabilities [batch_heads, t_q, t_k].
 *
 * Fused form -- one launch instead of FastNN's batched matmul + mul_scalar + add + softmax +
 * batched matmul (src/nn/transformer.rs:87-115), the scores never reach memory: taken when the
 * probabilities are not asked for and head_dim is in {32, 64, 96, 128}, t_k <= 256, scale > 0,
 * the operands are 16-byte aligned and the working set fits shared memory.
 * Every other call runs FastNN's own composition on this library's kernels: batched
 * scale * Q.K^T (NT GEMM), a masked row softmax in place, batched P.V (NN GEMM); the scores live
 * in attn_weights or in a per-stream scratch buffer.
 *
 * fastnn_cuda_scaled_dot_product_attention has the signature of FastNN's own entry
 * (cuda/include/kernels.h:209, cuda/kernels.cu:1707-1776: transpose + cuBLAS + softmax + cuBLAS
 * with a cudaMalloc per call) and replaces it.  There `causal` and `mask` are accepted and ignored
 * (the masking code is dead); here both are applied. */
FASTNN_B200_API int fastnn_b200_attention_forward(const float* q, const float* k, const float* v,
                                                  float* o, int batch_heads, int t_q, int t_k,
                                                  int head_dim, float scale, int causal,
                                                  void* stream);
FASTNN_B200_API int fastnn_b200_attention_forward_ex(const float* q, const float* k, const float* v,
                                                     float* o, float* attn_weights, const float* mask,
                                                     int batch_heads, int t_q, int t_k, int head_dim,
                                                     float scale, int causal, void* stream);
FASTNN_B200_API int fastnn_cuda_scaled_dot_product_attention(const float* query, const float* key,
                                                             const float* value, float* output,
                                                             float* attn_weights, const float* mask,
                                                             int batch_size, int num_heads,
                                                             int seq_len_q, int seq_len_k, int head_dim,
                                                             float scale, int causal);

/* The general GEMM with an all-gather of C fused into its epilogue, for the multi-GPU form of the
 * path in which the rows of C (or the batches) are split over GPUs and a caller wants all of C on
 * every device.  No counterpart in FastNN (it has no multi-GPU path); replaces "GEMM, then an
 * all-gather of the C shards" by one launch per rank:
 *   C[b] = act( alpha * op(A[b]) . op(B[b]) + bias )  as fastnn_b200_gemm_ex with beta = 0,
 * and every finished 32 x 32 tile is stored not only to c but also to peer_c[0..n_peers-1]: the
 * address of the SAME rows of C inside each other GPU's full-size buffer, as mapped into this
 * process (CUDA peer access / symmetric memory).  n_peers <= 7.  All destinations share ldc and
 * stride_c.  The stores are plain TMA stores over NVLink issued by the epilogue warps while the
 * tensor core works on the next tile; nothing is ever LOADED from a peer.  That form needs TMA-
 * addressable operands, c and every peer_c[i] 16-byte aligned and ldc a multiple of 4; any other
 * call is served by the ordinary GEMM into c followed by one strided device-to-device copy per
 * destination on the same stream (correct, not overlapped).
 * Completion: when the kernel has finished on this GPU its tiles are in every destination; the
 * ranks still need one barrier among themselves before any of them reads rows it did not
 * compute.  n_peers = 0 is fastnn_b200_gemm_ex. */
FASTNN_B200_API int fastnn_b200_gemm_gather_ex(int layout, const float* a, const float* b, float* c,
                                               int m, int n, int k, int batch,
                                               long long lda, long long ldb, long long ldc,
                                               long long stride_a, long long stride_b,
                                               long long stride_c, float alpha, const float* bias,
                                               int act, float* const* peer_c, int n_peers,
                                               void* stream);

/* The same gather through the NVSwitch: mc_c is the NVLink MULTICAST address of the rows this rank
 * computes (a multicast object bound to every rank's C buffer, e.g. the multicast pointer of torch's
 * symmetric memory, plus the shard's offset).  Every finished tile is written ONCE, 16 bytes per
 * multimem.st, and the switch delivers it to every GPU's C -- this GPU's own included, so c (which
 * must be this rank's local address of the same rows, and supplies alignment and shape) is not
 * written directly.  A rank then sends 1/N of C instead of (N-1)/N: the form for four GPUs and
 * more, where the unicast stores of fastnn_b200_gemm_gather_ex, not the tensor cores, set the time.
 * Needs TMA-addressable operands, 16-byte aligned c and mc_c, n and ldc multiples of 4 (-1
 * otherwise: use the unicast entry).  Completion as above: kernel end on every rank, then one
 * barrier among the ranks.  No counterpart in FastNN. */
FASTNN_B200_API int fastnn_b200_gemm_gather_mc_ex(int layout, const float* a, const float* b, float* c,
                                                  int m, int n, int k, int batch,
                                                  long long lda, long long ldb, long long ldc,
                                                  long long stride_a, long long stride_b,
                                                  long long stride_c, float alpha, const float* bias,
                                                  int act, float* mc_c, void* stream);

/* c[m,n] = act( alpha * (partials[0] + partials[1] + ... + partials[count-1]) + beta * c + bias ),
 * partials stored back to back as count dense [m,n] matrices, added in ascending order.
 * The reduce step of split-K, exposed for the multi-GPU weight-gradient path where the K
 * dimension is split over ranks and every rank stores its partial product for a block of rows
 * straight into the owning rank's memory (K-sharded form of FastNN's MatmulBackward
 * dB = A^T . dC, src/autograd/backward_ops.rs:93).  ldc in elements; stream as above. */
FASTNN_B200_API int fastnn_b200_reduce_partials(const float* partials, float* c, int m, int n,
                                                int count, long long ldc, float alpha, float beta,
                                                const float* bias, int act, void* stream);

/* Split-K GEMM that allocates nothing.  It has no counterpart in FastNN.
 *
 *   C[m,n] = op(A) . op(B)      dense operands, layout as above, alpha = 1, beta = 0
 *
 * Who it is for: callers that are not allowed to call cudaMalloc / cudaFree at the moment
 * they need a GEMM -- code running while another thread has a stream capture open (an
 * allocation would invalidate the capture or block), real-time loops that may not take the
 * allocator's device-wide synchronisation, and hosts whose memory budget is fixed up front and
 * audited, where a library that grows a hidden workspace is not acceptable.  The other entry
 * points keep their split-K partial sums in a workspace obtained from cudaMalloc on first
 * use; this one keeps them in a 16 MiB array that is part of the library image (every GPU
 * that loads the library holds those 16 MiB until the process exits).
 *
 * The K range is cut into split_k parts (clamped so each part has at least one 32-deep
 * block); each part's partial tile goes to the built-in array and a second kernel adds the
 * parts in ascending order into C.
 * Limits and rules:
 *   - m * n * split_k floats must fit the array (4 Mi floats); otherwise nothing is launched,
 *     a message goes to stderr and the call returns -2.
 *   - a, b, c 16-byte aligned; row lengths (k or m for A, k or n for B, n for C) multiples
 *     of 4 floats.  Other failures return -1.
 *   - It does not need fastnn_cuda_init.  The first call on each device looks up the device
 *     address of the array and of the tensor-map encoder; make that first call before any
 *     stream capture begins.
 *   - A bounded wait that runs out inside its kernels is reported through
 *     fastnn_b200_device_status, like every other kernel's.
 *   - All calls on one device share the array and it keeps the previous call's contents.
 *     Every element that is read was written earlier in the same call, so nothing has to be
 *     cleared, but two calls that overlap on the GPU (different streams without an ordering
 *     between them) race on it.  Calls on one stream are safe back to back.
 *   - No cudaMalloc, cudaFree or other allocating routine is called, on any call. */
FASTNN_B200_API int fastnn_b200_gemm_splitk_static(int layout, const float* a, const float* b,
                                                   float* c, int m, int n, int k, int split_k,
                                                   void* stream);

/* Stream-ordered forms of fastnn_cuda_memcpy_h2d / _d2h (cuda/kernels.cu:79-88, which are
 * synchronous): the copy is enqueued on `stream` and the call returns.  With pinned host memory a
 * caller can then run the upload of the next GEMM's operands, the GEMM (fastnn_b200_gemm_ex on a
 * second stream) and the download of the previous result at the same time; PCIe is full duplex.
 * The caller orders the streams with its own events. */
FASTNN_B200_API int fastnn_b200_memcpy_h2d_async(float* dst, const float* src, size_t size, void* stream);
FASTNN_B200_API int fastnn_b200_memcpy_d2h_async(float* dst, const float* src, size_t size, void* stream);
/* The same for fastnn_cuda_memcpy_d2d (cuda/kernels.cu:89-92).  Source and destination may lie on
 * different GPUs when both are mapped into this process (peer access / symmetric memory): the copy
 * engines then move the bytes over NVLink without occupying an SM -- the multi-GPU gather uses this
 * for finished row panels of C where the links, not the tensor cores, bound the step. */
FASTNN_B200_API int fastnn_b200_memcpy_d2d_async(float* dst, const float* src, size_t size, void* stream);

/* Kernel selection for tests and sweeps; applies to calls made by the CALLING THREAD only (other
 * threads keep the automatic choice).  policy: 0 = automatic (tcgen05 path whenever the
 * operands meet TMA's 16-byte alignment rules, SIMT path otherwise), 1 = SIMT path only,
 * 2 = tcgen05 path only (calls that cannot use it fail with -1), 3 = tcgen05 with single-CTA
 * 128-row tiles only, 4 = tcgen05 with CTA-pair 256-row tiles only, 5 = single-CTA tiles with the
 * K split done inside thread-block clusters (split_k = cluster size 2, 4 or 8; a call it cannot
 * serve -- fewer 32-deep k-blocks than split_k, a backward epilogue -- takes the workspace form
 * of the same split), 6 = automatic, but never the cluster form.  3 and 4 never take it either.
 * block_n in {0 (auto), 32, 64, 96, ..., 256} (rounded up to a multiple of 64 for CTA
 * pairs; with policy 4 also 512, the 256 x 512 pair tile); split_k >= 0 (0 = auto). */
FASTNN_B200_API int fastnn_b200_set_policy(int policy, int block_n, int split_k);

/* Which path the most recent call on this thread took: 1 = SIMT, 2 = tcgen05 1-CTA, 3 = tcgen05
 * 2-CTA, 4 = fused attention, 5 = conv2d, 6 = tcgen05 1-CTA with the K split inside clusters
 * (one launch, no workspace), 7 = a direct (FP32 FMA) convolution kernel, 8 = attention composed
 * from two batched GEMMs and a row softmax, 9 = conv2d with the input rows of every tile staged in
 * shared memory by TMA (5 is then the same kernel gathering from global memory), 11 = the conv2d weight
 * gradient with its gathered operand in tensor memory (5 is then the form that gathers from global
 * memory into shared memory); 0 before any call.
 * Also reports its tile and split choice. */
FASTNN_B200_API int fastnn_b200_last_path(int* block_n, int* split_k, int* num_ctas);

/* The host planner's choice for C[m,n] = op(A).op(B) (x batch), without launching: tile width,
 * K split, whether CTA pairs (256-row tiles) and whether the split runs inside thread-block
 * clusters.  Uses the initialised current device's SM and cluster counts, or a B200's when
 * there is none (so it also answers on a machine without a GPU).  0, or -1 on bad arguments.
 * No counterpart in the reference: cuBLAS picks its kernels internally (cuda/kernels.cu:431-526). */
FASTNN_B200_API int fastnn_b200_plan_query(int layout, int m, int n, int k, int batch, int* block_n,
                                           int* split_k, int* cta_pair, int* cluster_k);

/* Reads and clears the status words of the current device (synchronises the device).  0 = no
 * kernel reported a problem; otherwise the code of the first bounded wait that ran out.  Covers
 * both the kernels launched after fastnn_cuda_init and those of fastnn_b200_gemm_splitk_static
 * (which keeps a word of its own inside the library image); works whether or not
 * fastnn_cuda_init has been called, and allocates nothing. */
FASTNN_B200_API int fastnn_b200_device_status(unsigned int* status);

/* Exercises the bounded wait every kernel of this library uses on its mbarriers: one warp waits,
 * with a budget of budget_us microseconds (1 .. 100000, counted in SM clock ticks at the maximum
 * clock), on a barrier nothing arrives on.  Nothing else is in flight, so the launch cannot fault
 * or hang.  Returns 0 when the wait gave up as designed; the device status word then holds code
 * 0x1F0 until fastnn_b200_device_status reads and clears it.  waited_us (may be NULL) receives how
 * long the wait lasted.  Needs fastnn_cuda_init.  No counterpart in FastNN. */
FASTNN_B200_API int fastnn_b200_selftest_bounded_wait(unsigned int budget_us, unsigned int* waited_us);

/* Number of kernels this library has launched since load (all threads). */
FASTNN_B200_API unsigned long long fastnn_b200_launch_count(void);

/* Library version string, static storage. */
FASTNN_B200_API const char* fastnn_b200_version(void);

#ifdef __cplusplus
}
#endif

#endif /* FASTNN_B200_KERNELS_H */
