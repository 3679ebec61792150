/*
 * CPU oracle for the FastNN matrix-multiply path.  TEST INFRASTRUCTURE ONLY.
 *
 * This file restates, in plain C, the arithmetic FastNN's CPU tensors perform for
 * matmul / matmul_nt / matmul_tn / batched matmul and the Linear (+ReLU/GELU)
 * composition.  It exists to check the CUDA kernels and to be timed as the CPU
 * baseline; nothing in the product path may link or call it.
 *
 * The reference CPU path is Rust (src/tensor/ops.rs) and cannot be compiled in an
 * image without cargo/rustc, so this is a port, not the reference binary.  Its
 * pin is (1) the known-answer vectors in tests/golden/ that were derived by hand
 * from the loop nests cited below, and (2) the reference's own GPU library
 * (cuda/kernels.cu -> cuBLAS TF32) run on identical SplitMix64 inputs with the
 * tolerance of the reference's tests/cuda_parity.rs:50-58,109-111.
 *
 * Build: gcc -O2 -ffp-contract=off -fno-fast-math (rustc never contracts a*b+c
 * into an FMA, so contraction must stay off to keep the rounding identical).
 *
 * Every function cites the reference lines it follows (paths relative to the
 * FastNN project root).
 */
#include <math.h>
#include <pthread.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define ORACLE_API __attribute__((visibility("default")))

/* ---------------------------------------------------------------------------
 * SplitMix64 uniform [-1, 1) generator: tests/cuda_parity.rs:29-43 and
 * tests/gradcheck.rs:21-40 (the two copies are identical).
 * ------------------------------------------------------------------------- */
ORACLE_API void oracle_rand_data(float* out, size_t n, uint64_t seed) {
  uint64_t s = seed + 0x9E3779B97F4A7C15ull;           /* Rng::new */
  for (size_t i = 0; i < n; ++i) {
    s += 0x9E3779B97F4A7C15ull;                         /* next_u64 */
    uint64_t z = s;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    z ^= (z >> 31);
    /* unit(): (next >> 40) as f32 / 2^24 * 2 - 1, evaluated in f32 */
    float u = (float)(z >> 40) / (float)(1ull << 24);
    out[i] = u * 2.0f - 1.0f;
  }
}

/* ---------------------------------------------------------------------------
 * 2-D NN: src/tensor/ops.rs:366-377.  result starts at zero; loop order i, p, j;
 * one f32 multiply and one f32 add per term (no FMA).
 * Rows [row0, row1) only, so the row-parallel twin can reuse the same body.
 * ------------------------------------------------------------------------- */
static void nn_rows(const float* a, const float* b, float* c, size_t n, size_t k,
                    size_t row0, size_t row1) {
  for (size_t i = row0; i < row1; ++i) {
    float* ci = c + i * n;
    for (size_t j = 0; j < n; ++j) ci[j] = 0.0f;
    for (size_t p = 0; p < k; ++p) {
      const float a_val = a[i * k + p];
      const float* bp = b + p * n;
      for (size_t j = 0; j < n; ++j) ci[j] += a_val * bp[j];
    }
  }
}

ORACLE_API void oracle_matmul_nn(const float* a, const float* b, float* c,
                                 size_t m, size_t n, size_t k) {
  nn_rows(a, b, c, n, k, 0, m);
}

/* Row slab of the same product: rows [row0,row1) of C, written at c + row0*n.
 * Used for bounded CPU samples of the large configurations. */
ORACLE_API void oracle_matmul_nn_rows(const float* a, const float* b, float* c,
                                      size_t n, size_t k, size_t row0, size_t row1) {
  nn_rows(a, b, c, n, k, row0, row1);
}

/* ---------------------------------------------------------------------------
 * Transpose of the last two dims, CPU arm: src/tensor/ops.rs:528-555.
 * ------------------------------------------------------------------------- */
ORACLE_API void oracle_transpose(const float* in, float* out, size_t outer,
                                 size_t rows, size_t cols) {
  for (size_t o = 0; o < outer; ++o) {
    const size_t base = o * rows * cols;
    for (size_t i = 0; i < rows; ++i)
      for (size_t j = 0; j < cols; ++j)
        out[base + j * rows + i] = in[base + i * cols + j];
  }
}

/* ---------------------------------------------------------------------------
 * Batched NN with batch-1 broadcast: src/tensor/ops.rs:399-422.
 * ------------------------------------------------------------------------- */
ORACLE_API void oracle_matmul_batched(const float* a, const float* b, float* c,
                                      size_t m, size_t n, size_t k,
                                      size_t a_batch, size_t b_batch) {
  const size_t out_batch = a_batch > b_batch ? a_batch : b_batch;
  for (size_t bt = 0; bt < out_batch; ++bt) {
    const size_t ab = (a_batch == 1) ? 0 : bt;
    const size_t bb = (b_batch == 1) ? 0 : bt;
    nn_rows(a + ab * m * k, b + bb * k * n, c + bt * m * n, n, k, 0, m);
  }
}

/* ---------------------------------------------------------------------------
 * matmul_nt on CPU tensors = self.matmul(&other.transpose()):
 * src/tensor/ops.rs:476-477 (b is [batch, n, k]).
 * matmul_tn on CPU tensors = self.transpose().matmul(other):
 * src/tensor/ops.rs:516-517 (a is [batch, k, m]).
 * The transposed copy does not change the p-ascending summation order.
 * ------------------------------------------------------------------------- */
ORACLE_API int oracle_matmul_nt(const float* a, const float* b, float* c,
                                size_t m, size_t n, size_t k, size_t batch) {
  float* bt = (float*)malloc(sizeof(float) * (batch * n * k ? batch * n * k : 1));
  if (!bt) return -1;
  oracle_transpose(b, bt, batch, n, k);                 /* [n,k] -> [k,n] */
  oracle_matmul_batched(a, bt, c, m, n, k, batch, batch);
  free(bt);
  return 0;
}

ORACLE_API int oracle_matmul_tn(const float* a, const float* b, float* c,
                                size_t m, size_t n, size_t k, size_t batch) {
  float* at = (float*)malloc(sizeof(float) * (batch * k * m ? batch * k * m : 1));
  if (!at) return -1;
  oracle_transpose(a, at, batch, k, m);                 /* [k,m] -> [m,k] */
  oracle_matmul_batched(at, b, c, m, n, k, batch, batch);
  free(at);
  return 0;
}

/* ---------------------------------------------------------------------------
 * Epilogue math.
 *   bias add : src/nn/linear.rs:78-82 (expand bias over rows, then add)
 *   ReLU     : src/tensor/ops.rs:191-198   a.max(0.0)
 *   GELU     : src/tensor/ops.rs:220-230   0.5*a*(1+erff(a*FRAC_1_SQRT_2))
 * act: 0 none, 1 ReLU, 2 GELU(erf).
 * ------------------------------------------------------------------------- */
static inline float act_apply(float x, int act) {
  if (act == 1) return x > 0.0f ? x : 0.0f;            /* f32::max(a, 0.0) */
  if (act == 2) return 0.5f * x * (1.0f + erff(x * 0.70710678118654752440f));
  return x;
}

ORACLE_API void oracle_bias_act(float* c, const float* bias, size_t rows, size_t n, int act) {
  for (size_t i = 0; i < rows; ++i)
    for (size_t j = 0; j < n; ++j) {
      float v = c[i * n + j];
      if (bias) v = v + bias[j];
      c[i * n + j] = act_apply(v, act);
    }
}

/* Linear::forward, src/nn/linear.rs:71-82: y = x[batch,in] . transpose(W[out,in]) + bias. */
ORACLE_API int oracle_linear(const float* x, const float* w, const float* bias, float* y,
                             size_t batch, size_t in_f, size_t out_f, int act) {
  int rc = oracle_matmul_nt(x, w, y, batch, out_f, in_f, 1);
  if (rc) return rc;
  oracle_bias_act(y, bias, batch, out_f, act);
  return 0;
}

/* ---------------------------------------------------------------------------
 * Activation backward on CPU tensors, in place on the incoming gradient g[rows, n]:
 *   ReluBackward (src/autograd/backward_ops.rs:152-156): g * (x > 0 ? 1 : 0)
 *   GeluBackward (src/autograd/backward_ops.rs:208-214): g * (cdf + x * pdf) with
 *     cdf = 0.5 (1 + erff(x / sqrt 2)), pdf = exp(-x^2 / 2) / sqrt(2 pi), all in f32
 *     (same expression as cuda/kernels.cu:244-252).
 * followed by the bias gradient the expand in Linear::forward (src/nn/linear.rs:78-82) implies:
 * colsum[j] = sum over rows of g[i, j], rows added in order (sum_axis over axis 0).
 * colsum may be null.  act: 0 none, 1 ReLU, 2 GELU.
 * ------------------------------------------------------------------------- */
ORACLE_API void oracle_act_backward_colsum(float* g, const float* x, float* colsum, size_t rows,
                                           size_t n, int act) {
  for (size_t i = 0; i < rows; ++i)
    for (size_t j = 0; j < n; ++j) {
      float d = 1.0f;
      if (act == 1) d = x[i * n + j] > 0.0f ? 1.0f : 0.0f;
      if (act == 2) {
        const float v = x[i * n + j];
        const float cdf = 0.5f * (1.0f + erff(v * 0.70710678118654752440f));
        const float pdf = expf(-0.5f * v * v) * (1.0f / sqrtf(2.0f * 3.14159265358979323846f));
        d = cdf + v * pdf;
      }
      g[i * n + j] = g[i * n + j] * d;
    }
  if (colsum)
    for (size_t j = 0; j < n; ++j) {
      float s = 0.0f;
      for (size_t i = 0; i < rows; ++i) s += g[i * n + j];
      colsum[j] = s;
    }
}

/* ---------------------------------------------------------------------------
 * Conv2d::forward on CPU tensors, src/nn/conv.rs:97-123: for every (b, oc, oh, ow) the sum
 * starts at bias[oc] (0 without bias) and adds input * weight over ic, ki, kj in that nesting
 * order, skipping taps that fall into the zero padding.  NCHW, f32 throughout.
 * ------------------------------------------------------------------------- */
ORACLE_API void oracle_conv2d_forward(const float* x, const float* w, const float* bias, float* out,
                                      size_t batch, size_t ci, size_t co, size_t h, size_t wd,
                                      size_t kh, size_t kw, size_t sh, size_t sw, size_t ph, size_t pw) {
  const size_t oh_n = (h + 2 * ph - kh) / sh + 1;
  const size_t ow_n = (wd + 2 * pw - kw) / sw + 1;
  for (size_t b = 0; b < batch; ++b)
    for (size_t oc = 0; oc < co; ++oc)
      for (size_t oh = 0; oh < oh_n; ++oh)
        for (size_t ow = 0; ow < ow_n; ++ow) {
          float sum = bias ? bias[oc] : 0.0f;
          for (size_t ic = 0; ic < ci; ++ic)
            for (size_t ki = 0; ki < kh; ++ki)
              for (size_t kj = 0; kj < kw; ++kj) {
                const long ih = (long)(oh * sh + ki) - (long)ph;
                const long iw = (long)(ow * sw + kj) - (long)pw;
                if (ih >= 0 && ih < (long)h && iw >= 0 && iw < (long)wd)
                  sum += x[((b * ci + ic) * h + (size_t)ih) * wd + (size_t)iw] *
                         w[((oc * ci + ic) * kh + ki) * kw + kj];
              }
          out[((b * co + oc) * oh_n + oh) * ow_n + ow] = sum;
        }
}

/* Conv2dBackward on CPU tensors, src/autograd/backward_ops.rs:753-770: one pass over
 * (b, oc, oh, ow, ic, ki, kj) adding go * w into grad_input and go * input into grad_weight
 * (both start at zero).  gi or gw may be null. */
ORACLE_API void oracle_conv2d_backward(const float* x, const float* w, const float* go, float* gi,
                                       float* gw, size_t batch, size_t ci, size_t co, size_t h,
                                       size_t wd, size_t kh, size_t kw, size_t sh, size_t sw, size_t ph,
                                       size_t pw) {
  const size_t oh_n = (h + 2 * ph - kh) / sh + 1;
  const size_t ow_n = (wd + 2 * pw - kw) / sw + 1;
  if (gi) for (size_t i = 0; i < batch * ci * h * wd; ++i) gi[i] = 0.0f;
  if (gw) for (size_t i = 0; i < co * ci * kh * kw; ++i) gw[i] = 0.0f;
  for (size_t b = 0; b < batch; ++b)
    for (size_t oc = 0; oc < co; ++oc)
      for (size_t oh = 0; oh < oh_n; ++oh)
        for (size_t ow = 0; ow < ow_n; ++ow) {
          const float g = go[((b * co + oc) * oh_n + oh) * ow_n + ow];
          for (size_t ic = 0; ic < ci; ++ic)
            for (size_t ki = 0; ki < kh; ++ki)
              for (size_t kj = 0; kj < kw; ++kj) {
                const long ih = (long)(oh * sh + ki) - (long)ph;
                const long iw = (long)(ow * sw + kj) - (long)pw;
                if (ih >= 0 && ih < (long)h && iw >= 0 && iw < (long)wd) {
                  const size_t wi = ((oc * ci + ic) * kh + ki) * kw + kj;
                  const size_t ii = ((b * ci + ic) * h + (size_t)ih) * wd + (size_t)iw;
                  if (gi) gi[ii] += g * w[wi];
                  if (gw) gw[wi] += g * x[ii];
                }
              }
        }
}

/* ---------------------------------------------------------------------------
 * Attention probabilities used as the left operand of the batched P.V product:
 * scores*scale (src/nn/transformer.rs:94) + additive causal mask 0/-1e9
 * (src/nn/transformer.rs:22-27) -> row softmax (src/tensor/ops.rs:273-284).
 * In place on s[batch, t, t].
 * ------------------------------------------------------------------------- */
ORACLE_API void oracle_causal_softmax(float* s, size_t batch, size_t t, float scale) {
  for (size_t b = 0; b < batch; ++b)
    for (size_t qi = 0; qi < t; ++qi) {
      float* row = s + (b * t + qi) * t;
      for (size_t ki = 0; ki < t; ++ki) {
        float v = row[ki] * scale;
        row[ki] = v + (ki > qi ? -1e9f : 0.0f);
      }
      float mx = -INFINITY;
      for (size_t ki = 0; ki < t; ++ki) mx = row[ki] > mx ? row[ki] : mx;
      float sum = 0.0f;
      for (size_t ki = 0; ki < t; ++ki) sum += expf(row[ki] - mx);
      for (size_t ki = 0; ki < t; ++ki) row[ki] = expf(row[ki] - mx) / sum;
    }
}

/* Rectangular form of the same composition (t_q queries, t_k keys), mask optional:
 * mul_scalar(scale) -> (+ 0/-1e9 mask where key > query) -> row softmax over keys.
 * In place on s[batch, t_q, t_k]. */
ORACLE_API void oracle_masked_softmax(float* s, size_t batch, size_t tq, size_t tk, float scale,
                                      int causal) {
  for (size_t b = 0; b < batch; ++b)
    for (size_t qi = 0; qi < tq; ++qi) {
      float* row = s + (b * tq + qi) * tk;
      for (size_t ki = 0; ki < tk; ++ki) {
        float v = row[ki] * scale;
        if (causal) v = v + (ki > qi ? -1e9f : 0.0f);
        row[ki] = v;
      }
      float mx = -INFINITY;
      for (size_t ki = 0; ki < tk; ++ki) mx = row[ki] > mx ? row[ki] : mx;
      float sum = 0.0f;
      for (size_t ki = 0; ki < tk; ++ki) sum += expf(row[ki] - mx);
      for (size_t ki = 0; ki < tk; ++ki) row[ki] = expf(row[ki] - mx) / sum;
    }
}

/* The same with a general additive mask [tq, tk] shared by every batch entry, the form of
 * FastNN's cached mask tensor (src/nn/transformer.rs:15-30; added by `scores.add(&mask)`, :99-105):
 * mul_scalar(scale) -> + mask (+ the causal 0/-1e9 term) -> row softmax.  mask may be NULL. */
ORACLE_API void oracle_masked_softmax_add(float* s, size_t batch, size_t tq, size_t tk, float scale,
                                          int causal, const float* mask) {
  for (size_t b = 0; b < batch; ++b)
    for (size_t qi = 0; qi < tq; ++qi) {
      float* row = s + (b * tq + qi) * tk;
      for (size_t ki = 0; ki < tk; ++ki) {
        float v = row[ki] * scale;
        if (mask) v = v + mask[qi * tk + ki];
        if (causal) v = v + (ki > qi ? -1e9f : 0.0f);
        row[ki] = v;
      }
      float mx = -INFINITY;
      for (size_t ki = 0; ki < tk; ++ki) mx = row[ki] > mx ? row[ki] : mx;
      float sum = 0.0f;
      for (size_t ki = 0; ki < tk; ++ki) sum += expf(row[ki] - mx);
      for (size_t ki = 0; ki < tk; ++ki) row[ki] = expf(row[ki] - mx) / sum;
    }
}

/* ---------------------------------------------------------------------------
 * Row-parallel twin.  NOT in the reference (its rayon dependency is never
 * called): the outer row loop of the same nest is split over threads, each row
 * keeps its p-ascending order, so results are bit-identical to the serial form.
 * ------------------------------------------------------------------------- */
typedef struct {
  const float *a, *b;
  float* c;
  size_t n, k, row0, row1;
} slab_t;

static void* slab_main(void* p) {
  slab_t* s = (slab_t*)p;
  nn_rows(s->a, s->b, s->c, s->n, s->k, s->row0, s->row1);
  return NULL;
}

ORACLE_API int oracle_matmul_nn_rows_par(const float* a, const float* b, float* c,
                                         size_t n, size_t k, size_t row0, size_t row1,
                                         int nthreads) {
  if (nthreads < 1) nthreads = 1;
  if (nthreads > 256) nthreads = 256;
  pthread_t th[256];
  slab_t sl[256];
  const size_t rows = row1 - row0;
  int started = 0;
  for (int t = 0; t < nthreads; ++t) {
    sl[t].a = a; sl[t].b = b; sl[t].c = c; sl[t].n = n; sl[t].k = k;
    sl[t].row0 = row0 + rows * (size_t)t / (size_t)nthreads;
    sl[t].row1 = row0 + rows * (size_t)(t + 1) / (size_t)nthreads;
    if (pthread_create(&th[t], NULL, slab_main, &sl[t]) != 0) break;
    ++started;
  }
  for (int t = 0; t < started; ++t) pthread_join(th[t], NULL);
  return started == nthreads ? 0 : -1;
}

ORACLE_API int oracle_matmul_nn_par(const float* a, const float* b, float* c,
                                    size_t m, size_t n, size_t k, int nthreads) {
  return oracle_matmul_nn_rows_par(a, b, c, n, k, 0, m, nthreads);
}
