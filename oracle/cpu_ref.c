/* CPU oracle (plain C + OpenMP) for the BatchNorm / ApplyAdam / BiasAdd +
 * activation path.
 *
 * TEST INFRASTRUCTURE ONLY: used by the tests as a second checker next to
 * oracle/np_ref.py and by the benchmark as the timed CPU baseline (all host
 * threads).  The product never links or loads it.
 *
 * The arithmetic restates what TensorFlow's CPU kernels return for these ops,
 * following the conventions documented in the reference plugin:
 *   BatchNorm outputs  musa_ext/kernels/nn/musa_fused_batchnorm_op.cc:126-170
 *   BatchNorm gradient musa_ext/kernels/nn/musa_fused_batchnorm_op.cc:265-277,
 *                      musa_ext/kernels/nn/musa_fused_batchnorm_kernel.mu:23-29
 *   Adam               musa_ext/kernels/training/musa_apply_sparse_adam_kernel.mu:140-157,
 *                      musa_ext/kernels/training/musa_applyadam_op.cc:236-246
 *   BiasAdd            musa_ext/kernels/nn/musa_biasadd_op.cc:33-57
 * Parity against TensorFlow itself is unpinned for BatchNorm (see the header
 * of oracle/np_ref.py); this file is checked against np_ref.py in the tests.
 *
 * dtype codes: 0 float32, 1 float16, 2 bfloat16 (16-bit values as uint16_t).
 * Tensors are channels-last: [rows, channels].
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

static inline float bf16_to_f32(uint16_t h) {
  uint32_t u = (uint32_t)h << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}

static inline uint16_t f32_to_bf16(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x40u);
  u += 0x7fffu + ((u >> 16) & 1u); /* round to nearest even */
  return (uint16_t)(u >> 16);
}

static inline float f16_to_f32(uint16_t h) {
  _Float16 v;
  memcpy(&v, &h, 2);
  return (float)v;
}

static inline uint16_t f32_to_f16(float f) {
  _Float16 v = (_Float16)f; /* round to nearest even */
  uint16_t h;
  memcpy(&h, &v, 2);
  return h;
}

static inline float load(const void* p, int dtype, int64_t i) {
  if (dtype == 0) return ((const float*)p)[i];
  if (dtype == 1) return f16_to_f32(((const uint16_t*)p)[i]);
  return bf16_to_f32(((const uint16_t*)p)[i]);
}

static inline void store(void* p, int dtype, int64_t i, float v) {
  if (dtype == 0)
    ((float*)p)[i] = v;
  else if (dtype == 1)
    ((uint16_t*)p)[i] = f32_to_f16(v);
  else
    ((uint16_t*)p)[i] = f32_to_bf16(v);
}

int cpu_ref_num_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

/* Thread count of the following calls (a launcher may have pinned
 * OMP_NUM_THREADS=1 for its worker processes). */
void cpu_ref_set_num_threads(int n) {
#ifdef _OPENMP
  if (n > 0) omp_set_num_threads(n);
#else
  (void)n;
#endif
}

/* Per-channel sums of f(row) over row blocks: each thread keeps double
 * accumulators for all channels, combined in thread order. */
typedef void (*row_fn)(const void* a, const void* b, int dtype, int64_t row,
                       int64_t channels, const double* aux, double* s1,
                       double* s2);

static void reduce_rows(const void* a, const void* b, int dtype, int64_t rows,
                        int64_t channels, const double* aux, row_fn fn,
                        double* out1, double* out2) {
  int nt = cpu_ref_num_threads();
  double* acc = (double*)calloc((size_t)nt * 2 * channels, sizeof(double));
#pragma omp parallel num_threads(nt)
  {
#ifdef _OPENMP
    int t = omp_get_thread_num();
#else
    int t = 0;
#endif
    double* s1 = acc + (size_t)t * 2 * channels;
    double* s2 = s1 + channels;
#pragma omp for schedule(static)
    for (int64_t r = 0; r < rows; ++r) fn(a, b, dtype, r, channels, aux, s1, s2);
  }
  for (int64_t c = 0; c < channels; ++c) {
    double t1 = 0.0, t2 = 0.0;
    for (int t = 0; t < nt; ++t) {
      t1 += acc[(size_t)t * 2 * channels + c];
      t2 += acc[(size_t)t * 2 * channels + channels + c];
    }
    out1[c] = t1;
    if (out2) out2[c] = t2;
  }
  free(acc);
}

static void row_sum(const void* x, const void* unused, int dtype, int64_t r,
                    int64_t channels, const double* aux, double* s1,
                    double* s2) {
  (void)unused;
  (void)aux;
  (void)s2;
  for (int64_t c = 0; c < channels; ++c) s1[c] += load(x, dtype, r * channels + c);
}

static void row_sqdev(const void* x, const void* unused, int dtype, int64_t r,
                      int64_t channels, const double* mean, double* s1,
                      double* s2) {
  (void)unused;
  (void)s2;
  for (int64_t c = 0; c < channels; ++c) {
    double d = (double)load(x, dtype, r * channels + c) - mean[c];
    s1[c] += d * d;
  }
}

static void row_grad(const void* dy, const void* x, int dtype, int64_t r,
                     int64_t channels, const double* mean, double* s1,
                     double* s2) {
  for (int64_t c = 0; c < channels; ++c) {
    double g = load(dy, dtype, r * channels + c);
    s1[c] += g;
    s2[c] += g * ((double)load(x, dtype, r * channels + c) - mean[c]);
  }
}

/* FusedBatchNormV3, training mode, channels-last, exponential_avg_factor = 1. */
void cpu_bn_fwd_train(int dtype, const void* x, const float* scale,
                      const float* offset, void* y, float* batch_mean,
                      float* batch_var, float* saved_mean, float* saved_var,
                      int64_t rows, int64_t channels, float epsilon) {
  double* mean = (double*)malloc(sizeof(double) * channels);
  double* var = (double*)malloc(sizeof(double) * channels);
  float* a = (float*)malloc(sizeof(float) * channels);
  reduce_rows(x, NULL, dtype, rows, channels, NULL, row_sum, mean, NULL);
  for (int64_t c = 0; c < channels; ++c) mean[c] /= (double)rows;
  reduce_rows(x, NULL, dtype, rows, channels, mean, row_sqdev, var, NULL);
  for (int64_t c = 0; c < channels; ++c) {
    var[c] /= (double)rows;
    double unbiased = rows > 1 ? var[c] * ((double)rows / (double)(rows - 1)) : var[c];
    saved_mean[c] = (float)mean[c];
    saved_var[c] = (float)var[c];
    batch_mean[c] = (float)mean[c];
    batch_var[c] = (float)unbiased;
    a[c] = scale[c] * (1.0f / sqrtf(saved_var[c] + epsilon));
  }
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < rows; ++r) {
    for (int64_t c = 0; c < channels; ++c) {
      float d = load(x, dtype, r * channels + c) - saved_mean[c];
      store(y, dtype, r * channels + c, d * a[c] + offset[c]);
    }
  }
  free(mean);
  free(var);
  free(a);
}

/* FusedBatchNormGradV3, channels-last. */
void cpu_bn_grad(int dtype, const void* dy, const void* x, const float* scale,
                 const float* mean, const float* variance, void* dx,
                 float* dscale, float* doffset, int64_t rows, int64_t channels,
                 float epsilon, int is_training) {
  double* mean64 = (double*)malloc(sizeof(double) * channels);
  double* s1 = (double*)malloc(sizeof(double) * channels);
  double* s2 = (double*)malloc(sizeof(double) * channels);
  float* ca = (float*)malloc(sizeof(float) * channels);
  float* cb = (float*)malloc(sizeof(float) * channels);
  float* cc = (float*)malloc(sizeof(float) * channels);
  for (int64_t c = 0; c < channels; ++c) mean64[c] = mean[c];
  reduce_rows(dy, x, dtype, rows, channels, mean64, row_grad, s1, s2);
  for (int64_t c = 0; c < channels; ++c) {
    float inv = 1.0f / sqrtf(variance[c] + epsilon);
    doffset[c] = (float)s1[c];
    dscale[c] = (float)(s2[c] * (double)inv);
    ca[c] = scale[c] * inv;
    cb[c] = is_training ? (float)(s1[c] / (double)rows) : 0.0f;
    cc[c] = is_training ? (float)(s2[c] * (double)inv * (double)inv / (double)rows) : 0.0f;
  }
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < rows; ++r) {
    for (int64_t c = 0; c < channels; ++c) {
      float g = load(dy, dtype, r * channels + c);
      float d = load(x, dtype, r * channels + c) - mean[c];
      store(dx, dtype, r * channels + c, ca[c] * (g - cb[c] - d * cc[c]));
    }
  }
  free(mean64);
  free(s1);
  free(s2);
  free(ca);
  free(cb);
  free(cc);
}

/* ResourceApplyAdam, float32, use_nesterov = false; alpha computed by the
 * caller in float64 as the op does. */
void cpu_adam_f32(float* var, float* m, float* v, const float* grad, float beta1,
                  float beta2, float epsilon, float alpha, int64_t n) {
  const float omb1 = 1.0f - beta1, omb2 = 1.0f - beta2;
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; ++i) {
    const float g = grad[i];
    const float m_new = beta1 * m[i] + omb1 * g;
    const float v_new = beta2 * v[i] + omb2 * g * g;
    m[i] = m_new;
    v[i] = v_new;
    var[i] -= alpha * m_new / (sqrtf(v_new) + epsilon);
  }
}

/* y = act(x + bias[col]) on [rows, channels]; act: 0 identity, 1 relu,
 * 2 x*sigmoid(x+b), 3 sigmoid(x+b).  16-bit types round after every un-fused
 * op (BiasAdd, Sigmoid, Mul), as separate TensorFlow ops do. */
void cpu_bias_act(int dtype, const void* x, const void* bias, void* y,
                  int64_t rows, int64_t channels, int act) {
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < rows; ++r) {
    for (int64_t c = 0; c < channels; ++c) {
      const int64_t i = r * channels + c;
      const float xv = load(x, dtype, i);
      float t = xv + (bias ? load(bias, dtype, c) : 0.0f);
      if (dtype != 0) {
        store(y, dtype, i, t);
        t = load(y, dtype, i);
      }
      float out;
      if (act == 0) {
        out = t;
      } else if (act == 1) {
        out = t < 0.0f ? 0.0f : t;
      } else {
        float s = (float)(1.0 / (1.0 + exp(-(double)t)));
        if (dtype != 0) {
          store(y, dtype, i, s);
          s = load(y, dtype, i);
        }
        out = act == 2 ? xv * s : s;
      }
      store(y, dtype, i, out);
    }
  }
}
