/* C ABI of libmusa_plugin_kernels.so: the device-code launcher layer of the
 * `tensorflow_musa` plugin, rebuilt as hand-written CUDA for NVIDIA B200
 * (sm_100a).
 *
 * The reference plugin keeps its device code behind `extern "C" Launch*()`
 * functions that the C++ OpKernels call from `Compute()`; this header declares
 * the same layer for the memory-bound training path (FusedBatchNorm forward and
 * gradient, ApplyAdam and the optimizers of its shape, BiasAdd + activation
 * and its backward).  Each declaration cites the
 * reference interface it replaces, as `path:line` inside the reference project.
 *
 * Conventions shared by every launcher (they are the reference's):
 *   - pointers are borrowed DEVICE pointers, valid until the stream work ends;
 *   - host scalars are passed by value; nothing is read back from the device;
 *   - a launcher enqueues work on `stream` and returns without synchronising;
 *   - a launcher allocates nothing and keeps no state between calls beyond
 *     per-device launch constants (SM count, occupancy) cached on first use
 *     and the test knobs at the end of this file; scratch memory is
 *     passed in by the caller (TF: `OpKernelContext::allocate_temp`) after a
 *     `*WorkspaceBytes()` query;
 *   - a launcher is re-entrant (TF calls Compute() from several threads);
 *   - empty inputs (`n <= 0`) return at once.
 * The Adam launchers keep the reference's `void` return (the caller polls
 * `cudaGetLastError()`, as musa_applyadam_op.cc:258-261 does).  The launchers
 * that are new here return an int: 0 on success, a positive `cudaError_t` from
 * the launch, or a negative MUSA_KERNELS_E* code for an argument the launcher
 * refuses.  No launcher falls back to the host.
 */
#ifndef MUSA_PLUGIN_KERNELS_H_
#define MUSA_PLUGIN_KERNELS_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Opaque CUDA stream handle (`cudaStream_t`); declared here so that a C caller
 * does not need the CUDA headers.  The reference type is `musaStream_t`. */
#ifndef __DRIVER_TYPES_H__
typedef struct CUstream_st* cudaStream_t;
#endif

#define MUSA_KERNELS_OK 0
#define MUSA_KERNELS_EINVAL (-1)      /* null pointer / negative size          */
#define MUSA_KERNELS_EWORKSPACE (-2)  /* workspace missing or too small        */
#define MUSA_KERNELS_EUNSUPPORTED (-3)/* dtype / activation code not known     */
#define MUSA_KERNELS_ETOOLARGE (-4)   /* size beyond what the entry point holds */

/* Library identity; lets a loader check that it found the sm_100a build. */
const char* MusaKernelsVersion(void);
/* Compute capability the device code was compiled for (100 => sm_100a). */
int MusaKernelsTargetArch(void);

/* ------------------------------------------------------------------ Adam -- */

/* fp32 var/m/v/grad, one streaming pass: m = b1*m + (1-b1)*g;
 * v = b2*v + (1-b2)*g*g; var -= alpha*m/(sqrt(v)+eps), `alpha` being the
 * bias-corrected learning rate that the op computes on the host in fp64.
 * Replaces tensorflow::musa::LaunchResourceApplyAdamFloat
 * (musa_ext/kernels/training/musa_apply_sparse_adam_kernel.mu:159-169; declared
 * for the op at musa_ext/kernels/training/musa_applyadam_op.cc:34-37; the
 * reference gives this one C++ linkage, the argument list is unchanged). */
void LaunchResourceApplyAdamFloat(float* var, float* m, float* v,
                                  const float* grad, float beta1, float beta2,
                                  float epsilon, float alpha, int64_t total,
                                  cudaStream_t stream);

/* var/m/v/grad all bf16 (or all fp16): widen, fp32 arithmetic, round to
 * nearest even on store.  `use_nesterov` swaps the numerator for
 * b1*m + (1-b1)*g.  Replaces LaunchApplyAdamSameType_{BFloat16,Half}
 * (musa_ext/kernels/training/musa_applyadam_bf16_kernel.mu:133-156; declared
 * for the op at musa_ext/kernels/training/musa_applyadam_op.cc:20-29). */
void LaunchApplyAdamSameType_BFloat16(void* var, void* m, void* v,
                                      const void* grad, float lr_t, float beta1,
                                      float beta2, float epsilon, int64_t n,
                                      bool use_nesterov, cudaStream_t stream);
void LaunchApplyAdamSameType_Half(void* var, void* m, void* v, const void* grad,
                                  float lr_t, float beta1, float beta2,
                                  float epsilon, int64_t n, bool use_nesterov,
                                  cudaStream_t stream);

/* fp32 var/m/v with a grad of fp32, fp16 or bf16 (op
 * MusaResourceApplyAdamMixed).  Replaces LaunchApplyAdamMixed_{Float,Half,
 * BFloat16} (musa_ext/kernels/training/musa_applyadam_mixed_kernel.mu:108-137;
 * declared at musa_ext/kernels/training/musa_applyadam_mixed_op.cc:49-62). */
void LaunchApplyAdamMixed_Float(float* var, float* m, float* v,
                                const void* grad, float lr_t, float beta1,
                                float beta2, float epsilon, int64_t n,
                                bool use_nesterov, cudaStream_t stream);
void LaunchApplyAdamMixed_Half(float* var, float* m, float* v, const void* grad,
                               float lr_t, float beta1, float beta2,
                               float epsilon, int64_t n, bool use_nesterov,
                               cudaStream_t stream);
void LaunchApplyAdamMixed_BFloat16(float* var, float* m, float* v,
                                   const void* grad, float lr_t, float beta1,
                                   float beta2, float epsilon, int64_t n,
                                   bool use_nesterov, cudaStream_t stream);

/* ResourceApplyAdam / ApplyAdam for double tensors, one streaming pass
 * (56 B/element).  No launcher of this name exists in the reference: it serves
 * T = double with a chain of thirteen element-wise library calls
 * (musa_ext/kernels/training/musa_applyadam_op.cc:297-415, registrations
 * :672-687), each storing a double tensor.  This launcher performs the same
 * operations in the same order with one IEEE rounding each:
 *   m = m*b1 + g*(1-b1);  v = v*b2 + (g*g)*(1-b2);
 *   var = var - (m / (sqrt(v) + eps)) * alpha
 * (`alpha`: the bias-corrected step the op computes on the host, :236-246).
 * With use_nesterov the numerator is m*b1 + g*(1-b1), as in TensorFlow's CPU
 * kernel (the chain itself ignores the attribute). */
void LaunchApplyAdam_F64(double* var, double* m, double* v, const double* grad,
                         double alpha, double beta1, double beta2, double epsilon,
                         int64_t n, bool use_nesterov, cudaStream_t stream);

/* ------------------------- Nadam, RMSProp, gradient descent (same shape) -- */

/* ResourceApplyNadam over n elements, in place:
 *   m <- beta1*m + (1-beta1)*g;  v <- beta2*v + (1-beta2)*g*g
 *   var <- var - lr * ((beta1*m + (1-beta1)*g) / (1-beta1_power))
 *                   / (sqrt(v / (1-beta2_power)) + epsilon)
 * Scalars are float for every tensor type and 1-x is formed in float, as in
 * the reference launcher.  float / half / bfloat16 tensors compute in fp32
 * and round to nearest even on store (the reference's bfloat16 store
 * truncates); double tensors compute in fp64 (the reference narrows them to
 * fp32).  C names for the C++ template LaunchResourceApplyNadamKernel<T>
 * (musa_ext/kernels/training/musa_resource_apply_nadam_kernel.mu:48-104;
 * declared in musa_ext/kernels/training/musa_resource_apply_nadam_op.cc). */
void LaunchResourceApplyNadam_Float(void* var, void* m, void* v, const void* grad,
                                    float beta1_power, float beta2_power, float lr,
                                    float beta1, float beta2, float epsilon,
                                    int64_t n, cudaStream_t stream);
void LaunchResourceApplyNadam_Half(void* var, void* m, void* v, const void* grad,
                                   float beta1_power, float beta2_power, float lr,
                                   float beta1, float beta2, float epsilon,
                                   int64_t n, cudaStream_t stream);
void LaunchResourceApplyNadam_BFloat16(void* var, void* m, void* v,
                                       const void* grad, float beta1_power,
                                       float beta2_power, float lr, float beta1,
                                       float beta2, float epsilon, int64_t n,
                                       cudaStream_t stream);
void LaunchResourceApplyNadam_Double(void* var, void* m, void* v,
                                     const void* grad, float beta1_power,
                                     float beta2_power, float lr, float beta1,
                                     float beta2, float epsilon, int64_t n,
                                     cudaStream_t stream);

/* ResourceApplyRMSProp / ApplyRMSProp over n elements, in place:
 *   ms <- rho*ms + (1-rho)*g*g;  mom <- momentum*mom + lr*g / sqrt(ms + epsilon)
 *   var <- var - mom
 * and the centered form with mg <- rho*mg + (1-rho)*g and the denominator
 * sqrt(ms - mg*mg + epsilon).  Scalars arrive as double and are narrowed to
 * the compute type (fp32; fp64 for double tensors) before 1-rho is formed.
 * C names for LaunchFusedResourceApplyRMSPropKernel<T> and
 * LaunchFusedResourceApplyCenteredRMSPropKernel<T>
 * (musa_ext/kernels/training/musa_applyrmsprop_kernel.mu:72-133, :236-340),
 * which return without synchronising the stream, unlike the reference op's
 * CheckLaunchAndSync (musa_ext/kernels/training/musa_applyrmsprop_op.cc:170-182). */
void LaunchFusedResourceApplyRMSProp_Float(void* var, void* ms, void* mom,
                                           const void* grad, double lr, double rho,
                                           double momentum, double epsilon,
                                           int64_t n, cudaStream_t stream);
void LaunchFusedResourceApplyRMSProp_Half(void* var, void* ms, void* mom,
                                          const void* grad, double lr, double rho,
                                          double momentum, double epsilon,
                                          int64_t n, cudaStream_t stream);
void LaunchFusedResourceApplyRMSProp_BFloat16(void* var, void* ms, void* mom,
                                              const void* grad, double lr,
                                              double rho, double momentum,
                                              double epsilon, int64_t n,
                                              cudaStream_t stream);
void LaunchFusedResourceApplyRMSProp_Double(void* var, void* ms, void* mom,
                                            const void* grad, double lr,
                                            double rho, double momentum,
                                            double epsilon, int64_t n,
                                            cudaStream_t stream);
void LaunchFusedResourceApplyCenteredRMSProp_Float(
    void* var, void* mg, void* ms, void* mom, const void* grad, double lr,
    double rho, double momentum, double epsilon, int64_t n, cudaStream_t stream);
void LaunchFusedResourceApplyCenteredRMSProp_Half(
    void* var, void* mg, void* ms, void* mom, const void* grad, double lr,
    double rho, double momentum, double epsilon, int64_t n, cudaStream_t stream);
void LaunchFusedResourceApplyCenteredRMSProp_BFloat16(
    void* var, void* mg, void* ms, void* mom, const void* grad, double lr,
    double rho, double momentum, double epsilon, int64_t n, cudaStream_t stream);
void LaunchFusedResourceApplyCenteredRMSProp_Double(
    void* var, void* mg, void* ms, void* mom, const void* grad, double lr,
    double rho, double momentum, double epsilon, int64_t n, cudaStream_t stream);

/* ResourceApplyAdagradV2 / ApplyAdagradV2 over n elements, in place:
 *   accum <- accum + g*g (only with update_slots);
 *   var <- var - lr * g / (sqrt(accum) + epsilon).
 * C names for LaunchFusedApplyAdagradV2Kernel<T>
 * (musa_ext/kernels/training/musa_applyadagrad_kernel.mu:55-79; declared at
 * musa_ext/kernels/training/musa_applyadagrad_op.cc:36-40); no stream
 * synchronisation after the launch. */
void LaunchFusedApplyAdagradV2_Float(void* var, void* accum, const void* grad,
                                     double lr, double epsilon, bool update_slots,
                                     int64_t n, cudaStream_t stream);
void LaunchFusedApplyAdagradV2_Half(void* var, void* accum, const void* grad,
                                    double lr, double epsilon, bool update_slots,
                                    int64_t n, cudaStream_t stream);
void LaunchFusedApplyAdagradV2_BFloat16(void* var, void* accum, const void* grad,
                                        double lr, double epsilon, bool update_slots,
                                        int64_t n, cudaStream_t stream);
void LaunchFusedApplyAdagradV2_Double(void* var, void* accum, const void* grad,
                                      double lr, double epsilon, bool update_slots,
                                      int64_t n, cudaStream_t stream);

/* ResourceApplyGradientDescent: var <- var - alpha * grad over n elements.
 * Same names and arguments as the reference
 * (musa_ext/kernels/training/musa_applygradientdescent_kernel.mu:106-122). */
void LaunchResourceApplyGradientDescentFloat(float* var, const float* grad,
                                             float alpha, int64_t n,
                                             cudaStream_t stream);
void LaunchResourceApplyGradientDescentFloatBFloat16(float* var, const void* grad,
                                                     float alpha, int64_t n,
                                                     cudaStream_t stream);
/* The same update for half / bfloat16 variables: alpha*grad is rounded to the
 * tensor's type before the subtraction, like the two stored results of the
 * muDNN MUL and SUB passes that the reference runs for these types
 * (musa_ext/kernels/training/musa_applygradientdescent_op.cc:163-199). */
void LaunchResourceApplyGradientDescent_Half(void* var, const void* grad,
                                             float alpha, int64_t n,
                                             cudaStream_t stream);
void LaunchResourceApplyGradientDescent_BFloat16(void* var, const void* grad,
                                                 float alpha, int64_t n,
                                                 cudaStream_t stream);

/* MusaGroupedResourceApplyGradientDescentMixed, table form: the reference's
 * interface (musa_ext/kernels/training/musa_applygradientdescent_kernel.mu:
 * 124-146).  All five tables are DEVICE arrays; CTA b of the `total_blocks`
 * launched belongs to the tensor t with block_offsets[t] <= b <
 * block_offsets[t + 1] and strides over that tensor together with the other
 * CTAs of t (256 threads per CTA). */
void LaunchGroupedResourceApplyGradientDescentFloat(
    const uint64_t* var_ptrs, const uint64_t* grad_ptrs, const float* alphas,
    const int64_t* sizes, const int64_t* block_offsets, int num_tensors,
    int total_blocks, cudaStream_t stream);
void LaunchGroupedResourceApplyGradientDescentFloatBFloat16(
    const uint64_t* var_ptrs, const uint64_t* grad_ptrs, const float* alphas,
    const int64_t* sizes, const int64_t* block_offsets, int num_tensors,
    int total_blocks, cudaStream_t stream);

/* The grouped update from HOST tables: the descriptors of up to
 * MUSA_SGD_GROUP_MAX tensors travel in the kernel's parameter space, so the
 * op needs none of the five temporaries and staging copies of the table form
 * (musa_ext/kernels/training/musa_applygradientdescent_op.cc:388-428).  More
 * tensors are split over several launches.  var_ptrs[i] / delta_ptrs[i] are
 * device pointers to sizes[i] floats and sizes[i] floats or bfloat16s.
 * No counterpart symbol in the reference. */
#define MUSA_SGD_GROUP_MAX 256
int LaunchGroupedGradientDescentHostTable(void* const* var_ptrs,
                                          const void* const* delta_ptrs,
                                          const float* alphas,
                                          const int64_t* sizes, int num_tensors,
                                          int delta_is_bfloat16,
                                          cudaStream_t stream);

/* ------------------------------------------------ BiasAdd + activation -- */

/* Activation codes of LaunchBiasAct_*. */
#define MUSA_ACT_IDENTITY 0 /* y = x + b                  (BiasAdd)           */
#define MUSA_ACT_RELU 1     /* y = max(x + b, 0)          (Relu(BiasAdd))     */
#define MUSA_ACT_SWISH 2    /* y = x * sigmoid(x + b)     (Mul(x,Sigmoid(..)))*/
#define MUSA_ACT_SIGMOID 3  /* y = sigmoid(x + b)         (Sigmoid(BiasAdd))  */

/* One read of x and one write of y for the whole chain.  x and y are viewed
 * as [outer, channels, inner] with the bias indexed by the middle axis:
 * NHWC / 2-D inputs pass inner = 1, NCHW passes outer = N, inner = H*W.
 * `bias == NULL` applies the activation alone (the Relu and Sigmoid ops).
 * 16-bit types compute in fp32 and round once on store.
 * Replaces the muDNN Binary ADD with a stride-0 bias view
 * (musa_ext/kernels/nn/musa_biasadd_op.cc:46-57), the muDNN Unary RELU and
 * SIGMOID passes (musa_ext/kernels/nn/musa_relu_op.cc:33-36,
 * musa_ext/kernels/nn/musa_sigmoid_op.cc:29-33) and the unused
 * LaunchBiasAddReluKernel<T> (musa_ext/kernels/fusion/musa_linear_relu_kernel.mu:
 * 69-77). */
int LaunchBiasAct_F32(const void* x, const void* bias, void* y, int64_t outer,
                      int64_t channels, int64_t inner, int act,
                      cudaStream_t stream);
int LaunchBiasAct_F16(const void* x, const void* bias, void* y, int64_t outer,
                      int64_t channels, int64_t inner, int act,
                      cudaStream_t stream);
int LaunchBiasAct_BF16(const void* x, const void* bias, void* y, int64_t outer,
                       int64_t channels, int64_t inner, int act,
                       cudaStream_t stream);
/* BiasAdd for the other registered dtypes (musa_ext/kernels/nn/musa_biasadd_op.cc:75-80:
 * double, int32, int64); identity and relu only. */
int LaunchBiasAct_F64(const void* x, const void* bias, void* y, int64_t outer,
                      int64_t channels, int64_t inner, int act,
                      cudaStream_t stream);
int LaunchBiasAct_I32(const void* x, const void* bias, void* y, int64_t outer,
                      int64_t channels, int64_t inner, int act,
                      cudaStream_t stream);
int LaunchBiasAct_I64(const void* x, const void* bias, void* y, int64_t outer,
                      int64_t channels, int64_t inner, int act,
                      cudaStream_t stream);

/* ------------------------------------- backward of the BiasAdd + Relu chain */

/* Bytes of scratch that LaunchBiasAddGrad_* and LaunchBiasAddReluGrad_* need
 * for this geometry and element size (2, 4 or 8): the partial rows of the
 * two-level column sum.  The op allocates it as a temporary, in the place of
 * the reference's muDNN MemoryMaintainer callback
 * (musa_ext/kernels/nn/musa_biasadd_grad_op.cc:87-98).  0 for a geometry that
 * needs none or is invalid. */
size_t BiasGradWorkspaceBytes(int64_t outer, int64_t channels, int64_t inner,
                              int elem_bytes);

/* BiasAddGrad: bias_grad[c] = sum of out_backprop[outer, c, inner] over outer
 * and inner, in a fixed order; bias_grad has the tensor's type.  Floating
 * types add in fp32 / fp64 and round once, integer types wrap.  An empty
 * outer or inner axis zero-fills bias_grad
 * (musa_ext/kernels/nn/musa_biasadd_grad_op.cc:65-70); channels == 0 does
 * nothing.  Replaces the muDNN Reduce ADD
 * (musa_ext/kernels/nn/musa_biasadd_grad_op.cc:72-104), registered for the
 * same six types (:113-118). */
int LaunchBiasAddGrad_F32(const void* out_backprop, void* bias_grad,
                          int64_t outer, int64_t channels, int64_t inner,
                          void* workspace, size_t workspace_bytes,
                          cudaStream_t stream);
int LaunchBiasAddGrad_F16(const void* out_backprop, void* bias_grad,
                          int64_t outer, int64_t channels, int64_t inner,
                          void* workspace, size_t workspace_bytes,
                          cudaStream_t stream);
int LaunchBiasAddGrad_BF16(const void* out_backprop, void* bias_grad,
                           int64_t outer, int64_t channels, int64_t inner,
                           void* workspace, size_t workspace_bytes,
                           cudaStream_t stream);
int LaunchBiasAddGrad_F64(const void* out_backprop, void* bias_grad,
                          int64_t outer, int64_t channels, int64_t inner,
                          void* workspace, size_t workspace_bytes,
                          cudaStream_t stream);
int LaunchBiasAddGrad_I32(const void* out_backprop, void* bias_grad,
                          int64_t outer, int64_t channels, int64_t inner,
                          void* workspace, size_t workspace_bytes,
                          cudaStream_t stream);
int LaunchBiasAddGrad_I64(const void* out_backprop, void* bias_grad,
                          int64_t outer, int64_t channels, int64_t inner,
                          void* workspace, size_t workspace_bytes,
                          cudaStream_t stream);

/* ReluGrad: backprops[i] = gradients[i] * (features[i] > 0) over n elements.
 * Replaces the muDNN Binary LEAKY_RELU_BW pass
 * (musa_ext/kernels/nn/musa_relu_grad_op.cc:36-43), registered for float,
 * half and bfloat16 (:56-58). */
int LaunchReluGrad_F32(const void* gradients, const void* features,
                       void* backprops, int64_t n, cudaStream_t stream);
int LaunchReluGrad_F16(const void* gradients, const void* features,
                       void* backprops, int64_t n, cudaStream_t stream);
int LaunchReluGrad_BF16(const void* gradients, const void* features,
                        void* backprops, int64_t n, cudaStream_t stream);

/* BiasAddGrad(ReluGrad(gradients, features)) in one pass: backprops as
 * LaunchReluGrad_* stores it and bias_grad = the column sum of those values
 * before they are rounded to the tensor's type.  The reference runs the two
 * ops above back to back (5 tensor passes); this reads gradients and features
 * once and writes backprops once (3 passes).  No counterpart symbol in the
 * reference. */
int LaunchBiasAddReluGrad_F32(const void* gradients, const void* features,
                              void* backprops, void* bias_grad, int64_t outer,
                              int64_t channels, int64_t inner, void* workspace,
                              size_t workspace_bytes, cudaStream_t stream);
int LaunchBiasAddReluGrad_F16(const void* gradients, const void* features,
                              void* backprops, void* bias_grad, int64_t outer,
                              int64_t channels, int64_t inner, void* workspace,
                              size_t workspace_bytes, cudaStream_t stream);
int LaunchBiasAddReluGrad_BF16(const void* gradients, const void* features,
                               void* backprops, void* bias_grad, int64_t outer,
                               int64_t channels, int64_t inner, void* workspace,
                               size_t workspace_bytes, cudaStream_t stream);

/* --------------------------------------------- LayerNorm and RMSNorm rows -- */

/* MusaLayerNorm over [rows, row_size] (the op normalises the last axis):
 *   y = (x - mean) * rsqrt(var + epsilon) * gamma + beta, population variance,
 * statistics in fp32.  `mean` / `inv_std` are optional fp32 [rows] outputs
 * (NULL: not stored).  One read of x, one write of y.  Replaces the muDNN
 * LayerNorm call and its MemoryMaintainer
 * (musa_ext/kernels/fusion/musa_layernorm_op.cc:61-98), registered for float,
 * half and bfloat16 (:106-116). */
int LaunchLayerNorm_F32(const void* x, const void* gamma, const void* beta, void* y,
                        float* mean, float* inv_std, int64_t rows, int64_t row_size,
                        float epsilon, cudaStream_t stream);
int LaunchLayerNorm_F16(const void* x, const void* gamma, const void* beta, void* y,
                        float* mean, float* inv_std, int64_t rows, int64_t row_size,
                        float epsilon, cudaStream_t stream);
int LaunchLayerNorm_BF16(const void* x, const void* gamma, const void* beta, void* y,
                         float* mean, float* inv_std, int64_t rows, int64_t row_size,
                         float epsilon, cudaStream_t stream);

/* Scratch of LaunchLayerNormGrad_*: the partial rows of the dgamma / dbeta
 * column sums. */
size_t LayerNormGradWorkspaceBytes(int64_t rows, int64_t row_size);

/* MusaLayerNormGrad: with x_hat = (x - mean) * inv_std and g = dy * gamma,
 *   dx = inv_std * (g - mean_row(g) - x_hat * mean_row(g * x_hat)),
 *   dgamma = sum_rows dy * x_hat,  dbeta = sum_rows dy   (type T, fixed order).
 * The row statistics are recomputed from x (the op has no saved statistics).
 * One read of dy and x, one write of dx.  rows == 0 zero-fills dgamma / dbeta.
 * Replaces the muDNN LayerNorm backward of
 * musa_ext/kernels/fusion/musa_layernorm_grad_op.cc. */
int LaunchLayerNormGrad_F32(const void* dy, const void* x, const void* gamma, void* dx,
                            void* dgamma, void* dbeta, int64_t rows, int64_t row_size,
                            float epsilon, void* workspace, size_t workspace_bytes,
                            cudaStream_t stream);
int LaunchLayerNormGrad_F16(const void* dy, const void* x, const void* gamma, void* dx,
                            void* dgamma, void* dbeta, int64_t rows, int64_t row_size,
                            float epsilon, void* workspace, size_t workspace_bytes,
                            cudaStream_t stream);
int LaunchLayerNormGrad_BF16(const void* dy, const void* x, const void* gamma, void* dx,
                             void* dgamma, void* dbeta, int64_t rows, int64_t row_size,
                             float epsilon, void* workspace, size_t workspace_bytes,
                             cudaStream_t stream);

/* MusaRmsNorm: inv_rms[row] = rsqrt(mean(x^2) + epsilon); normalized = x *
 * inv_rms; y = normalized * gamma.  Names and arguments of the reference
 * (musa_ext/kernels/nn/musa_rmsnorm_kernel.mu:357-428; declared for the op at
 * musa_ext/kernels/nn/musa_rmsnorm_op.cc:8-19); bfloat16 pointers are passed
 * as void*.  bfloat16 results round to nearest even (the reference truncates). */
void LaunchRmsNormFloat(const float* x, const float* gamma, float* y, float* normalized,
                        float* inv_rms, int64_t num_rows, int64_t row_size,
                        float epsilon, cudaStream_t stream);
void LaunchRmsNormBFloat16(const void* x, const void* gamma, void* y, void* normalized,
                           void* inv_rms, int64_t num_rows, int64_t row_size,
                           float epsilon, cudaStream_t stream);
/* MusaRmsNormGradDx: dx = dy * gamma * inv_rms - x * (sum_row(x * dy * gamma) *
 * inv_rms^3 / row_size) (musa_ext/kernels/nn/musa_rmsnorm_kernel.mu:381-451). */
void LaunchRmsNormGradDxFloat(const float* x, const float* inv_rms, const float* gamma,
                              const float* dy, float* dx, int64_t num_rows,
                              int64_t row_size, cudaStream_t stream);
void LaunchRmsNormGradDxBFloat16(const void* x, const void* inv_rms, const void* gamma,
                                 const void* dy, void* dx, int64_t num_rows,
                                 int64_t row_size, cudaStream_t stream);

/* ------------------------------------------------------ FusedBatchNorm -- */

/* Tensor geometry: x, y, dy, dx are [outer, channels, inner], the statistics
 * run over outer*inner values per channel.  NHWC: outer = N*H*W, inner = 1.
 * NCHW: outer = N, inner = H*W.  scale/offset/mean/variance are fp32
 * [channels] for every x dtype. */

/* Bytes of scratch that the BatchNorm launchers below need for this geometry
 * (the per-CTA partial sums of the two-level reduction).  The same figure
 * serves forward and gradient.  16-byte
 * aligned memory is expected; its contents may be arbitrary. */
size_t BnWorkspaceBytes(int64_t outer, int64_t channels, int64_t inner);

/* Training-mode forward.  Outputs follow TensorFlow's CPU kernel:
 *   y = (x - mean) * rsqrt(var + eps) * scale + offset, mean/var of the batch;
 *   batch_mean = mean, batch_var = var * R/(R-1) (Bessel; R = outer*inner, not
 *   applied when R == 1), blended with est_mean/est_var by exp_avg_factor when
 *   that is not 1 (est_* may be NULL when it is 1);
 *   saved_mean = mean, saved_var = population variance.
 * y may be x itself (in place); any other overlap of y with x is not allowed.
 * Replaces muDNN BatchNorm::RunComposite plus the copies and the Bessel
 * fix-up after it (musa_ext/kernels/nn/musa_fused_batchnorm_op.cc:106-171). */
int LaunchBnFwdTrain_F32(const void* x, const float* scale, const float* offset,
                         const float* est_mean, const float* est_var, void* y,
                         float* batch_mean, float* batch_var, float* saved_mean,
                         float* saved_var, int64_t outer, int64_t channels,
                         int64_t inner, float epsilon, float exp_avg_factor,
                         void* workspace, size_t workspace_bytes,
                         cudaStream_t stream);
int LaunchBnFwdTrain_F16(const void* x, const float* scale, const float* offset,
                         const float* est_mean, const float* est_var, void* y,
                         float* batch_mean, float* batch_var, float* saved_mean,
                         float* saved_var, int64_t outer, int64_t channels,
                         int64_t inner, float epsilon, float exp_avg_factor,
                         void* workspace, size_t workspace_bytes,
                         cudaStream_t stream);
int LaunchBnFwdTrain_BF16(const void* x, const float* scale,
                          const float* offset, const float* est_mean,
                          const float* est_var, void* y, float* batch_mean,
                          float* batch_var, float* saved_mean, float* saved_var,
                          int64_t outer, int64_t channels, int64_t inner,
                          float epsilon, float exp_avg_factor, void* workspace,
                          size_t workspace_bytes, cudaStream_t stream);

/* Inference-mode forward: y from the given mean/variance, one pass.
 * Replaces muDNN BatchNorm::RunPure
 * (musa_ext/kernels/nn/musa_fused_batchnorm_op.cc:172-178). */
int LaunchBnFwdInfer_F32(const void* x, const float* scale, const float* offset,
                         const float* est_mean, const float* est_var, void* y,
                         int64_t outer, int64_t channels, int64_t inner,
                         float epsilon, cudaStream_t stream);
int LaunchBnFwdInfer_F16(const void* x, const float* scale, const float* offset,
                         const float* est_mean, const float* est_var, void* y,
                         int64_t outer, int64_t channels, int64_t inner,
                         float epsilon, cudaStream_t stream);
int LaunchBnFwdInfer_BF16(const void* x, const float* scale,
                          const float* offset, const float* est_mean,
                          const float* est_var, void* y, int64_t outer,
                          int64_t channels, int64_t inner, float epsilon,
                          cudaStream_t stream);

/* Gradient.  `mean` and `variance` are reserve_space_1/2 of the forward op:
 * the batch mean and the POPULATION variance (not an inverse std-dev).
 *   doffset = sum(dy); dscale = sum(dy * (x - mean)) * rsqrt(var + eps);
 *   training : dx = scale*inv * (dy - doffset/R - (x-mean)*inv*dscale/R)
 *   inference: dx = dy * scale * inv.
 * Every output element is written, so stale output memory cannot leak.
 * Replaces LaunchVarianceToInvStd plus muDNN BatchNorm::RunBwd and the memsets
 * before them (musa_ext/kernels/nn/musa_fused_batchnorm_op.cc:233-291). */
int LaunchBnGrad_F32(const void* dy, const void* x, const float* scale,
                     const float* mean, const float* variance, void* dx,
                     float* dscale, float* doffset, int64_t outer,
                     int64_t channels, int64_t inner, float epsilon,
                     bool is_training, void* workspace, size_t workspace_bytes,
                     cudaStream_t stream);
int LaunchBnGrad_F16(const void* dy, const void* x, const float* scale,
                     const float* mean, const float* variance, void* dx,
                     float* dscale, float* doffset, int64_t outer,
                     int64_t channels, int64_t inner, float epsilon,
                     bool is_training, void* workspace, size_t workspace_bytes,
                     cudaStream_t stream);
int LaunchBnGrad_BF16(const void* dy, const void* x, const float* scale,
                      const float* mean, const float* variance, void* dx,
                      float* dscale, float* doffset, int64_t outer,
                      int64_t channels, int64_t inner, float epsilon,
                      bool is_training, void* workspace, size_t workspace_bytes,
                      cudaStream_t stream);

/* Training-mode forward for callers that may not allocate device memory.
 * No counterpart in the reference.
 *
 * Who needs it: code that runs where cudaMalloc is off limits - inside a
 * serving or training loop that forbids allocation after start-up because
 * cudaMalloc synchronises the whole device, inside a host callback or a
 * library hook that has no framework allocator (no OpKernelContext to ask for
 * a temporary) at hand, or in a process whose memory budget was handed out in
 * full at start.  Such a caller cannot supply the workspace that
 * LaunchBnFwdTrain_* asks for, so this entry point brings its own: a 4 MiB +
 * 64 KiB array that is part of the library image on every GPU that loads it.
 * It calls no cudaMalloc / cudaFree and no allocating library routine.
 *
 * Same arguments and results as LaunchBnFwdTrain_{F32,F16,BF16} (dtype:
 * MUSA_DT_*), minus the workspace.  Limits: channels <= BnNoAllocMaxChannels()
 * (8192); beyond that, or if the geometry would need more scratch than the
 * array holds, it returns MUSA_KERNELS_ETOOLARGE and launches nothing.
 *
 * The first call on each device looks up the array's device address (with
 * that device current); make that first call outside any stream capture.
 * All calls share the one array per device: it keeps whatever the last call
 * left there (nothing in it has to start at zero - every word that is read was
 * written earlier in the same call), and two calls whose kernels can overlap
 * on the GPU - different streams, or the same stream from two threads without
 * ordering - race on it.  Issue them on one stream, or order them with events. */
size_t BnNoAllocMaxChannels(void);
int LaunchBnFwdTrainNoAlloc(int dtype, const void* x, const float* scale,
                            const float* offset, const float* est_mean,
                            const float* est_var, void* y, float* batch_mean,
                            float* batch_var, float* saved_mean,
                            float* saved_var, int64_t outer, int64_t channels,
                            int64_t inner, float epsilon, float exp_avg_factor,
                            cudaStream_t stream);

/* The two BatchNorm fix-up launchers of the reference, kept for callers that
 * still hold muDNN-convention statistics: data[i] *= factor, and
 * inv_std[i] = rsqrt(variance[i] + epsilon).  Replace LaunchBesselCorrection
 * and LaunchVarianceToInvStd
 * (musa_ext/kernels/nn/musa_fused_batchnorm_kernel.mu:38-56). */
void LaunchBesselCorrection(float* data, float factor, int count,
                            cudaStream_t stream);
void LaunchVarianceToInvStd(const float* variance, float* inv_std,
                            float epsilon, int count, cudaStream_t stream);

/* ---- Cross-replica (SyncBN) halves: the same kernels, split where the
 * all-reduce of the per-channel sums goes.  `dtype`: 0 fp32, 1 fp16, 2 bf16.
 * The reference has no collective backend
 * (musa_ext/mu/collective/musa_collective_runtime.cc:58-63 returns
 * Unimplemented); these are what a cross-replica BatchNorm built on the same
 * op pair calls either side of an NCCL all-reduce. */
#define MUSA_DT_F32 0
#define MUSA_DT_F16 1
#define MUSA_DT_BF16 2

/* sums[0:C] = sum(x), sums[C:2C] = sum(x*x) over this replica's rows. */
int LaunchBnStatsSums(int dtype, const void* x, float* sums, int64_t outer,
                      int64_t channels, int64_t inner, void* workspace,
                      size_t workspace_bytes, cudaStream_t stream);
/* Same, and sums[2C] = the local row count, so that replicas with different
 * batch sizes learn the global count from the same all-reduce (sums holds
 * 2C + 1 floats). */
int LaunchBnStatsSumsCount(int dtype, const void* x, float* sums, int64_t outer,
                           int64_t channels, int64_t inner, void* workspace,
                           size_t workspace_bytes, cudaStream_t stream);
/* The cancellation-safe form of the same exchange: moments[0:C] = mean,
 * moments[C:2C] = sum((x - mean)^2), moments[2C] = the row count, all of this
 * replica's rows (2C + 1 floats).  Raw sums lose the variance when
 * |mean| >> std (sum(x*x) and mean^2 agree in all fp32 digits); moments of
 * replicas are merged, not added: LaunchExchangeMoments over peer memory, or
 * an all-gather followed by LaunchBnMergeMoments. */
int LaunchBnStatsMoments(int dtype, const void* x, float* moments, int64_t outer,
                         int64_t channels, int64_t inner, void* workspace,
                         size_t workspace_bytes, cudaStream_t stream);
/* gathered = `world` moment vectors of 2C + 1 floats back to back, in rank
 * order; merged (2C + 1 floats) = the moments of all rows together, in fp64
 * and rank order (every replica computes the same bits). */
int LaunchBnMergeMoments(const float* gathered, int world, int64_t channels,
                         float* merged, cudaStream_t stream);
/* LaunchBnApplyFromSums for merged moments (mean and sum of squared
 * deviations over `total_count` values per channel). */
int LaunchBnApplyFromMoments(int dtype, const void* x, const float* scale,
                             const float* offset, const float* moments,
                             double total_count, const float* est_mean,
                             const float* est_var, float exp_avg_factor, void* y,
                             float* batch_mean, float* batch_var,
                             float* saved_mean, float* saved_var, int64_t outer,
                             int64_t channels, int64_t inner, float epsilon,
                             cudaStream_t stream);
/* From all-reduced sums over `total_count` values per channel to the four
 * statistic outputs of the forward op. */
int LaunchBnFinalizeFromSums(const float* sums, double total_count,
                             const float* est_mean, const float* est_var,
                             float* batch_mean, float* batch_var,
                             float* saved_mean, float* saved_var,
                             int64_t channels, float exp_avg_factor,
                             cudaStream_t stream);
/* y = (x - mean) * rsqrt(var + eps) * scale + offset (same as inference). */
int LaunchBnApply(int dtype, const void* x, const float* scale,
                  const float* offset, const float* mean, const float* variance,
                  void* y, int64_t outer, int64_t channels, int64_t inner,
                  float epsilon, cudaStream_t stream);
/* LaunchBnFinalizeFromSums and LaunchBnApply as one launch: the element-wise
 * kernel derives mean and variance from the all-reduced sums in its prologue
 * and writes the four statistic outputs itself.  `x` must be the tensor whose
 * statistics the LaunchBnStats* call before it on `stream` took, unchanged
 * since: the kernel requests its first rows of x while it still waits for the
 * kernel that delivers `sums` (the same holds for LaunchBnApplyFromMoments,
 * and for dy and x of LaunchBnGradApplyFromSums after
 * LaunchBnGradStatsSums*). */
int LaunchBnApplyFromSums(int dtype, const void* x, const float* scale,
                          const float* offset, const float* sums,
                          double total_count, const float* est_mean,
                          const float* est_var, float exp_avg_factor, void* y,
                          float* batch_mean, float* batch_var,
                          float* saved_mean, float* saved_var, int64_t outer,
                          int64_t channels, int64_t inner, float epsilon,
                          cudaStream_t stream);
/* sums[0:C] = sum(dy), sums[C:2C] = sum(dy * (x - mean)) over local rows. */
int LaunchBnGradStatsSums(int dtype, const void* dy, const void* x,
                          const float* mean, float* sums, int64_t outer,
                          int64_t channels, int64_t inner, void* workspace,
                          size_t workspace_bytes, cudaStream_t stream);
/* dx, dscale, doffset from all-reduced sums over `total_count` values. */
int LaunchBnGradApplyFromSums(int dtype, const void* dy, const void* x,
                              const float* scale, const float* mean,
                              const float* variance, const float* sums,
                              double total_count, void* dx, float* dscale,
                              float* doffset, int64_t outer, int64_t channels,
                              int64_t inner, float epsilon,
                              cudaStream_t stream);

/* ---- Peer-memory exchange of the cross-replica sums (one process per GPU on
 * one NVLink-connected node).  Replaces the NCCL all-reduce between
 * LaunchBnStatsSumsCount and LaunchBnApplyFromSums (and between the two
 * gradient halves) by ONE single-CTA kernel per replica that pushes its vector
 * into every replica's memory with peer stores, waits (bounded) for the others'
 * vectors to land in its own memory and sums them in rank order, so all
 * replicas get bit-identical totals.  No counterpart in the reference.
 *
 * Set-up (allocates; not for the hot path): MusaExchangeCreate on every rank
 * with the device current, exchange the 64-byte handles of
 * MusaExchangeIpcHandle between the processes, MusaExchangeOpenPeers.
 * Per exchange: LaunchExchangeSums(handle, vector, n, stream) - in place, no
 * host synchronisation, works inside CUDA graph capture (the epoch counter
 * lives on the device).  MusaExchangeStatus (synchronises; call between steps)
 * returns 1 + q if a wait for replica q ever ran out (after about a second),
 * which leaves that exchange's totals incomplete instead of hanging the GPU;
 * until the host has read the status, later exchanges do not wait for that
 * replica again. */
void* MusaExchangeCreate(int rank, int world, int64_t max_floats);
int MusaExchangeIpcHandle(void* handle, void* out64);
int MusaExchangeOpenPeers(void* handle, const void* handles);
int LaunchExchangeSums(void* handle, float* vector, int64_t n, cudaStream_t stream);
/* The same exchange with the merge of LaunchBnMergeMoments as its combine
 * step: `moments` (2 * channels + 1 floats, see LaunchBnStatsMoments) becomes
 * the moments of the rows of all replicas, bit-identical everywhere. */
int LaunchExchangeMoments(void* handle, float* moments, int64_t channels,
                          cudaStream_t stream);
int MusaExchangeStatus(void* handle);
/* LaunchBnStatsMoments + LaunchExchangeMoments, and LaunchBnGradStatsSums +
 * LaunchExchangeSums, without the exchange kernel: the finalize kernel of the
 * statistics pass pushes the values of its own channels to the replicas, waits
 * (bounded, same status word) for theirs and writes the result over ALL
 * replicas into `moments` (2C + 1 floats) / `sums` (2C floats).  One kernel and
 * two kernel boundaries less in every cross-replica BatchNorm pass.  Every
 * replica must call with the same `channels`, in the same order as its other
 * exchanges on `exchange`. */
int LaunchBnStatsMomentsExchange(int dtype, const void* x, float* moments, int64_t outer,
                                 int64_t channels, int64_t inner, void* workspace,
                                 size_t workspace_bytes, void* exchange,
                                 cudaStream_t stream);
int LaunchBnGradStatsSumsExchange(int dtype, const void* dy, const void* x,
                                  const float* mean, float* sums, int64_t outer,
                                  int64_t channels, int64_t inner, void* workspace,
                                  size_t workspace_bytes, void* exchange,
                                  cudaStream_t stream);
void MusaExchangeDestroy(void* handle);
/* Peer-visible device memory for the set-up of the two peer-memory paths: a
 * cudaMalloc block, its 64-byte CUDA IPC handle, and the mapping of another
 * process's handle (all ranks on one node).  Set-up time only. */
void* MusaPeerAlloc(int64_t bytes);
int MusaPeerFree(void* ptr);
int MusaPeerIpcHandle(void* ptr, void* out64);
void* MusaPeerOpen(const void* handle64);
int MusaPeerClose(void* mapped);
/* One cudaMemcpyAsync (device to device, local or peer-mapped addresses). */
int MusaPeerCopyAsync(void* dst, const void* src, int64_t bytes, cudaStream_t stream);

/* Range-sharded ResourceApplyAdam (fp32) fused with the all-gather of the
 * updated weights: updates var[lo, lo + n) from this replica's m, v (n
 * elements each) and grad (the n elements of its range) and stores every new
 * value into [lo, lo + n) of ALL `world` replicas' var (`var_replicas[q]`:
 * base of replica q's copy as mapped in this process; entry `rank` is the
 * local one), over NVLink peer stores.  The update arithmetic is
 * LaunchResourceApplyAdamFloat's.  The peers may read their var only after
 * they have learnt that this launch completed (an exchange of one float with
 * LaunchExchangeSums after it does that).  128-bit path when lo % 4 == 0 and
 * all pointers are 16-byte aligned.  No counterpart in the reference. */
int LaunchAdamShardBroadcastFloat(float* const* var_replicas, int world, int rank,
                                  int64_t lo, float* m, float* v, const float* grad,
                                  float beta1, float beta2, float epsilon, float alpha,
                                  int64_t n, cudaStream_t stream);

/* The same step with the gradient in fp32, fp16 or bf16 beside fp32 state:
 * the range-sharded form of MusaResourceApplyAdamMixed
 * (musa_ext/kernels/training/musa_applyadam_mixed_op.cc:125-258; arithmetic
 * and use_nesterov as LaunchApplyAdamMixed_*).  `grad_dtype`: MUSA_DT_F32,
 * MUSA_DT_F16 or MUSA_DT_BF16 (else MUSA_KERNELS_EUNSUPPORTED).  128-bit path
 * when lo % 4 == 0, the state pointers are 16-byte aligned and grad is aligned
 * to four of its elements.  No counterpart in the reference. */
int LaunchAdamShardBroadcastMixed(int grad_dtype, float* const* var_replicas, int world,
                                  int rank, int64_t lo, float* m, float* v, const void* grad,
                                  float beta1, float beta2, float epsilon, float alpha,
                                  int64_t n, bool use_nesterov, cudaStream_t stream);

/* The same step over an NVSwitch multicast mapping of the replicas' copies
 * (`var_multicast`: the multicast address of the vector's base, e.g. from
 * torch.distributed._symmetric_memory; `var_local`: this replica's own copy):
 * one multimem.st per 128-bit pack writes the new weights into every replica,
 * so the shard leaves the GPU once instead of world - 1 times and the step is
 * bound by HBM again.  Needs lo % 4 == 0 and 16-byte aligned pointers
 * (MUSA_KERNELS_EINVAL otherwise).  Same results and completion rule as
 * LaunchAdamShardBroadcastFloat.  No counterpart in the reference. */
int LaunchAdamShardMulticastFloat(float* var_local, float* var_multicast, int64_t lo,
                                  float* m, float* v, const float* grad, float beta1,
                                  float beta2, float epsilon, float alpha, int64_t n,
                                  cudaStream_t stream);

/* The same step with the copy engines as the all-gather, for four replicas
 * and more, where the step is bound by the bytes that leave the GPU over
 * NVLink and copy engines move them faster than SM stores: the local range is
 * updated in `chunks` (1..8) pieces with LaunchResourceApplyAdamFloat's kernel
 * on `stream`, and every finished piece goes to each peer with one
 * cudaMemcpyAsync on a side stream of the pipe while the next piece updates;
 * `stream` joins the side streams before the call returns, so the call is one
 * asynchronous operation on `stream` (capturable in a CUDA graph).  Same
 * results, bit for bit, and the same completion rule as
 * LaunchAdamShardBroadcastFloat.  MusaShardPipeCreate (set-up: world - 1
 * streams and the events) with the device current.  No counterpart in the
 * reference. */
void* MusaShardPipeCreate(int world, int rank);
void MusaShardPipeDestroy(void* pipe);
int LaunchAdamShardCopyFloat(void* pipe, float* const* var_replicas, int64_t lo, float* m,
                             float* v, const float* grad, float beta1, float beta2,
                             float epsilon, float alpha, int64_t n, int chunks,
                             cudaStream_t stream);

/* Test hook: `world` (<= 8) replicas emulated on one GPU by one cooperative
 * launch of `world` CTAs; `vectors` is a device array of `world` device
 * pointers to n floats each.  missing_rank = world - 1 leaves that replica out
 * to check that the others' waits run out (returns 1000 + world). */
int MusaExchangeSelfTest(int world, int64_t n, float* const* vectors, int rounds,
                         int missing_rank, int mode, cudaStream_t stream);
/* `mode`: 0 sums, 1 moments (n = 2 * channels + 1). */

/* ---- Tracing of the launcher layer (off by default).  With
 * MUSA_B200_TRACE=1 in the environment, or after MusaKernelsTraceEnable(1),
 * every launcher call sits inside an NVTX range named after the launcher (a
 * profiler that injects NVTX shows them; without one the range calls are
 * no-ops) and adds to per-launcher counters: calls, algorithmic bytes (the
 * bytes the op has to move, as in the roofline figures), host nanoseconds
 * spent inside the call and the kernel launches it made.  The reference traces its allocator and copy paths
 * only (musa_ext/mu/device/musa_telemetry.h:47-199); no counterpart there. */
typedef struct MusaLaunchCounter {
  const char* name;   /* launcher family, a static string */
  long long calls;
  long long bytes;
  long long host_ns;
  long long kernels;  /* kernel launches made inside the calls */
} MusaLaunchCounter;
/* Returns the previous state (0 / 1). */
int MusaKernelsTraceEnable(int on);
/* Copies up to max_entries counters; returns how many (out == NULL: how many
 * exist). */
int MusaKernelsTraceSnapshot(MusaLaunchCounter* out, int max_entries);
void MusaKernelsTraceReset(void);
/* Kernel launches this library has made since it was loaded (counted whether
 * tracing is on or not: one relaxed add per launch); the difference around a
 * region is the number of this library's kernels launched in it. */
long long MusaKernelsLaunchCount(void);

/* Test and sweep hooks, not part of the reference boundary: launch-shape
 * knobs (grid sizes, pipeline depths, cache hints; csrc/tuning.h lists the
 * keys) that let a sweep compare variants without rebuilding.  They change
 * HOW a launcher runs, never what it computes.  The table is process-wide and
 * is read by every launcher at every call: set a knob only while no other
 * thread is launching.  Set returns the previous value (-1: unknown key). */
int MusaKernelsSetTuning(int key, int value);
int MusaKernelsGetTuning(int key);

#ifdef __cplusplus
} /* extern "C" */
#endif

#endif /* MUSA_PLUGIN_KERNELS_H_ */
