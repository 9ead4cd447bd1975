// The streaming optimizer updates that share Adam's shape: every one is a
// single pass that reads a few state vectors and the gradient and writes the
// state back with 128-bit accesses.  One kernel template, one rule per
// optimizer:
//
//   Nadam            musa_ext/kernels/training/musa_resource_apply_nadam_kernel.mu:48-81
//   RMSProp          musa_ext/kernels/training/musa_applyrmsprop_kernel.mu:72-99
//   centered RMSProp musa_ext/kernels/training/musa_applyrmsprop_kernel.mu:101-133
//   gradient descent musa_ext/kernels/training/musa_applygradientdescent_kernel.mu:14-96
//   Adagrad (V2)     musa_ext/kernels/training/musa_applyadagrad_kernel.mu:55-79
//   Adam, double     the op chain of musa_ext/kernels/training/musa_applyadam_op.cc:297-415
//
// Arithmetic: fp32 for float / half / bfloat16 tensors with one round-to-
// nearest-even on store, fp64 for double tensors.  Every rounding is spelled
// out so that the vector path, the element path and a range-sharded run give
// the same bits.
#include "common.cuh"
#include "trace.h"
#include "tuning.h"
#include "../../include/musa_plugin_kernels.h"

namespace musa_b200 {
namespace {

constexpr int kThreads = 256;

// ---- IEEE round-to-nearest operations in fp32 and fp64 --------------------
__device__ __forceinline__ float Mul(float a, float b) { return __fmul_rn(a, b); }
__device__ __forceinline__ float Add(float a, float b) { return __fadd_rn(a, b); }
__device__ __forceinline__ float Sub(float a, float b) { return __fsub_rn(a, b); }
__device__ __forceinline__ float Div(float a, float b) { return __fdiv_rn(a, b); }
__device__ __forceinline__ float Sqrt(float a) { return __fsqrt_rn(a); }
__device__ __forceinline__ float Fma(float a, float b, float c) { return fmaf(a, b, c); }
__device__ __forceinline__ double Mul(double a, double b) { return __dmul_rn(a, b); }
__device__ __forceinline__ double Add(double a, double b) { return __dadd_rn(a, b); }
__device__ __forceinline__ double Sub(double a, double b) { return __dsub_rn(a, b); }
__device__ __forceinline__ double Div(double a, double b) { return __ddiv_rn(a, b); }
__device__ __forceinline__ double Sqrt(double a) { return __dsqrt_rn(a); }
__device__ __forceinline__ double Fma(double a, double b, double c) { return fma(a, b, c); }

template <typename C, typename T>
__device__ __forceinline__ C Load(T v) {
  if constexpr (sizeof(T) == 2) {
    return static_cast<C>(ToF32(v));
  } else {
    return static_cast<C>(v);
  }
}
template <typename T, typename C>
__device__ __forceinline__ T Store(C v) {
  if constexpr (sizeof(T) == 2) {
    return FromF32<T>(static_cast<float>(v));
  } else {
    return static_cast<T>(v);
  }
}

template <typename T>
struct ComputeOf {
  using type = float;
};
template <>
struct ComputeOf<double> {
  using type = double;
};

// ---- Rules: kStates state vectors (state[0] is the variable), one gradient,
// Step() maps the old state and the gradient to the new state.

template <typename T>
struct NadamRule {
  using StateT = T;
  using GradT = T;
  using C = typename ComputeOf<T>::type;
  static constexpr int kStates = 3;  // var, m, v
  struct Params {
    C lr, beta1, one_minus_b1, beta2, one_minus_b2, epsilon;
    C one_minus_b1_power, one_minus_b2_power;
  };
  static __device__ __forceinline__ void Step(C (&s)[kStates], C g,
                                              const Params& p) {
    const C m = Fma(p.beta1, s[1], Mul(p.one_minus_b1, g));
    const C v = Fma(p.beta2, s[2], Mul(Mul(p.one_minus_b2, g), g));
    const C m_hat =
        Div(Fma(p.beta1, m, Mul(p.one_minus_b1, g)), p.one_minus_b1_power);
    const C v_hat = Div(v, p.one_minus_b2_power);
    s[0] = Sub(s[0], Div(Mul(p.lr, m_hat), Add(Sqrt(v_hat), p.epsilon)));
    s[1] = m;
    s[2] = v;
  }
};

template <typename T>
struct RmsPropRule {
  using StateT = T;
  using GradT = T;
  using C = typename ComputeOf<T>::type;
  static constexpr int kStates = 3;  // var, ms, mom
  struct Params {
    C lr, rho, one_minus_rho, momentum, epsilon;
  };
  static __device__ __forceinline__ void Step(C (&s)[kStates], C g,
                                              const Params& p) {
    const C ms = Fma(p.rho, s[1], Mul(Mul(p.one_minus_rho, g), g));
    const C mom =
        Fma(p.momentum, s[2], Div(Mul(p.lr, g), Sqrt(Add(ms, p.epsilon))));
    s[0] = Sub(s[0], mom);
    s[1] = ms;
    s[2] = mom;
  }
};

template <typename T>
struct CenteredRmsPropRule {
  using StateT = T;
  using GradT = T;
  using C = typename ComputeOf<T>::type;
  static constexpr int kStates = 4;  // var, mg, ms, mom
  using Params = typename RmsPropRule<T>::Params;
  static __device__ __forceinline__ void Step(C (&s)[kStates], C g,
                                              const Params& p) {
    const C mg = Fma(p.rho, s[1], Mul(p.one_minus_rho, g));
    const C ms = Fma(p.rho, s[2], Mul(Mul(p.one_minus_rho, g), g));
    const C denom = Add(Sub(ms, Mul(mg, mg)), p.epsilon);
    const C mom = Fma(p.momentum, s[3], Div(Mul(p.lr, g), Sqrt(denom)));
    s[0] = Sub(s[0], mom);
    s[1] = mg;
    s[2] = ms;
    s[3] = mom;
  }
};

// Adam for double tensors.  The reference serves this dtype with a chain of
// thirteen element-wise library calls, every one of which stores a double
// tensor (musa_applyadam_op.cc:297-415): multiply, multiply, add for each
// moment, then sqrt, add epsilon, divide, multiply by alpha, subtract.  This
// rule performs the same operations in the same order with one IEEE rounding
// each (no contraction into fused multiply-adds), in one pass.
template <bool kNesterov>
struct AdamChainRule {
  using StateT = double;
  using GradT = double;
  using C = double;
  static constexpr int kStates = 3;  // var, m, v
  struct Params {
    double alpha, beta1, one_minus_b1, beta2, one_minus_b2, epsilon;
  };
  static __device__ __forceinline__ void Step(C (&s)[kStates], C g,
                                              const Params& p) {
    const C m = Add(Mul(s[1], p.beta1), Mul(g, p.one_minus_b1));
    const C v = Add(Mul(s[2], p.beta2), Mul(Mul(g, g), p.one_minus_b2));
    // The chain has no Nesterov branch; with the attribute set the numerator
    // is TensorFlow's m * beta1 + g * (1 - beta1), built the same way.
    const C numer = kNesterov ? Add(Mul(m, p.beta1), Mul(g, p.one_minus_b1)) : m;
    s[0] = Sub(s[0], Mul(Div(numer, Add(Sqrt(v), p.epsilon)), p.alpha));
    s[1] = m;
    s[2] = v;
  }
};

// accum += g*g (with update_slots); var -= lr * g / (sqrt(accum) + epsilon).
template <typename T, bool kUpdateSlots>
struct AdagradRule {
  using StateT = T;
  using GradT = T;
  using C = typename ComputeOf<T>::type;
  static constexpr int kStates = 2;  // var, accum
  struct Params {
    C lr, epsilon;
  };
  static __device__ __forceinline__ void Step(C (&s)[kStates], C g,
                                              const Params& p) {
    // Without update_slots the accumulator is read but stays as it is (it is
    // stored back unchanged).
    const C accum = kUpdateSlots ? Fma(g, g, s[1]) : s[1];
    s[0] = Sub(s[0], Div(Mul(p.lr, g), Add(Sqrt(accum), p.epsilon)));
    s[1] = accum;
  }
};

// var -= alpha * delta.  A 16-bit variable rounds the product to the
// tensor's type before the subtraction, as the two ops of the un-fused form
// (multiply, subtract) each store a tensor of that type.
template <typename VarT, typename DeltaT>
struct SgdRule {
  using StateT = VarT;
  using GradT = DeltaT;
  using C = float;
  static constexpr int kStates = 1;
  struct Params {
    float alpha;
  };
  static __device__ __forceinline__ void Step(C (&s)[kStates], C g,
                                              const Params& p) {
    float step = Mul(p.alpha, g);
    if constexpr (sizeof(VarT) == 2) step = ToF32(FromF32<VarT>(step));
    s[0] = Sub(s[0], step);
  }
};

template <typename Rule>
struct UpdateArgs {
  typename Rule::StateT* state[Rule::kStates];
  const typename Rule::GradT* grad;
  typename Rule::Params p;
};

template <typename Rule>
__device__ __forceinline__ void UpdateElement(const UpdateArgs<Rule>& a,
                                              int64_t i) {
  using C = typename Rule::C;
  C s[Rule::kStates];
#pragma unroll
  for (int k = 0; k < Rule::kStates; ++k) s[k] = Load<C>(a.state[k][i]);
  Rule::Step(s, Load<C>(a.grad[i]), a.p);
#pragma unroll
  for (int k = 0; k < Rule::kStates; ++k) {
    a.state[k][i] = Store<typename Rule::StateT>(s[k]);
  }
}

// A tile is blockDim.x * kUnroll consecutive packs of kEpt elements; all loads
// of a tile are issued before the first use.
template <typename Rule, int kEpt, int kUnroll>
__device__ __forceinline__ void UpdateTile(const UpdateArgs<Rule>& a,
                                           int64_t base, int64_t n_packs) {
  using ST = typename Rule::StateT;
  using GT = typename Rule::GradT;
  using C = typename Rule::C;
  constexpr int kS = Rule::kStates;
  using SPack = Pack<ST, kEpt>;
  using GPack = Pack<GT, kEpt>;
  SPack ps[kUnroll][kS];
  GPack pg[kUnroll];
#pragma unroll
  for (int u = 0; u < kUnroll; ++u) {
    const int64_t i = base + static_cast<int64_t>(u) * kThreads;
    if (i < n_packs) {
      pg[u] = LoadStream(reinterpret_cast<const GPack*>(a.grad) + i);
#pragma unroll
      for (int k = kS - 1; k >= 0; --k) {
        ps[u][k] = LoadStream(reinterpret_cast<const SPack*>(a.state[k]) + i);
      }
    }
  }
#pragma unroll
  for (int u = 0; u < kUnroll; ++u) {
    const int64_t i = base + static_cast<int64_t>(u) * kThreads;
    if (i < n_packs) {
#pragma unroll
      for (int e = 0; e < kEpt; ++e) {
        C s[kS];
#pragma unroll
        for (int k = 0; k < kS; ++k) s[k] = Load<C>(ps[u][k].v[e]);
        Rule::Step(s, Load<C>(pg[u].v[e]), a.p);
#pragma unroll
        for (int k = 0; k < kS; ++k) ps[u][k].v[e] = Store<ST>(s[k]);
      }
#pragma unroll
      for (int k = kS - 1; k >= 0; --k) {
        StoreStream(reinterpret_cast<SPack*>(a.state[k]) + i, ps[u][k]);
      }
    }
  }
}

template <typename Rule, int kEpt, int kUnroll>
__global__ void __launch_bounds__(kThreads)
    StreamUpdateKernel(UpdateArgs<Rule> a, int64_t n) {
  const int64_t n_packs = n / kEpt;
  const int64_t tile = static_cast<int64_t>(kThreads) * kUnroll;
  const int64_t n_tiles = (n_packs + tile - 1) / tile;
  for (int64_t t = blockIdx.x; t < n_tiles; t += gridDim.x) {
    UpdateTile<Rule, kEpt, kUnroll>(a, t * tile + threadIdx.x, n_packs);
  }
  // Ragged tail (n not a multiple of the pack width): one thread per element.
  if (kEpt > 1 && blockIdx.x == 0) {
    const int64_t i = n_packs * kEpt + threadIdx.x;
    if (threadIdx.x < kEpt && i < n) UpdateElement<Rule>(a, i);
  }
}

template <typename Rule, int kEpt, int kUnroll>
void LaunchStream(const UpdateArgs<Rule>& a, int64_t n, cudaStream_t stream) {
  const int64_t tile = static_cast<int64_t>(kThreads) * kUnroll;
  int64_t blocks = CeilDiv(n / kEpt, tile);
  if (blocks < 1) blocks = 1;
  if (blocks > 0x7fffffffLL) blocks = 0x7fffffffLL;
  StreamUpdateKernel<Rule, kEpt, kUnroll>
      <<<static_cast<unsigned>(blocks), kThreads, 0, stream>>>(a, n);
  CountKernelLaunch();
}

// 128-bit state packs when every pointer allows it (the gradient pack has the
// same element count), element accesses otherwise.
template <typename Rule>
void LaunchUpdate(const UpdateArgs<Rule>& a, int64_t n, cudaStream_t stream) {
  MUSA_TRACE("LaunchStreamUpdate",
             n > 0 ? (2 * Rule::kStates * sizeof(typename Rule::StateT) +
                      sizeof(typename Rule::GradT)) * n
                   : 0);
  if (n <= 0) return;
  constexpr int kEpt = VecWidth<typename Rule::StateT>::value;
  constexpr size_t kGradPackBytes = sizeof(typename Rule::GradT) * kEpt;
  bool vec_ok = (reinterpret_cast<uintptr_t>(a.grad) % kGradPackBytes) == 0;
  for (int k = 0; k < Rule::kStates; ++k) vec_ok = vec_ok && Aligned16(a.state[k]);
  if (vec_ok) {
    LaunchStream<Rule, kEpt, 2>(a, n, stream);
  } else {
    LaunchStream<Rule, 1, 4>(a, n, stream);
  }
}

template <typename T>
void Nadam(void* var, void* m, void* v, const void* grad, float beta1_power,
           float beta2_power, float lr, float beta1, float beta2, float epsilon,
           int64_t n, cudaStream_t stream) {
  using Rule = NadamRule<T>;
  using C = typename Rule::C;
  UpdateArgs<Rule> a;
  a.state[0] = static_cast<T*>(var);
  a.state[1] = static_cast<T*>(m);
  a.state[2] = static_cast<T*>(v);
  a.grad = static_cast<const T*>(grad);
  // The reference takes every scalar as float and forms 1 - x in float
  // (musa_resource_apply_nadam_kernel.mu:52-54, :64-72).
  a.p.lr = static_cast<C>(lr);
  a.p.beta1 = static_cast<C>(beta1);
  a.p.one_minus_b1 = static_cast<C>(1.0f - beta1);
  a.p.beta2 = static_cast<C>(beta2);
  a.p.one_minus_b2 = static_cast<C>(1.0f - beta2);
  a.p.epsilon = static_cast<C>(epsilon);
  a.p.one_minus_b1_power = static_cast<C>(1.0f - beta1_power);
  a.p.one_minus_b2_power = static_cast<C>(1.0f - beta2_power);
  LaunchUpdate<Rule>(a, n, stream);
}

template <typename T>
typename RmsPropRule<T>::Params RmsParams(double lr, double rho, double momentum,
                                          double epsilon) {
  using C = typename ComputeOf<T>::type;
  // Scalars arrive as double and are narrowed to the compute type first;
  // 1 - rho is formed in that type (musa_applyrmsprop_kernel.mu:84-88).
  typename RmsPropRule<T>::Params p;
  p.lr = static_cast<C>(lr);
  p.rho = static_cast<C>(rho);
  p.one_minus_rho = static_cast<C>(1.0) - p.rho;
  p.momentum = static_cast<C>(momentum);
  p.epsilon = static_cast<C>(epsilon);
  return p;
}

template <typename T>
void RmsProp(void* var, void* ms, void* mom, const void* grad, double lr,
             double rho, double momentum, double epsilon, int64_t n,
             cudaStream_t stream) {
  using Rule = RmsPropRule<T>;
  UpdateArgs<Rule> a;
  a.state[0] = static_cast<T*>(var);
  a.state[1] = static_cast<T*>(ms);
  a.state[2] = static_cast<T*>(mom);
  a.grad = static_cast<const T*>(grad);
  a.p = RmsParams<T>(lr, rho, momentum, epsilon);
  LaunchUpdate<Rule>(a, n, stream);
}

template <typename T>
void CenteredRmsProp(void* var, void* mg, void* ms, void* mom, const void* grad,
                     double lr, double rho, double momentum, double epsilon,
                     int64_t n, cudaStream_t stream) {
  using Rule = CenteredRmsPropRule<T>;
  UpdateArgs<Rule> a;
  a.state[0] = static_cast<T*>(var);
  a.state[1] = static_cast<T*>(mg);
  a.state[2] = static_cast<T*>(ms);
  a.state[3] = static_cast<T*>(mom);
  a.grad = static_cast<const T*>(grad);
  a.p = RmsParams<T>(lr, rho, momentum, epsilon);
  LaunchUpdate<Rule>(a, n, stream);
}

template <typename T>
void Adagrad(void* var, void* accum, const void* grad, double lr, double epsilon,
             bool update_slots, int64_t n, cudaStream_t stream) {
  using C = typename ComputeOf<T>::type;
  auto run = [&](auto rule) {
    using Rule = decltype(rule);
    UpdateArgs<Rule> a;
    a.state[0] = static_cast<T*>(var);
    a.state[1] = static_cast<T*>(accum);
    a.grad = static_cast<const T*>(grad);
    a.p.lr = static_cast<C>(lr);
    a.p.epsilon = static_cast<C>(epsilon);
    LaunchUpdate<Rule>(a, n, stream);
  };
  if (update_slots) {
    run(AdagradRule<T, true>());
  } else {
    run(AdagradRule<T, false>());
  }
}

template <typename VarT, typename DeltaT>
void Sgd(void* var, const void* delta, float alpha, int64_t n,
         cudaStream_t stream) {
  using Rule = SgdRule<VarT, DeltaT>;
  UpdateArgs<Rule> a;
  a.state[0] = static_cast<VarT*>(var);
  a.grad = static_cast<const DeltaT*>(delta);
  a.p.alpha = alpha;
  LaunchUpdate<Rule>(a, n, stream);
}

// ---- Grouped gradient descent: many (variable, gradient) pairs, one launch.
//
// Table form (the reference's interface): five device arrays, CTA b belongs to
// the tensor t with block_offsets[t] <= b < block_offsets[t + 1] and strides
// over it with the CTAs of that tensor.
template <typename DeltaT>
__global__ void __launch_bounds__(kThreads)
    GroupedSgdTableKernel(const uint64_t* __restrict__ var_ptrs,
                          const uint64_t* __restrict__ grad_ptrs,
                          const float* __restrict__ alphas,
                          const int64_t* __restrict__ sizes,
                          const int64_t* __restrict__ block_offsets,
                          int num_tensors) {
  using Rule = SgdRule<float, DeltaT>;
  constexpr int kEpt = 4;
  const int64_t block = blockIdx.x;
  int lo = 0, hi = num_tensors;
  while (lo + 1 < hi) {
    const int mid = (lo + hi) / 2;
    if (block_offsets[mid] <= block) {
      lo = mid;
    } else {
      hi = mid;
    }
  }
  const int64_t n = sizes[lo];
  const int64_t local = block - block_offsets[lo];
  const int64_t ctas = block_offsets[lo + 1] - block_offsets[lo];
  UpdateArgs<Rule> a;
  a.state[0] = reinterpret_cast<float*>(var_ptrs[lo]);
  a.grad = reinterpret_cast<const DeltaT*>(grad_ptrs[lo]);
  a.p.alpha = alphas[lo];
  const bool vec_ok = (var_ptrs[lo] % 16) == 0 &&
                      (grad_ptrs[lo] % (sizeof(DeltaT) * kEpt)) == 0;
  if (vec_ok) {
    const int64_t n_packs = n / kEpt;
    for (int64_t i = local * kThreads + threadIdx.x; i < n_packs;
         i += ctas * kThreads) {
      UpdateTile<Rule, kEpt, 1>(a, i, n_packs);
    }
    const int64_t tail = n_packs * kEpt + threadIdx.x;
    if (local == 0 && threadIdx.x < kEpt && tail < n) UpdateElement<Rule>(a, tail);
  } else {
    for (int64_t i = local * kThreads + threadIdx.x; i < n; i += ctas * kThreads) {
      UpdateElement<Rule>(a, i);
    }
  }
}

// Parameter form: the descriptors travel in the kernel's parameter space, so
// the launch needs no device tables, no staging copies and no temporaries.
constexpr int kGroupMax = MUSA_SGD_GROUP_MAX;
struct SgdGroup {
  float* var[kGroupMax];
  const void* delta[kGroupMax];
  int64_t n[kGroupMax];
  float alpha[kGroupMax];
  int tile_begin[kGroupMax + 1];  // first tile of each tensor in the grid
  int count;
};

template <typename DeltaT>
__global__ void __launch_bounds__(kThreads)
    GroupedSgdParamKernel(const __grid_constant__ SgdGroup g) {
  using Rule = SgdRule<float, DeltaT>;
  constexpr int kEpt = 4;
  constexpr int kUnroll = 2;
  const int tile_idx = blockIdx.x;
  int lo = 0, hi = g.count;
  while (lo + 1 < hi) {
    const int mid = (lo + hi) / 2;
    if (g.tile_begin[mid] <= tile_idx) {
      lo = mid;
    } else {
      hi = mid;
    }
  }
  const int64_t n = g.n[lo];
  const int64_t local = tile_idx - g.tile_begin[lo];
  UpdateArgs<Rule> a;
  a.state[0] = g.var[lo];
  a.grad = static_cast<const DeltaT*>(g.delta[lo]);
  a.p.alpha = g.alpha[lo];
  const bool vec_ok =
      (reinterpret_cast<uintptr_t>(a.state[0]) % 16) == 0 &&
      (reinterpret_cast<uintptr_t>(a.grad) % (sizeof(DeltaT) * kEpt)) == 0;
  // A tile covers kThreads * kUnroll * kEpt elements on either path.
  if (vec_ok) {
    const int64_t n_packs = n / kEpt;
    UpdateTile<Rule, kEpt, kUnroll>(
        a, local * (kThreads * kUnroll) + threadIdx.x, n_packs);
    const int64_t tail = n_packs * kEpt + threadIdx.x;
    if (local == 0 && threadIdx.x < kEpt && tail < n) UpdateElement<Rule>(a, tail);
  } else {
    const int64_t begin = local * (kThreads * kUnroll * kEpt);
#pragma unroll
    for (int u = 0; u < kUnroll * kEpt; ++u) {
      const int64_t i = begin + static_cast<int64_t>(u) * kThreads + threadIdx.x;
      if (i < n) UpdateElement<Rule>(a, i);
    }
  }
}

template <typename DeltaT>
int GroupedSgdHost(void* const* var_ptrs, const void* const* delta_ptrs,
                   const float* alphas, const int64_t* sizes, int num_tensors,
                   cudaStream_t stream) {
  if (num_tensors < 0) return MUSA_KERNELS_EINVAL;
  if (num_tensors == 0) return MUSA_KERNELS_OK;
  if (var_ptrs == nullptr || delta_ptrs == nullptr || alphas == nullptr ||
      sizes == nullptr) {
    return MUSA_KERNELS_EINVAL;
  }
  constexpr int64_t kTileElems = static_cast<int64_t>(kThreads) * 2 * 4;
  for (int i = 0; i < num_tensors; ++i) {
    if (sizes[i] < 0) return MUSA_KERNELS_EINVAL;
    if (sizes[i] > 0 && (var_ptrs[i] == nullptr || delta_ptrs[i] == nullptr)) {
      return MUSA_KERNELS_EINVAL;
    }
  }
  int next = 0;
  while (next < num_tensors) {
    SgdGroup g;
    g.count = 0;
    int64_t tiles = 0;
    while (next < num_tensors && g.count < kGroupMax) {
      const int64_t n = sizes[next];
      if (n > 0) {
        const int64_t t = CeilDiv(n, kTileElems);
        if (tiles + t > 0x7fffffffLL) {
          if (g.count == 0) return MUSA_KERNELS_ETOOLARGE;
          break;  // this tensor opens the next launch
        }
        g.var[g.count] = static_cast<float*>(var_ptrs[next]);
        g.delta[g.count] = delta_ptrs[next];
        g.n[g.count] = n;
        g.alpha[g.count] = alphas[next];
        g.tile_begin[g.count] = static_cast<int>(tiles);
        tiles += t;
        ++g.count;
      }
      ++next;
    }
    if (g.count == 0) continue;
    g.tile_begin[g.count] = static_cast<int>(tiles);
    GroupedSgdParamKernel<DeltaT>
        <<<static_cast<unsigned>(tiles), kThreads, 0, stream>>>(g);
    CountKernelLaunch();
    const cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return static_cast<int>(e);
  }
  return MUSA_KERNELS_OK;
}

}  // namespace
}  // namespace musa_b200

using namespace musa_b200;

extern "C" {

#define MUSA_DEFINE_STATEFUL(SUFFIX, TYPE)                                     \
  void LaunchResourceApplyNadam_##SUFFIX(                                      \
      void* var, void* m, void* v, const void* grad, float beta1_power,        \
      float beta2_power, float lr, float beta1, float beta2, float epsilon,    \
      int64_t n, cudaStream_t stream) {                                        \
    Nadam<TYPE>(var, m, v, grad, beta1_power, beta2_power, lr, beta1, beta2,   \
                epsilon, n, stream);                                           \
  }                                                                            \
  void LaunchFusedResourceApplyRMSProp_##SUFFIX(                               \
      void* var, void* ms, void* mom, const void* grad, double lr, double rho, \
      double momentum, double epsilon, int64_t n, cudaStream_t stream) {       \
    RmsProp<TYPE>(var, ms, mom, grad, lr, rho, momentum, epsilon, n, stream);  \
  }                                                                            \
  void LaunchFusedResourceApplyCenteredRMSProp_##SUFFIX(                       \
      void* var, void* mg, void* ms, void* mom, const void* grad, double lr,   \
      double rho, double momentum, double epsilon, int64_t n,                  \
      cudaStream_t stream) {                                                   \
    CenteredRmsProp<TYPE>(var, mg, ms, mom, grad, lr, rho, momentum, epsilon,  \
                          n, stream);                                          \
  }                                                                            \
  void LaunchFusedApplyAdagradV2_##SUFFIX(void* var, void* accum,              \
                                          const void* grad, double lr,         \
                                          double epsilon, bool update_slots,   \
                                          int64_t n, cudaStream_t stream) {    \
    Adagrad<TYPE>(var, accum, grad, lr, epsilon, update_slots, n, stream);     \
  }
MUSA_DEFINE_STATEFUL(Float, float)
MUSA_DEFINE_STATEFUL(Half, __half)
MUSA_DEFINE_STATEFUL(BFloat16, __nv_bfloat16)
MUSA_DEFINE_STATEFUL(Double, double)
#undef MUSA_DEFINE_STATEFUL

void LaunchApplyAdam_F64(double* var, double* m, double* v, const double* grad,
                         double alpha, double beta1, double beta2, double epsilon,
                         int64_t n, bool use_nesterov, cudaStream_t stream) {
  auto run = [&](auto rule) {
    using Rule = decltype(rule);
    UpdateArgs<Rule> a;
    a.state[0] = var;
    a.state[1] = m;
    a.state[2] = v;
    a.grad = grad;
    a.p.alpha = alpha;
    a.p.beta1 = beta1;
    a.p.one_minus_b1 = 1.0 - beta1;
    a.p.beta2 = beta2;
    a.p.one_minus_b2 = 1.0 - beta2;
    a.p.epsilon = epsilon;
    LaunchUpdate<Rule>(a, n, stream);
  };
  if (use_nesterov) {
    run(AdamChainRule<true>());
  } else {
    run(AdamChainRule<false>());
  }
}

void LaunchResourceApplyGradientDescentFloat(float* var, const float* grad,
                                             float alpha, int64_t n,
                                             cudaStream_t stream) {
  Sgd<float, float>(var, grad, alpha, n, stream);
}
void LaunchResourceApplyGradientDescentFloatBFloat16(float* var, const void* grad,
                                                     float alpha, int64_t n,
                                                     cudaStream_t stream) {
  Sgd<float, __nv_bfloat16>(var, grad, alpha, n, stream);
}
void LaunchResourceApplyGradientDescent_Half(void* var, const void* grad,
                                             float alpha, int64_t n,
                                             cudaStream_t stream) {
  Sgd<__half, __half>(var, grad, alpha, n, stream);
}
void LaunchResourceApplyGradientDescent_BFloat16(void* var, const void* grad,
                                                 float alpha, int64_t n,
                                                 cudaStream_t stream) {
  Sgd<__nv_bfloat16, __nv_bfloat16>(var, grad, alpha, n, stream);
}

void LaunchGroupedResourceApplyGradientDescentFloat(
    const uint64_t* var_ptrs, const uint64_t* grad_ptrs, const float* alphas,
    const int64_t* sizes, const int64_t* block_offsets, int num_tensors,
    int total_blocks, cudaStream_t stream) {
  if (num_tensors <= 0 || total_blocks <= 0) return;
  GroupedSgdTableKernel<float><<<total_blocks, kThreads, 0, stream>>>(
      var_ptrs, grad_ptrs, alphas, sizes, block_offsets, num_tensors);
  CountKernelLaunch();
}
void LaunchGroupedResourceApplyGradientDescentFloatBFloat16(
    const uint64_t* var_ptrs, const uint64_t* grad_ptrs, const float* alphas,
    const int64_t* sizes, const int64_t* block_offsets, int num_tensors,
    int total_blocks, cudaStream_t stream) {
  if (num_tensors <= 0 || total_blocks <= 0) return;
  GroupedSgdTableKernel<__nv_bfloat16><<<total_blocks, kThreads, 0, stream>>>(
      var_ptrs, grad_ptrs, alphas, sizes, block_offsets, num_tensors);
  CountKernelLaunch();
}

int LaunchGroupedGradientDescentHostTable(void* const* var_ptrs,
                                          const void* const* delta_ptrs,
                                          const float* alphas,
                                          const int64_t* sizes, int num_tensors,
                                          int delta_is_bfloat16,
                                          cudaStream_t stream) {
  if (delta_is_bfloat16) {
    return GroupedSgdHost<__nv_bfloat16>(var_ptrs, delta_ptrs, alphas, sizes,
                                         num_tensors, stream);
  }
  return GroupedSgdHost<float>(var_ptrs, delta_ptrs, alphas, sizes, num_tensors,
                               stream);
}

}  // extern "C"
