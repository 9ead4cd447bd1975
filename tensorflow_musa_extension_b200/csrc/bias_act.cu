// BiasAdd + activation chains as one read of x and one write of y.
//
// y = act(x + bias[channel]) with act in {identity, relu, swish, sigmoid};
// `swish` is the three-op chain Mul(x, Sigmoid(BiasAdd(x, b))).  The tensor is
// viewed as [outer, channels, inner]; channels-last inputs (inner == 1) take a
// 128-bit path where the bias pack comes from L1, everything else a pack path
// with one bias value per pack or an element-wise path.
//
// Semantics follow the un-fused ops the chain replaces: BiasAdd
// (musa_ext/kernels/nn/musa_biasadd_op.cc:23-61), Relu
// (musa_ext/kernels/nn/musa_relu_op.cc:19-57), Sigmoid
// (musa_ext/kernels/nn/musa_sigmoid_op.cc:18-35).
#include "common.cuh"
#include "trace.h"
#include "tuning.h"
#include "../../include/musa_plugin_kernels.h"

namespace musa_b200 {
namespace {

// fp32 keeps libm-grade exp and an IEEE divide (rtol 1e-5 against the CPU op,
// inputs up to +-100); the 16-bit types round to 8 or 11 mantissa bits on
// store, so the hardware exp2/rcp approximations (1e-6 relative) are exact
// after rounding for all practical purposes and halve the instruction count.
template <bool kFast>
__device__ __forceinline__ float Sigmoid(float t) {
  if constexpr (kFast) {
    return __fdividef(1.0f, 1.0f + __expf(-t));
  } else {
    return 1.0f / (1.0f + expf(-t));
  }
}

template <int kAct, bool kFast>
__device__ __forceinline__ float Activate(float x, float b) {
  const float t = x + b;
  if constexpr (kAct == MUSA_ACT_IDENTITY) {
    return t;
  } else if constexpr (kAct == MUSA_ACT_RELU) {
    // max(t, 0) that lets NaN through, as the CPU op does.
    return t < 0.0f ? 0.0f : t;
  } else if constexpr (kAct == MUSA_ACT_SWISH) {
    return x * Sigmoid<kFast>(t);
  } else {
    return Sigmoid<kFast>(t);
  }
}

// 16-bit element pairs.  BiasAdd is a packed half-precision add: IEEE-rounded,
// so it returns exactly what the un-fused BiasAdd op stores (a float add of two
// 16-bit values followed by one rounding gives the same bits).  Relu is a packed
// max.  The sigmoid runs in fp32 as 1 / (1 + 2^(-t * log2 e)) on the exp2 and
// reciprocal units (relative error ~1e-6 over the whole range, including the
// far negative side where a tanh form would cancel).
__device__ __forceinline__ float2 Widen2(__half2 v) { return __half22float2(v); }
__device__ __forceinline__ float2 Widen2(__nv_bfloat162 v) {
  return __bfloat1622float2(v);
}
__device__ __forceinline__ void Narrow2(float a, float b, __half2& out) {
  out = __floats2half2_rn(a, b);
}
__device__ __forceinline__ void Narrow2(float a, float b, __nv_bfloat162& out) {
  out = __floats2bfloat162_rn(a, b);
}

template <typename T2, int kAct, bool kHasBias>
__device__ __forceinline__ T2 ActivatePair(T2 x, T2 b) {
  const T2 t = kHasBias ? __hadd2(x, b) : x;
  if constexpr (kAct == MUSA_ACT_IDENTITY) {
    return t;
  } else if constexpr (kAct == MUSA_ACT_RELU) {
    const float2 z = make_float2(0.0f, 0.0f);
    T2 zero;
    Narrow2(z.x, z.y, zero);
    return __hmax2(t, zero);
  } else {
    const float2 tf = Widen2(t);
    const float s0 = Sigmoid<true>(tf.x);
    const float s1 = Sigmoid<true>(tf.y);
    // The sigmoid is rounded to T and the product taken in T, which is what
    // the separate Sigmoid and Mul ops of the un-fused chain store.
    T2 out;
    Narrow2(s0, s1, out);
    if constexpr (kAct == MUSA_ACT_SWISH) out = __hmul2(x, out);
    return out;
  }
}

template <typename T>
struct PairOf {
  using type = void;
};
template <>
struct PairOf<__half> {
  using type = __half2;
};
template <>
struct PairOf<__nv_bfloat16> {
  using type = __nv_bfloat162;
};

// One pack of x and the matching pack of bias values -> one pack of y.
template <typename T, int kEpt, int kAct, bool kHasBias>
__device__ __forceinline__ Pack<T, kEpt> ActivatePack(const Pack<T, kEpt>& px,
                                                      const Pack<T, kEpt>& pb) {
  constexpr bool kFast = sizeof(T) == 2;
  Pack<T, kEpt> out;
  if constexpr (sizeof(T) == 2 && kEpt % 2 == 0) {
    using T2 = typename PairOf<T>::type;
    const T2* x2 = reinterpret_cast<const T2*>(&px);
    const T2* b2 = reinterpret_cast<const T2*>(&pb);
    T2* o2 = reinterpret_cast<T2*>(&out);
#pragma unroll
    for (int e = 0; e < kEpt / 2; ++e) {
      o2[e] = ActivatePair<T2, kAct, kHasBias>(x2[e], b2[e]);
    }
  } else {
#pragma unroll
    for (int e = 0; e < kEpt; ++e) {
      const float b = kHasBias ? ToF32(pb.v[e]) : 0.0f;
      out.v[e] = FromF32<T>(Activate<kAct, kFast>(ToF32(px.v[e]), b));
    }
  }
  return out;
}

// Channels-last pack kernel.  Pack p of the flat tensor covers channels
// [(p % cv) * kEpt, +kEpt); the column is tracked incrementally, no division
// in the loop.
template <typename T, int kEpt, int kUnroll, int kAct, bool kHasBias>
__global__ void __launch_bounds__(256)
    BiasActLastKernel(const T* __restrict__ x, const T* __restrict__ bias,
                      T* __restrict__ y, int64_t n_packs, int cv) {
  using P = Pack<T, kEpt>;
  constexpr bool kFast = sizeof(T) == 2;
  const P* xp = reinterpret_cast<const P*>(x);
  const P* bp = reinterpret_cast<const P*>(bias);
  P* yp = reinterpret_cast<P*>(y);
  const int64_t tile = static_cast<int64_t>(blockDim.x) * kUnroll;
  const int64_t n_tiles = (n_packs + tile - 1) / tile;
  const int step = static_cast<int>(blockDim.x % cv);

  // When the block width is a multiple of the row width in packs, a thread
  // meets the same bias pack in every pack it handles: fetch it once.
  const bool fixed_col = kHasBias && step == 0;
  P fixed_bias;
  if (fixed_col) fixed_bias = LoadKeep(bp + (threadIdx.x % cv));

  for (int64_t t = blockIdx.x; t < n_tiles; t += gridDim.x) {
    const int64_t base = t * tile + threadIdx.x;
    int col = fixed_col ? 0 : static_cast<int>(base % cv);
    P px[kUnroll];
    P pb[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const int64_t i = base + static_cast<int64_t>(u) * blockDim.x;
      if (i < n_packs) {
        px[u] = LoadStream(xp + i);
        if constexpr (kHasBias) {
          if (fixed_col) {
            pb[u] = fixed_bias;
          } else {
            pb[u] = LoadKeep(bp + col);
          }
        }
      }
      if (!fixed_col) {
        col += step;
        if (col >= cv) col -= cv;
      }
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const int64_t i = base + static_cast<int64_t>(u) * blockDim.x;
      if (i < n_packs) {
        StoreStream(yp + i, ActivatePack<T, kEpt, kAct, kHasBias>(px[u], pb[u]));
      }
    }
  }
}

// Channels-last with a row of packs that divides the CTA width (channel counts
// of 8 .. 2048 in fp16 / bf16 that are powers of two, and the like): with a grid
// stride that is a multiple of the CTA width a thread meets the same bias pack
// in every pack it handles.  It is fetched once, and the loop is nothing but
// four loads, the math and four stores around two pointer bumps - the index
// bookkeeping of the general kernel costs as many issue slots as a sigmoid.
template <typename T, int kEpt, int kAct>
__global__ void __launch_bounds__(256)
    BiasActFixedKernel(const T* __restrict__ x, const T* __restrict__ bias,
                       T* __restrict__ y, int64_t n_packs, int cv) {
  using P = Pack<T, kEpt>;
  const P pb = LoadKeep(reinterpret_cast<const P*>(bias) + (threadIdx.x % cv));
  // A tile is 4 * 256 consecutive packs (16 KB): the four loads of a warp stay
  // inside one DRAM neighbourhood.
  const int64_t n_tiles = (n_packs + 1023) / 1024;
  for (int64_t t = blockIdx.x; t < n_tiles; t += gridDim.x) {
    const int64_t base = t * 1024 + threadIdx.x;
    const P* xp = reinterpret_cast<const P*>(x) + base;
    P* yp = reinterpret_cast<P*>(y) + base;
    if (base + 768 < n_packs) {
      const P a0 = LoadStream(xp);
      const P a1 = LoadStream(xp + 256);
      const P a2 = LoadStream(xp + 512);
      const P a3 = LoadStream(xp + 768);
      StoreStream(yp, ActivatePack<T, kEpt, kAct, true>(a0, pb));
      StoreStream(yp + 256, ActivatePack<T, kEpt, kAct, true>(a1, pb));
      StoreStream(yp + 512, ActivatePack<T, kEpt, kAct, true>(a2, pb));
      StoreStream(yp + 768, ActivatePack<T, kEpt, kAct, true>(a3, pb));
    } else {
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        if (base + u * 256 < n_packs) {
          StoreStream(yp + u * 256,
                      ActivatePack<T, kEpt, kAct, true>(LoadStream(xp + u * 256), pb));
        }
      }
    }
  }
}

// General layout: [outer, channels, inner] with packs of kEpt elements that
// never straddle a channel (inner % kEpt == 0), or kEpt == 1.
template <typename T, int kEpt, int kAct, bool kHasBias>
__global__ void __launch_bounds__(256)
    BiasActInnerKernel(const T* __restrict__ x, const T* __restrict__ bias,
                       T* __restrict__ y, int64_t n_packs, int64_t inner_packs,
                       int64_t channels) {
  using P = Pack<T, kEpt>;
  constexpr bool kFast = sizeof(T) == 2;
  const P* xp = reinterpret_cast<const P*>(x);
  P* yp = reinterpret_cast<P*>(y);
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
       i < n_packs; i += stride) {
    const P px = LoadStream(xp + i);
    float b = 0.0f;
    if constexpr (kHasBias) b = ToF32(bias[(i / inner_packs) % channels]);
    P out;
#pragma unroll
    for (int e = 0; e < kEpt; ++e) {
      out.v[e] = FromF32<T>(Activate<kAct, kFast>(ToF32(px.v[e]), b));
    }
    StoreStream(yp + i, out);
  }
}

// Channel-major layouts ([outer, channels, inner], inner >= the pack width):
// the tensor is read as one flat run of 128-bit packs, whatever the plane
// length.  A pack starts `r` elements into a plane of channel `c` and crosses
// into the next plane at most once, so its bias values are bias[c] up to the
// crossing and bias[c + 1] after it.  Every thread tracks (r, c) of its packs
// incrementally: no division in the loop.
template <typename T, int kEpt, int kAct>
__global__ void __launch_bounds__(256)
    BiasActFlatKernel(const T* __restrict__ x, const T* __restrict__ bias,
                      T* __restrict__ y, int64_t n, int64_t inner,
                      int64_t channels) {
  using P = Pack<T, kEpt>;
  constexpr int kUnroll = 4;
  const int64_t n_packs = n / kEpt;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  // Position of pack i, and how it moves when i grows by `stride`.
  const int64_t e0 = i * kEpt;
  int64_t r = e0 % inner;
  int64_t c = (e0 / inner) % channels;
  const int64_t step = stride * kEpt;
  const int64_t dr = step % inner;
  const int64_t dc = (step / inner) % channels;
  const P* xp = reinterpret_cast<const P*>(x);
  P* yp = reinterpret_cast<P*>(y);
  while (i < n_packs) {
    P px[kUnroll];
    P pb[kUnroll];
    int64_t at[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      at[u] = i < n_packs ? i : -1;
      if (at[u] >= 0) {
        px[u] = LoadStream(xp + i);
        const T b0 = bias[c];
        const T b1 = bias[c + 1 == channels ? 0 : c + 1];
        const int64_t before = inner - r;  // elements of this pack in plane c
#pragma unroll
        for (int e = 0; e < kEpt; ++e) pb[u].v[e] = e < before ? b0 : b1;
      }
      i += stride;
      r += dr;
      c += dc;
      if (r >= inner) {
        r -= inner;
        ++c;
      }
      if (c >= channels) c -= channels;
      if (c >= channels) c -= channels;
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      if (at[u] >= 0) {
        StoreStream(yp + at[u], ActivatePack<T, kEpt, kAct, true>(px[u], pb[u]));
      }
    }
  }
  // Elements past the last whole pack.
  if (blockIdx.x == 0 && threadIdx.x < kEpt) {
    const int64_t t = n_packs * kEpt + threadIdx.x;
    if (t < n) {
      const float b = ToF32(bias[(t / inner) % channels]);
      y[t] = FromF32<T>(Activate<kAct, sizeof(T) == 2>(ToF32(x[t]), b));
    }
  }
}

// Exact-arithmetic kernel for the remaining BiasAdd dtypes (double, int32,
// int64): the add is done in T.
template <typename T, bool kRelu>
__global__ void __launch_bounds__(256)
    BiasAddExactKernel(const T* __restrict__ x, const T* __restrict__ bias,
                       T* __restrict__ y, int64_t n, int64_t inner,
                       int64_t channels) {
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
       i < n; i += stride) {
    T t = x[i];
    if (bias != nullptr) t = t + bias[(i / inner) % channels];
    if (kRelu) t = t < T(0) ? T(0) : t;
    y[i] = t;
  }
}

int GridFor(int64_t work_items, int per_sm_cap) {
  int64_t blocks = work_items < 1 ? 1 : work_items;
  const int64_t cap = static_cast<int64_t>(SmCount()) * per_sm_cap;
  if (per_sm_cap > 0 && blocks > cap) blocks = cap;
  if (blocks > 0x7fffffffLL) blocks = 0x7fffffffLL;
  return static_cast<int>(blocks);
}

template <typename T, int kAct, bool kHasBias>
int LaunchTyped(const T* x, const T* bias, T* y, int64_t outer,
                int64_t channels, int64_t inner, cudaStream_t stream) {
  constexpr int kVec = VecWidth<T>::value;
  const int64_t n = outer * channels * inner;
  const bool aligned = Aligned16(x) && Aligned16(y);
  if (!kHasBias && aligned && n >= kVec) {
    // Activation alone: the tensor is one flat run of packs plus a tail.
    const int64_t n_packs = n / kVec;
    const int grid =
        GridFor(CeilDiv(n_packs, 256 * 4), GetTuning(kTuneBiasActCtasPerSm));
    BiasActLastKernel<T, kVec, 4, kAct, false>
        <<<grid, 256, 0, stream>>>(x, bias, y, n_packs, 1);
    CountKernelLaunch();
    const int64_t done = n_packs * kVec;
    if (done < n) {
      BiasActInnerKernel<T, 1, kAct, false><<<1, 256, 0, stream>>>(
          x + done, bias, y + done, n - done, 1, 1);
      CountKernelLaunch();
    }
    return static_cast<int>(cudaGetLastError());
  }
  if (inner == 1 && channels % kVec == 0 && aligned &&
      (!kHasBias || Aligned16(bias)) && channels / kVec <= 0x7fffffff) {
    const int64_t n_packs = n / kVec;
    const int cv = static_cast<int>(channels / kVec);
    const int per_sm = GetTuning(kTuneBiasActCtasPerSm);
    const int unroll = GetTuning(kTuneBiasActUnroll);
    if constexpr (kHasBias) {
      if (256 % cv == 0 && unroll != 2 && unroll != 8) {
        const int grid = GridFor(CeilDiv(n_packs, 1024), per_sm);
        BiasActFixedKernel<T, kVec, kAct>
            <<<grid, 256, 0, stream>>>(x, bias, y, n_packs, cv);
        CountKernelLaunch();
        return static_cast<int>(cudaGetLastError());
      }
    }
    if (unroll == 2) {
      const int grid = GridFor(CeilDiv(n_packs, 256 * 2), per_sm);
      BiasActLastKernel<T, kVec, 2, kAct, kHasBias>
          <<<grid, 256, 0, stream>>>(x, bias, y, n_packs, cv);
      CountKernelLaunch();
    } else if (unroll == 8) {
      const int grid = GridFor(CeilDiv(n_packs, 256 * 8), per_sm);
      BiasActLastKernel<T, kVec, 8, kAct, kHasBias>
          <<<grid, 256, 0, stream>>>(x, bias, y, n_packs, cv);
      CountKernelLaunch();
    } else {
      const int grid = GridFor(CeilDiv(n_packs, 256 * 4), per_sm);
      BiasActLastKernel<T, kVec, 4, kAct, kHasBias>
          <<<grid, 256, 0, stream>>>(x, bias, y, n_packs, cv);
      CountKernelLaunch();
    }
  } else if (inner % kVec == 0 && aligned) {
    // Planes of whole packs: one bias value per pack.
    const int64_t n_packs = n / kVec;
    const int grid = GridFor(CeilDiv(n_packs, 256), 16);
    BiasActInnerKernel<T, kVec, kAct, kHasBias><<<grid, 256, 0, stream>>>(
        x, bias, y, n_packs, inner / kVec, channels);
    CountKernelLaunch();
  } else if (kHasBias && aligned && inner >= kVec && n >= kVec) {
    // Any other plane length (14x14, 7x7, ...): flat packs that may cross into
    // the next plane once.
    const int64_t n_packs = n / kVec;
    const int grid = GridFor(CeilDiv(n_packs, 256 * 4), 8);
    if constexpr (kHasBias) {
      BiasActFlatKernel<T, kVec, kAct><<<grid, 256, 0, stream>>>(x, bias, y, n, inner,
                                                               channels);
      CountKernelLaunch();
    }
  } else {
    const int grid = GridFor(CeilDiv(n, 256), 16);
    BiasActInnerKernel<T, 1, kAct, kHasBias>
        <<<grid, 256, 0, stream>>>(x, bias, y, n, inner, channels);
    CountKernelLaunch();
  }
  return static_cast<int>(cudaGetLastError());
}

template <typename T>
int LaunchBiasAct(const void* x, const void* bias, void* y, int64_t outer,
                  int64_t channels, int64_t inner, int act,
                  cudaStream_t stream) {
  if (outer < 0 || channels < 0 || inner < 0) return MUSA_KERNELS_EINVAL;
  MUSA_TRACE("LaunchBiasAct", 2 * sizeof(T) * outer * channels * inner);
  if (outer == 0 || channels == 0 || inner == 0) return MUSA_KERNELS_OK;
  if (x == nullptr || y == nullptr) return MUSA_KERNELS_EINVAL;
  const T* xt = static_cast<const T*>(x);
  const T* bt = static_cast<const T*>(bias);
  T* yt = static_cast<T*>(y);
#define MUSA_DISPATCH_ACT(ACT)                                               \
  case ACT:                                                                  \
    return bias != nullptr                                                   \
               ? LaunchTyped<T, ACT, true>(xt, bt, yt, outer, channels,      \
                                           inner, stream)                    \
               : LaunchTyped<T, ACT, false>(xt, bt, yt, outer, channels,     \
                                            inner, stream);
  switch (act) {
    MUSA_DISPATCH_ACT(MUSA_ACT_IDENTITY)
    MUSA_DISPATCH_ACT(MUSA_ACT_RELU)
    MUSA_DISPATCH_ACT(MUSA_ACT_SWISH)
    MUSA_DISPATCH_ACT(MUSA_ACT_SIGMOID)
    default:
      return MUSA_KERNELS_EUNSUPPORTED;
  }
#undef MUSA_DISPATCH_ACT
}

template <typename T>
int LaunchBiasAddExact(const void* x, const void* bias, void* y, int64_t outer,
                       int64_t channels, int64_t inner, int act,
                       cudaStream_t stream) {
  if (outer < 0 || channels < 0 || inner < 0) return MUSA_KERNELS_EINVAL;
  if (outer == 0 || channels == 0 || inner == 0) return MUSA_KERNELS_OK;
  if (x == nullptr || y == nullptr) return MUSA_KERNELS_EINVAL;
  if (act != MUSA_ACT_IDENTITY && act != MUSA_ACT_RELU) {
    return MUSA_KERNELS_EUNSUPPORTED;
  }
  const int64_t n = outer * channels * inner;
  const int grid = GridFor(CeilDiv(n, 256), 16);
  if (act == MUSA_ACT_RELU) {
    BiasAddExactKernel<T, true><<<grid, 256, 0, stream>>>(
        static_cast<const T*>(x), static_cast<const T*>(bias),
        static_cast<T*>(y), n, inner, channels);
    CountKernelLaunch();
  } else {
    BiasAddExactKernel<T, false><<<grid, 256, 0, stream>>>(
        static_cast<const T*>(x), static_cast<const T*>(bias),
        static_cast<T*>(y), n, inner, channels);
    CountKernelLaunch();
  }
  return static_cast<int>(cudaGetLastError());
}

}  // namespace
}  // namespace musa_b200

using namespace musa_b200;

extern "C" {

int LaunchBiasAct_F32(const void* x, const void* bias, void* y, int64_t outer,
                      int64_t channels, int64_t inner, int act,
                      cudaStream_t stream) {
  return LaunchBiasAct<float>(x, bias, y, outer, channels, inner, act, stream);
}
int LaunchBiasAct_F16(const void* x, const void* bias, void* y, int64_t outer,
                      int64_t channels, int64_t inner, int act,
                      cudaStream_t stream) {
  return LaunchBiasAct<__half>(x, bias, y, outer, channels, inner, act, stream);
}
int LaunchBiasAct_BF16(const void* x, const void* bias, void* y, int64_t outer,
                       int64_t channels, int64_t inner, int act,
                       cudaStream_t stream) {
  return LaunchBiasAct<__nv_bfloat16>(x, bias, y, outer, channels, inner, act,
                                      stream);
}
int LaunchBiasAct_F64(const void* x, const void* bias, void* y, int64_t outer,
                      int64_t channels, int64_t inner, int act,
                      cudaStream_t stream) {
  return LaunchBiasAddExact<double>(x, bias, y, outer, channels, inner, act,
                                    stream);
}
int LaunchBiasAct_I32(const void* x, const void* bias, void* y, int64_t outer,
                      int64_t channels, int64_t inner, int act,
                      cudaStream_t stream) {
  return LaunchBiasAddExact<int32_t>(x, bias, y, outer, channels, inner, act,
                                     stream);
}
int LaunchBiasAct_I64(const void* x, const void* bias, void* y, int64_t outer,
                      int64_t channels, int64_t inner, int act,
                      cudaStream_t stream) {
  return LaunchBiasAddExact<int64_t>(x, bias, y, outer, channels, inner, act,
                                     stream);
}

}  // extern "C"
