// Backward of the BiasAdd + Relu chain: ReluGrad, BiasAddGrad, and both as one
// pass over the gradient.
//
//   ReluGrad      backprops = gradients * (features > 0)
//                 (musa_ext/kernels/nn/musa_relu_grad_op.cc:19-48)
//   BiasAddGrad   bias_grad[c] = sum of out_backprop over every axis but the
//                 channel axis (musa_ext/kernels/nn/musa_biasadd_grad_op.cc:23-106)
//   fused         backprops as above and bias_grad[c] = sum of backprops, with
//                 one read of gradients and features and one write of
//                 backprops; the un-fused pair reads backprops a second time.
//
// The tensor is viewed as [outer, channels, inner].  The column sum is a
// two-level reduction with a fixed order (no atomics): level 1 leaves one
// partial row per row split in the caller's workspace, level 2 adds the
// partial rows in a wider type and rounds once to the output type.  The two
// kernels are chained with programmatic dependent launch.
#include "common.cuh"
#include "trace.h"
#include "tuning.h"
#include "../../include/musa_plugin_kernels.h"

namespace musa_b200 {
namespace {

constexpr int kThreads = 256;
constexpr int kMaxCtasPerSm = 8;
// Column packs per CTA of the channels-last kernel: one warp reads 512
// contiguous bytes of a row, and a CTA folds 8 rows at a time, which keeps the
// number of partial rows (and with it the second level) small.
constexpr int kColsPerCta = 32;

// Accumulator of level 1 and the wider type of level 2.  Floating types
// accumulate in fp32 (a thread adds a few dozen rows), level 2 in fp64.
// Integer sums wrap like the arithmetic of the tensor's own type.
template <typename T>
struct AccOf {
  using type = float;
  using wide = double;
};
template <>
struct AccOf<double> {
  using type = double;
  using wide = double;
};
template <>
struct AccOf<int32_t> {
  using type = uint32_t;
  using wide = uint32_t;
};
template <>
struct AccOf<int64_t> {
  using type = unsigned long long;
  using wide = unsigned long long;
};

template <typename T>
__device__ __forceinline__ typename AccOf<T>::type Widen(T v) {
  if constexpr (sizeof(T) == 2) {
    return ToF32(v);
  } else {
    return static_cast<typename AccOf<T>::type>(v);
  }
}
template <typename T, typename W>
__device__ __forceinline__ T NarrowTo(W v) {
  if constexpr (sizeof(T) == 2) {
    return FromF32<T>(static_cast<float>(v));
  } else {
    return static_cast<T>(v);
  }
}

// gradients * (features > 0): a multiply by a 0/1 mask, so a non-finite
// gradient at an inactive position gives NaN as the CPU op does.  The product
// is exact in every type (g * 1 or g * 0).
template <typename T>
__device__ __forceinline__ float MaskGrad(T g, T f) {
  return ToF32(g) * (ToF32(f) > 0.0f ? 1.0f : 0.0f);
}

template <typename T>
struct PairOf;
template <>
struct PairOf<__half> {
  using type = __half2;
};
template <>
struct PairOf<__nv_bfloat16> {
  using type = __nv_bfloat162;
};
__device__ __forceinline__ float2 WidenPair(__half2 v) { return __half22float2(v); }
__device__ __forceinline__ float2 WidenPair(__nv_bfloat162 v) {
  const uint32_t w = *reinterpret_cast<const uint32_t*>(&v);
  return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xffff0000u));
}

__device__ __forceinline__ void ZeroPair(__half2& z) { z = __float2half2_rn(0.0f); }
__device__ __forceinline__ void ZeroPair(__nv_bfloat162& z) {
  z = __float2bfloat162_rn(0.0f);
}

// acc += column values of one pack; with kFused the values are the masked
// gradients, which are also returned in `o`.  16-bit packs work on element
// pairs: a packed compare gives the 0/1 mask, a packed multiply applies it and
// one packed fp32 add accumulates both lanes.
template <typename T, int kVec, bool kFused>
__device__ __forceinline__ void Accumulate(const Pack<T, kVec>& a,
                                           const Pack<T, kVec>& f,
                                           Pack<T, kVec>& o,
                                           typename AccOf<T>::type (&acc)[kVec]) {
  if constexpr (sizeof(T) == 2 && kVec % 2 == 0) {
    using T2 = typename PairOf<T>::type;
    const T2* a2 = reinterpret_cast<const T2*>(&a);
    const T2* f2 = reinterpret_cast<const T2*>(&f);
    T2* o2 = reinterpret_cast<T2*>(&o);
    float2* acc2 = reinterpret_cast<float2*>(&acc[0]);
    T2 zero;
    ZeroPair(zero);
#pragma unroll
    for (int i = 0; i < kVec / 2; ++i) {
      T2 z = a2[i];
      if constexpr (kFused) {
        z = __hmul2(z, __hgt2(f2[i], zero));
        o2[i] = z;
      }
      acc2[i] = Add2(acc2[i], WidenPair(z));
    }
  } else {
#pragma unroll
    for (int i = 0; i < kVec; ++i) {
      if constexpr (kFused) {
        const float z = MaskGrad(a.v[i], f.v[i]);
        o.v[i] = NarrowTo<T>(z);
        acc[i] += z;
      } else {
        acc[i] += Widen(a.v[i]);
      }
    }
  }
}

struct LastGeom {
  int64_t rows;
  int64_t rows_per_split;
  int cv;     // packs per row
  int cols;   // packs of one row that a CTA covers
  int lanes;  // rows that a CTA reads at once
};

// Channels-last.  A thread owns one pack of kVec channels and walks the rows
// of its split with kUnroll independent loads in flight.
template <typename T, int kVec, int kUnroll, bool kFused>
__global__ void __launch_bounds__(kThreads)
    BiasGradLastKernel(const T* __restrict__ dy, const T* __restrict__ feat,
                       T* __restrict__ dx,
                       typename AccOf<T>::type* __restrict__ partial,
                       LastGeom g) {
  using A = typename AccOf<T>::type;
  using P = Pack<T, kVec>;
  __shared__ A red[kThreads * kVec];

  const int tcol = threadIdx.x % g.cols;
  const int lane = threadIdx.x / g.cols;
  const int col = blockIdx.x * g.cols + tcol;
  const bool active = lane < g.lanes && col < g.cv;
  const int64_t r0 = static_cast<int64_t>(blockIdx.y) * g.rows_per_split;
  const int64_t r1 = min(g.rows, r0 + g.rows_per_split);

  alignas(8) A acc[kVec];
#pragma unroll
  for (int i = 0; i < kVec; ++i) acc[i] = A(0);

  GridDepWait();
  GridDepLaunch();

  if (active) {
    const P* gy = reinterpret_cast<const P*>(dy);
    const P* gf = reinterpret_cast<const P*>(feat);
    P* gx = reinterpret_cast<P*>(dx);
    const int64_t step = static_cast<int64_t>(g.lanes) * kUnroll;
    int64_t r = r0 + lane;
    for (; r + step - g.lanes < r1; r += step) {
      P a[kUnroll];
      P f[kUnroll];
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        const int64_t at = (r + static_cast<int64_t>(u) * g.lanes) * g.cv + col;
        a[u] = LoadStream(gy + at);
        if constexpr (kFused) f[u] = LoadStream(gf + at);
      }
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        P o;
        Accumulate<T, kVec, kFused>(a[u], f[u], o, acc);
        if constexpr (kFused) {
          StoreStream(gx + (r + static_cast<int64_t>(u) * g.lanes) * g.cv + col, o);
        }
      }
    }
    if (r < r1) {
      // Last partial group: the same loads, each under its own row check.
      P a[kUnroll];
      P f[kUnroll];
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        const int64_t rr = r + static_cast<int64_t>(u) * g.lanes;
        if (rr < r1) {
          a[u] = LoadStream(gy + rr * g.cv + col);
          if constexpr (kFused) f[u] = LoadStream(gf + rr * g.cv + col);
        }
      }
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        const int64_t rr = r + static_cast<int64_t>(u) * g.lanes;
        if (rr < r1) {
          P o;
          Accumulate<T, kVec, kFused>(a[u], f[u], o, acc);
          if constexpr (kFused) StoreStream(gx + rr * g.cv + col, o);
        }
      }
    }
  }

  // Row lanes of the CTA -> one value per channel, added in lane order.
#pragma unroll
  for (int i = 0; i < kVec; ++i) red[threadIdx.x * kVec + i] = acc[i];
  __syncthreads();
  if (active && lane == 0) {
#pragma unroll
    for (int i = 0; i < kVec; ++i) {
      A s = acc[i];
      for (int l = 1; l < g.lanes; ++l) s += red[(l * g.cols + tcol) * kVec + i];
      partial[static_cast<int64_t>(blockIdx.y) * g.cv * kVec +
              static_cast<int64_t>(col) * kVec + i] = s;
    }
  }
}

struct PlaneGeom {
  int64_t outer;
  int64_t channels;
  int64_t inner;
  int64_t outer_per_split;
};

// Channel-major ([outer, channels, inner], inner > 1).  A plane (n, c) is a run
// of `inner` contiguous elements.  A warp owns one channel and walks the
// planes of its CTA's split of the outer axis as ONE flattened sequence of
// packs (lane l takes packs l, l + 32, ... of it, whatever the plane length),
// with kPlaneUnroll loads per input in flight; the pack width is the widest
// that divides the plane, so no access straddles planes.  8 channels per CTA.
constexpr int kPlaneUnroll = 4;
constexpr int kPlaneWarps = kThreads / 32;

template <typename T, int kVec, bool kFused>
__global__ void __launch_bounds__(kThreads)
    BiasGradPlaneKernel(const T* __restrict__ dy, const T* __restrict__ feat,
                        T* __restrict__ dx,
                        typename AccOf<T>::type* __restrict__ partial,
                        PlaneGeom g) {
  using A = typename AccOf<T>::type;
  using P = Pack<T, kVec>;
  GridDepWait();
  GridDepLaunch();
  const int lane = threadIdx.x & 31;
  const int64_t c = static_cast<int64_t>(blockIdx.x) * kPlaneWarps + (threadIdx.x >> 5);
  if (c >= g.channels) return;  // whole warp; nothing below synchronises the CTA
  const int64_t n0 = static_cast<int64_t>(blockIdx.y) * g.outer_per_split;
  const int64_t n1 = min(g.outer, n0 + g.outer_per_split);
  const int64_t ip = g.inner / kVec;        // packs per plane
  const int64_t dn = 32 / ip, di = 32 % ip;  // 32 packs further along the walk
  int64_t n = n0 + lane / ip, i = lane % ip;
  const int64_t plane_stride = g.channels * g.inner;
  const T* yc = dy + c * g.inner;
  const T* fc = feat + c * g.inner;
  T* xc = dx + c * g.inner;
  alignas(8) A acc[kVec];
#pragma unroll
  for (int e = 0; e < kVec; ++e) acc[e] = A(0);
  while (n < n1) {
    P a[kPlaneUnroll];
    P f[kPlaneUnroll];
    int64_t at[kPlaneUnroll];
#pragma unroll
    for (int u = 0; u < kPlaneUnroll; ++u) {
      at[u] = n < n1 ? n * plane_stride + i * kVec : -1;
      if (at[u] >= 0) {
        a[u] = LoadStream(reinterpret_cast<const P*>(yc + at[u]));
        if constexpr (kFused) f[u] = LoadStream(reinterpret_cast<const P*>(fc + at[u]));
      }
      n += dn;
      i += di;
      if (i >= ip) {
        i -= ip;
        ++n;
      }
    }
#pragma unroll
    for (int u = 0; u < kPlaneUnroll; ++u) {
      if (at[u] >= 0) {
        P o;
        Accumulate<T, kVec, kFused>(a[u], f[u], o, acc);
        if constexpr (kFused) StoreStream(reinterpret_cast<P*>(xc + at[u]), o);
      }
    }
  }
  A s = acc[0];
#pragma unroll
  for (int e = 1; e < kVec; ++e) s += acc[e];
  // Lanes of the warp, in a fixed order.
  if constexpr (sizeof(A) == 4) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const unsigned other = __shfl_xor_sync(0xffffffffu, *reinterpret_cast<unsigned*>(&s), o);
      s += *reinterpret_cast<const A*>(&other);
    }
  } else {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const unsigned long long other =
          __shfl_xor_sync(0xffffffffu, *reinterpret_cast<unsigned long long*>(&s), o);
      s += *reinterpret_cast<const A*>(&other);
    }
  }
  if (lane == 0) partial[static_cast<int64_t>(blockIdx.y) * g.channels + c] = s;
}

// Level 2: bias_grad[c] = sum over the partial rows.  A CTA owns 8 channels
// and reads 32 partial rows at once (a warp covers 4 rows x 8 channels, one
// 32-byte sector per row); every thread keeps four independent sums so that
// four loads are in flight, and all adds happen in a fixed order in the wide
// type.
constexpr int kFinCh = 8;
constexpr int kFinLanes = kThreads / kFinCh;

template <typename T>
__global__ void __launch_bounds__(kThreads)
    BiasGradFinalizeKernel(const typename AccOf<T>::type* __restrict__ partial,
                           int splits, int64_t channels, T* __restrict__ out) {
  using W = typename AccOf<T>::wide;
  __shared__ W red[kThreads];
  const int tc = threadIdx.x % kFinCh;
  const int tl = threadIdx.x / kFinCh;
  const int64_t c = static_cast<int64_t>(blockIdx.x) * kFinCh + tc;

  GridDepWait();
  GridDepLaunch();

  W s0 = W(0), s1 = W(0), s2 = W(0), s3 = W(0);
  if (c < channels) {
    const typename AccOf<T>::type* src = partial + c;
    int p = tl;
    for (; p + 3 * kFinLanes < splits; p += 4 * kFinLanes) {
      const auto v0 = src[static_cast<int64_t>(p) * channels];
      const auto v1 = src[static_cast<int64_t>(p + kFinLanes) * channels];
      const auto v2 = src[static_cast<int64_t>(p + 2 * kFinLanes) * channels];
      const auto v3 = src[static_cast<int64_t>(p + 3 * kFinLanes) * channels];
      s0 += static_cast<W>(v0);
      s1 += static_cast<W>(v1);
      s2 += static_cast<W>(v2);
      s3 += static_cast<W>(v3);
    }
    for (; p < splits; p += kFinLanes) {
      s0 += static_cast<W>(src[static_cast<int64_t>(p) * channels]);
    }
  }
  W s = (s0 + s1) + (s2 + s3);
  red[threadIdx.x] = s;
  __syncthreads();
  if (tl == 0 && c < channels) {
    for (int l = 1; l < kFinLanes; ++l) s += red[l * kFinCh + tc];
    out[c] = NarrowTo<T>(s);
  }
}

template <typename T, int kVec>
__global__ void __launch_bounds__(kThreads)
    ReluGradKernel(const T* __restrict__ dy, const T* __restrict__ feat,
                   T* __restrict__ dx, int64_t packs, int64_t n) {
  using P = Pack<T, kVec>;
  constexpr int kUnroll = 4;
  const P* gy = reinterpret_cast<const P*>(dy);
  const P* gf = reinterpret_cast<const P*>(feat);
  P* gx = reinterpret_cast<P*>(dx);
  const int64_t stride = static_cast<int64_t>(gridDim.x) * kThreads;
  int64_t i = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x;
  for (; i + (kUnroll - 1) * stride < packs; i += kUnroll * stride) {
    P a[kUnroll];
    P f[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      a[u] = LoadStream(gy + i + u * stride);
      f[u] = LoadStream(gf + i + u * stride);
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      P o;
#pragma unroll
      for (int k = 0; k < kVec; ++k) {
        o.v[k] = NarrowTo<T>(MaskGrad(a[u].v[k], f[u].v[k]));
      }
      StoreStream(gx + i + u * stride, o);
    }
  }
  for (; i < packs; i += stride) {
    const P a = LoadStream(gy + i);
    const P f = LoadStream(gf + i);
    P o;
#pragma unroll
    for (int k = 0; k < kVec; ++k) o.v[k] = NarrowTo<T>(MaskGrad(a.v[k], f.v[k]));
    StoreStream(gx + i, o);
  }
  // Elements past the last whole pack.
  const int64_t tail = packs * kVec + static_cast<int64_t>(blockIdx.x) * kThreads +
                       threadIdx.x;
  if (tail < n) dx[tail] = NarrowTo<T>(MaskGrad(dy[tail], feat[tail]));
}

// ---------------------------------------------------------------------------

inline int LastError() { return static_cast<int>(cudaGetLastError()); }

struct Geom {
  int64_t outer, channels, inner;
};

inline bool BadGeom(const Geom& g) {
  return g.outer < 0 || g.channels < 0 || g.inner < 0 ||
         g.channels > (int64_t(1) << 30);
}

// Upper bound of the row splits for a geometry: one wave of the largest grid
// that can be resident, divided by the CTAs that one row needs.  The same
// figure sizes the workspace and caps the launch.
inline int MaxSplits(const Geom& g, size_t elem) {
  const int64_t budget = static_cast<int64_t>(SmCount()) * kMaxCtasPerSm;
  if (g.inner == 1) {
    const int vec = static_cast<int>(16 / elem);
    const int64_t cv = CeilDiv(g.channels, vec);
    const int64_t cols = cv < kColsPerCta ? cv : kColsPerCta;
    const int64_t grid_x = CeilDiv(cv, cols);
    const int64_t lanes = kThreads / cols;
    int64_t s = budget / grid_x;
    const int64_t by_rows = CeilDiv(g.outer, lanes * 4);
    if (s > by_rows) s = by_rows;
    return static_cast<int>(s < 1 ? 1 : s);
  }
  // Channel-major: 8 channels (warps) per CTA along x.
  const int64_t gx = CeilDiv(g.channels > 0 ? g.channels : 1, kThreads / 32);
  int64_t s = budget / gx;
  if (s > g.outer) s = g.outer;
  if (s > 65535) s = 65535;
  return static_cast<int>(s < 1 ? 1 : s);
}

inline size_t WorkspaceBytes(const Geom& g, size_t elem) {
  if (g.channels == 0) return 0;
  // One partial row of 8-byte accumulators per split.
  return static_cast<size_t>(MaxSplits(g, elem)) *
         static_cast<size_t>(g.channels) * 8;
}

template <typename T, int kVec, bool kFused>
int LaunchLast(const T* dy, const T* feat, T* dx,
               typename AccOf<T>::type* partial, const Geom& g, int splits,
               cudaStream_t stream, int* splits_used) {
  constexpr int kUnroll = kFused ? 4 : 8;
  auto kernel = BiasGradLastKernel<T, kVec, kUnroll, kFused>;
  LastGeom lg;
  lg.rows = g.outer;
  lg.cv = static_cast<int>(g.channels / kVec);
  lg.cols = lg.cv < kColsPerCta ? lg.cv : kColsPerCta;
  lg.lanes = kThreads / lg.cols;
  const int grid_x = static_cast<int>(CeilDiv(lg.cv, lg.cols));

  static std::atomic<int> per_sm_by_device[kMaxDevices];
  int per_sm = PerDevice(per_sm_by_device, [&] {
    int n = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kernel, kThreads, 0) !=
        cudaSuccess) {
      cudaGetLastError();
    }
    return n > 0 ? n : 1;
  });
  if (per_sm > kMaxCtasPerSm) per_sm = kMaxCtasPerSm;
  int64_t want = static_cast<int64_t>(SmCount()) * per_sm / grid_x;
  const int64_t by_rows = CeilDiv(g.outer, static_cast<int64_t>(lg.lanes) * 4);
  if (want > by_rows) want = by_rows;
  if (want > splits) want = splits;
  if (want < 1) want = 1;
  lg.rows_per_split = CeilDiv(g.outer, want);
  const int used = static_cast<int>(CeilDiv(g.outer, lg.rows_per_split));
  *splits_used = used;
  const cudaError_t e =
      LaunchChained(true, kernel, dim3(grid_x, used), dim3(kThreads), 0, stream,
                    dy, feat, dx, partial, lg);
  return static_cast<int>(e);
}

template <typename T, int kVec, bool kFused>
int LaunchPlanes(const T* dy, const T* feat, T* dx,
                 typename AccOf<T>::type* partial, const Geom& g, int splits,
                 cudaStream_t stream, int* splits_used) {
  PlaneGeom pg;
  pg.outer = g.outer;
  pg.channels = g.channels;
  pg.inner = g.inner;
  const int64_t gx = CeilDiv(g.channels, kPlaneWarps);
  int64_t want = static_cast<int64_t>(SmCount()) * kMaxCtasPerSm / gx;
  if (want > splits) want = splits;
  if (want > g.outer) want = g.outer;
  if (want < 1) want = 1;
  pg.outer_per_split = CeilDiv(g.outer, want);
  const int used = static_cast<int>(CeilDiv(g.outer, pg.outer_per_split));
  *splits_used = used;
  const cudaError_t e = LaunchChained(
      true, BiasGradPlaneKernel<T, kVec, kFused>, dim3(static_cast<unsigned>(gx), used),
      dim3(kThreads), 0, stream, dy, feat, dx, partial, pg);
  return static_cast<int>(e);
}

// Widest pack (in elements, at most 16 bytes) that divides a plane.
template <typename T>
int PlaneVec(int64_t inner, bool aligned) {
  if (!aligned) return 1;
  for (int v = VecWidth<T>::value; v > 1; v >>= 1) {
    if (inner % v == 0) return v;
  }
  return 1;
}

template <typename T, bool kFused>
int BiasGrad(const void* dy_v, const void* feat_v, void* dx_v, void* out_v,
             const Geom& g, void* workspace, size_t workspace_bytes,
             cudaStream_t stream) {
  using A = typename AccOf<T>::type;
  if (BadGeom(g)) return MUSA_KERNELS_EINVAL;
  MUSA_TRACE(kFused ? "LaunchBiasAddReluGrad" : "LaunchBiasAddGrad",
             (kFused ? 3 : 1) * sizeof(T) * g.outer * g.channels * g.inner);
  if (g.channels == 0) return MUSA_KERNELS_OK;
  if (out_v == nullptr) return MUSA_KERNELS_EINVAL;
  T* out = static_cast<T*>(out_v);
  if (g.outer == 0 || g.inner == 0) {
    // Nothing to add: the sum over an empty axis is zero.
    const cudaError_t e =
        cudaMemsetAsync(out, 0, sizeof(T) * g.channels, stream);
    return static_cast<int>(e);
  }
  if (dy_v == nullptr || (kFused && (feat_v == nullptr || dx_v == nullptr))) {
    return MUSA_KERNELS_EINVAL;
  }
  if (workspace == nullptr || workspace_bytes < WorkspaceBytes(g, sizeof(T)) ||
      (reinterpret_cast<uintptr_t>(workspace) & 15u) != 0) {
    return MUSA_KERNELS_EWORKSPACE;
  }
  const T* dy = static_cast<const T*>(dy_v);
  const T* feat = static_cast<const T*>(feat_v);
  T* dx = static_cast<T*>(dx_v);
  A* partial = static_cast<A*>(workspace);
  const int splits = MaxSplits(g, sizeof(T));
  constexpr int kFull = VecWidth<T>::value;
  const bool aligned =
      Aligned16(dy) && (!kFused || (Aligned16(feat) && Aligned16(dx)));
  int used = 0;
  int rc;
  if (g.inner == 1) {
    if (aligned && g.channels % kFull == 0) {
      rc = LaunchLast<T, kFull, kFused>(dy, feat, dx, partial, g, splits, stream,
                                        &used);
    } else {
      rc = LaunchLast<T, 1, kFused>(dy, feat, dx, partial, g, splits, stream,
                                    &used);
    }
  } else {
    switch (PlaneVec<T>(g.inner, aligned)) {
      case 8:
        if constexpr (kFull >= 8) {
          rc = LaunchPlanes<T, 8, kFused>(dy, feat, dx, partial, g, splits, stream, &used);
        } else {
          rc = MUSA_KERNELS_EINVAL;
        }
        break;
      case 4:
        if constexpr (kFull >= 4) {
          rc = LaunchPlanes<T, 4, kFused>(dy, feat, dx, partial, g, splits, stream, &used);
        } else {
          rc = MUSA_KERNELS_EINVAL;
        }
        break;
      case 2:
        rc = LaunchPlanes<T, 2, kFused>(dy, feat, dx, partial, g, splits, stream, &used);
        break;
      default:
        rc = LaunchPlanes<T, 1, kFused>(dy, feat, dx, partial, g, splits, stream, &used);
    }
  }
  if (rc != 0) return rc;
  const cudaError_t e = LaunchChained(
      true, BiasGradFinalizeKernel<T>,
      dim3(static_cast<unsigned>(CeilDiv(g.channels, kFinCh))), dim3(kThreads), 0,
      stream, static_cast<const A*>(partial), used, g.channels, out);
  if (e != cudaSuccess) return static_cast<int>(e);
  return LastError();
}

template <typename T>
int ReluGrad(const void* dy_v, const void* feat_v, void* dx_v, int64_t n,
             cudaStream_t stream) {
  if (n < 0) return MUSA_KERNELS_EINVAL;
  MUSA_TRACE("LaunchReluGrad", 3 * sizeof(T) * n);
  if (n == 0) return MUSA_KERNELS_OK;
  if (dy_v == nullptr || feat_v == nullptr || dx_v == nullptr) {
    return MUSA_KERNELS_EINVAL;
  }
  const T* dy = static_cast<const T*>(dy_v);
  const T* feat = static_cast<const T*>(feat_v);
  T* dx = static_cast<T*>(dx_v);
  constexpr int kFull = VecWidth<T>::value;
  const bool aligned = Aligned16(dy) && Aligned16(feat) && Aligned16(dx);
  if (aligned) {
    const int64_t packs = n / kFull;
    auto kernel = ReluGradKernel<T, kFull>;
    static std::atomic<int> per_sm_by_device[kMaxDevices];
    const int per_sm = PerDevice(per_sm_by_device, [&] {
      int n = 0;
      if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kernel, kThreads, 0) !=
          cudaSuccess) {
        cudaGetLastError();
      }
      return n > 0 ? n : 1;
    });
    int64_t grid = static_cast<int64_t>(SmCount()) * per_sm;
    const int64_t need = CeilDiv(packs > 0 ? packs : 1, kThreads);
    if (grid > need) grid = need;
    kernel<<<static_cast<unsigned>(grid), kThreads, 0, stream>>>(dy, feat, dx,
                                                                 packs, n);
    CountKernelLaunch();
  } else {
    int64_t grid = CeilDiv(n, kThreads);
    const int64_t cap = static_cast<int64_t>(SmCount()) * kMaxCtasPerSm;
    if (grid > cap) grid = cap;
    ReluGradKernel<T, 1><<<static_cast<unsigned>(grid), kThreads, 0, stream>>>(
        dy, feat, dx, n, n);
    CountKernelLaunch();
  }
  return LastError();
}

}  // namespace
}  // namespace musa_b200

using musa_b200::BiasGrad;
using musa_b200::Geom;
using musa_b200::ReluGrad;

extern "C" {

size_t BiasGradWorkspaceBytes(int64_t outer, int64_t channels, int64_t inner,
                              int elem_bytes) {
  const Geom g{outer, channels, inner};
  if (musa_b200::BadGeom(g) || elem_bytes < 2 || elem_bytes > 8) return 0;
  return musa_b200::WorkspaceBytes(g, static_cast<size_t>(elem_bytes));
}

#define MUSA_DEFINE_BIAS_ADD_GRAD(SUFFIX, TYPE)                               \
  int LaunchBiasAddGrad_##SUFFIX(const void* out_backprop, void* bias_grad,   \
                                 int64_t outer, int64_t channels,             \
                                 int64_t inner, void* workspace,              \
                                 size_t workspace_bytes, cudaStream_t stream) { \
    return BiasGrad<TYPE, false>(out_backprop, nullptr, nullptr, bias_grad,   \
                                 Geom{outer, channels, inner}, workspace,     \
                                 workspace_bytes, stream);                    \
  }
MUSA_DEFINE_BIAS_ADD_GRAD(F32, float)
MUSA_DEFINE_BIAS_ADD_GRAD(F16, __half)
MUSA_DEFINE_BIAS_ADD_GRAD(BF16, __nv_bfloat16)
MUSA_DEFINE_BIAS_ADD_GRAD(F64, double)
MUSA_DEFINE_BIAS_ADD_GRAD(I32, int32_t)
MUSA_DEFINE_BIAS_ADD_GRAD(I64, int64_t)
#undef MUSA_DEFINE_BIAS_ADD_GRAD

#define MUSA_DEFINE_RELU_GRAD(SUFFIX, TYPE)                                   \
  int LaunchReluGrad_##SUFFIX(const void* gradients, const void* features,    \
                              void* backprops, int64_t n,                     \
                              cudaStream_t stream) {                          \
    return ReluGrad<TYPE>(gradients, features, backprops, n, stream);         \
  }                                                                           \
  int LaunchBiasAddReluGrad_##SUFFIX(                                         \
      const void* gradients, const void* features, void* backprops,           \
      void* bias_grad, int64_t outer, int64_t channels, int64_t inner,        \
      void* workspace, size_t workspace_bytes, cudaStream_t stream) {         \
    return BiasGrad<TYPE, true>(gradients, features, backprops, bias_grad,    \
                                Geom{outer, channels, inner}, workspace,      \
                                workspace_bytes, stream);                     \
  }
MUSA_DEFINE_RELU_GRAD(F32, float)
MUSA_DEFINE_RELU_GRAD(F16, __half)
MUSA_DEFINE_RELU_GRAD(BF16, __nv_bfloat16)
#undef MUSA_DEFINE_RELU_GRAD

}  // extern "C"
