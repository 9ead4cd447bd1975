// ApplyAdam for sm_100a: one streaming pass that reads var, m, v, grad and
// writes var, m, v with 128-bit accesses (28 B/element in fp32).
//
// Arithmetic follows the reference kernels exactly: fp32 math, IEEE sqrt and
// divide, (1-beta) taken on the host
// (musa_ext/kernels/training/musa_apply_sparse_adam_kernel.mu:140-157,
//  musa_ext/kernels/training/musa_applyadam_bf16_kernel.mu:82-112,
//  musa_ext/kernels/training/musa_applyadam_mixed_kernel.mu:55-86).
#include <new>

#include "common.cuh"
#include "trace.h"
#include "tuning.h"
#include "../../include/musa_plugin_kernels.h"

namespace musa_b200 {
namespace {

struct AdamParams {
  float lr_t;  // bias-corrected step size ("alpha" in the fp32 launcher)
  float beta1;
  float one_minus_b1;
  float beta2;
  float one_minus_b2;
  float epsilon;
};

template <bool kNesterov>
__device__ __forceinline__ void AdamStep(float& var, float& m, float& v,
                                         float g, const AdamParams& p) {
  // Every rounding is spelled out (one fused multiply-add per moment, IEEE
  // multiply / sqrt / divide / subtract elsewhere) so that all kernels built
  // from this function - vector, element-wise, sharded, broadcasting - return
  // the same bits; left to the compiler, the contraction of a*b + c*d differs
  // from one instantiation to the next by an ulp.
  const float m_new = fmaf(p.beta1, m, __fmul_rn(p.one_minus_b1, g));
  const float v_new = fmaf(p.beta2, v, __fmul_rn(__fmul_rn(p.one_minus_b2, g), g));
  const float numer =
      kNesterov ? fmaf(p.beta1, m_new, __fmul_rn(p.one_minus_b1, g)) : m_new;
  m = m_new;
  v = v_new;
  var = __fsub_rn(var, __fdiv_rn(__fmul_rn(p.lr_t, numer),
                                 __fadd_rn(__fsqrt_rn(v_new), p.epsilon)));
}

// Each thread owns kUnroll packs of kEpt elements per tile; a tile is
// blockDim.x * kUnroll consecutive packs, so that every load instruction of a
// warp covers 32 consecutive packs.  All loads of a tile are issued before the
// first use to keep 4 * kUnroll requests per thread in flight.
template <typename StateT, typename GradT, int kEpt, int kUnroll,
          bool kNesterov>
__global__ void __launch_bounds__(256)
    AdamKernel(StateT* __restrict__ var, StateT* __restrict__ m,
               StateT* __restrict__ v, const GradT* __restrict__ grad,
               AdamParams p, int64_t n) {
  using SPack = Pack<StateT, kEpt>;
  using GPack = Pack<GradT, kEpt>;
  const int64_t n_packs = n / kEpt;
  const int64_t tile = static_cast<int64_t>(blockDim.x) * kUnroll;
  const int64_t n_tiles = (n_packs + tile - 1) / tile;

  SPack* var_p = reinterpret_cast<SPack*>(var);
  SPack* m_p = reinterpret_cast<SPack*>(m);
  SPack* v_p = reinterpret_cast<SPack*>(v);
  const GPack* g_p = reinterpret_cast<const GPack*>(grad);

  for (int64_t t = blockIdx.x; t < n_tiles; t += gridDim.x) {
    const int64_t base = t * tile + threadIdx.x;
    SPack pv[kUnroll], pm[kUnroll], pvv[kUnroll];
    GPack pg[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const int64_t i = base + static_cast<int64_t>(u) * blockDim.x;
      if (i < n_packs) {
        pg[u] = LoadStream(g_p + i);
        pm[u] = LoadStream(m_p + i);
        pvv[u] = LoadStream(v_p + i);
        pv[u] = LoadStream(var_p + i);
      }
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const int64_t i = base + static_cast<int64_t>(u) * blockDim.x;
      if (i < n_packs) {
#pragma unroll
        for (int e = 0; e < kEpt; ++e) {
          float fvar = ToF32(pv[u].v[e]);
          float fm = ToF32(pm[u].v[e]);
          float fv = ToF32(pvv[u].v[e]);
          AdamStep<kNesterov>(fvar, fm, fv, ToF32(pg[u].v[e]), p);
          pv[u].v[e] = FromF32<StateT>(fvar);
          pm[u].v[e] = FromF32<StateT>(fm);
          pvv[u].v[e] = FromF32<StateT>(fv);
        }
        StoreStream(m_p + i, pm[u]);
        StoreStream(v_p + i, pvv[u]);
        StoreStream(var_p + i, pv[u]);
      }
    }
  }

  // Ragged tail (n not a multiple of the pack width): one thread per element.
  if (kEpt > 1 && blockIdx.x == 0) {
    const int64_t i = n_packs * kEpt + threadIdx.x;
    if (threadIdx.x < kEpt && i < n) {
      float fvar = ToF32(var[i]);
      float fm = ToF32(m[i]);
      float fv = ToF32(v[i]);
      AdamStep<kNesterov>(fvar, fm, fv, ToF32(grad[i]), p);
      var[i] = FromF32<StateT>(fvar);
      m[i] = FromF32<StateT>(fm);
      v[i] = FromF32<StateT>(fv);
    }
  }
}

template <typename StateT, typename GradT, int kEpt, int kUnroll>
void LaunchWithNesterov(StateT* var, StateT* m, StateT* v, const GradT* grad,
                        const AdamParams& p, int64_t n, bool nesterov,
                        cudaStream_t stream) {
  const int threads = 256;
  const int64_t n_packs = n / kEpt;
  const int64_t tile = static_cast<int64_t>(threads) * kUnroll;
  int64_t tiles = CeilDiv(n_packs, tile);
  if (tiles < 1) tiles = 1;
  // Tuning value 0: one tile per CTA.  k > 0: a persistent grid of k CTAs per
  // SM that strides over the tiles.
  const int per_sm = GetTuning(kTuneAdamCtasPerSm);
  int64_t blocks = tiles;
  if (per_sm > 0) {
    const int64_t cap = static_cast<int64_t>(SmCount()) * per_sm;
    if (blocks > cap) blocks = cap;
  }
  if (blocks > 0x7fffffffLL) blocks = 0x7fffffffLL;
  if (nesterov) {
    AdamKernel<StateT, GradT, kEpt, kUnroll, true>
        <<<static_cast<unsigned>(blocks), threads, 0, stream>>>(var, m, v, grad,
                                                               p, n);
    CountKernelLaunch();
  } else {
    AdamKernel<StateT, GradT, kEpt, kUnroll, false>
        <<<static_cast<unsigned>(blocks), threads, 0, stream>>>(var, m, v, grad,
                                                               p, n);
    CountKernelLaunch();
  }
}

// Picks the 128-bit path when every pointer allows it, else element-wise
// accesses (TF's BFC allocator hands out 64-byte aligned buffers, so the
// vector path is the normal one; sliced or offset tensors take the other).
template <typename StateT, typename GradT>
void LaunchAdam(StateT* var, StateT* m, StateT* v, const GradT* grad,
                float lr_t, float beta1, float beta2, float epsilon, int64_t n,
                bool nesterov, cudaStream_t stream) {
  MUSA_TRACE("LaunchApplyAdam",
             n > 0 ? (6 * sizeof(StateT) + sizeof(GradT)) * n : 0);
  if (n <= 0) return;
  AdamParams p;
  p.lr_t = lr_t;
  p.beta1 = beta1;
  p.one_minus_b1 = 1.0f - beta1;
  p.beta2 = beta2;
  p.one_minus_b2 = 1.0f - beta2;
  p.epsilon = epsilon;
  // State packs are 16 bytes; the grad pack has the same element count.
  constexpr int kEpt = VecWidth<StateT>::value;
  constexpr size_t kGradPackBytes = sizeof(GradT) * kEpt;
  const bool vec_ok =
      Aligned16(var) && Aligned16(m) && Aligned16(v) &&
      (reinterpret_cast<uintptr_t>(grad) % kGradPackBytes) == 0;
  if (vec_ok) {
    if (GetTuning(kTuneAdamUnroll) == 1) {
      LaunchWithNesterov<StateT, GradT, kEpt, 1>(var, m, v, grad, p, n,
                                                 nesterov, stream);
    } else if (GetTuning(kTuneAdamUnroll) == 4) {
      LaunchWithNesterov<StateT, GradT, kEpt, 4>(var, m, v, grad, p, n,
                                                 nesterov, stream);
    } else {
      LaunchWithNesterov<StateT, GradT, kEpt, 2>(var, m, v, grad, p, n,
                                                 nesterov, stream);
    }
  } else {
    LaunchWithNesterov<StateT, GradT, 1, 4>(var, m, v, grad, p, n, nesterov,
                                            stream);
  }
}

// ---- Range-sharded Adam whose update IS the all-gather: a replica updates
// its range [lo, lo + n) of the parameter vector and stores every new value
// into that range of EVERY replica's copy (its own and, over NVLink, the
// peers'), so no separate collective re-reads and re-sends the shard.
struct Replicas {
  float* var[16];
  int world;
  int rank;
};

// GradT: the gradient's type (fp32 as ResourceApplyAdam, or fp16 / bf16 beside
// fp32 state as MusaResourceApplyAdamMixed, which also honours use_nesterov).
template <typename GradT, int kEpt, bool kNesterov>
__global__ void __launch_bounds__(256)
    AdamShardBroadcastKernel(Replicas r, int64_t lo, float* __restrict__ m,
                             float* __restrict__ v, const GradT* __restrict__ grad,
                             AdamParams p, int64_t n) {
  GridDepWait();
  GridDepLaunch();
  using SPack = Pack<float, kEpt>;
  using GPack = Pack<GradT, kEpt>;
  constexpr int kUnroll = 2;
  const int64_t n_packs = n / kEpt;
  const int64_t tile = static_cast<int64_t>(blockDim.x) * kUnroll;
  const int64_t n_tiles = (n_packs + tile - 1) / tile;
  const SPack* var_p = reinterpret_cast<const SPack*>(r.var[r.rank] + lo);
  SPack* m_p = reinterpret_cast<SPack*>(m);
  SPack* v_p = reinterpret_cast<SPack*>(v);
  const GPack* g_p = reinterpret_cast<const GPack*>(grad);
  for (int64_t t = blockIdx.x; t < n_tiles; t += gridDim.x) {
    const int64_t base = t * tile + threadIdx.x;
    SPack pv[kUnroll], pm[kUnroll], pvv[kUnroll];
    GPack pg[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const int64_t i = base + static_cast<int64_t>(u) * blockDim.x;
      if (i < n_packs) {
        pg[u] = LoadStream(g_p + i);
        pm[u] = LoadStream(m_p + i);
        pvv[u] = LoadStream(v_p + i);
        pv[u] = LoadStream(var_p + i);
      }
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const int64_t i = base + static_cast<int64_t>(u) * blockDim.x;
      if (i < n_packs) {
#pragma unroll
        for (int e = 0; e < kEpt; ++e) {
          AdamStep<kNesterov>(pv[u].v[e], pm[u].v[e], pvv[u].v[e], ToF32(pg[u].v[e]), p);
        }
        StoreStream(m_p + i, pm[u]);
        StoreStream(v_p + i, pvv[u]);
        // Own copy first, then the peers, each replica starting at a
        // different peer so that the links load evenly.
        for (int k = 0; k < r.world; ++k) {
          const int q = (r.rank + k) % r.world;
          reinterpret_cast<SPack*>(r.var[q] + lo)[i] = pv[u];
        }
      }
    }
  }
  if (kEpt > 1 && blockIdx.x == 0) {
    const int64_t i = n_packs * kEpt + threadIdx.x;
    if (threadIdx.x < kEpt && i < n) {
      float fvar = r.var[r.rank][lo + i], fm = m[i], fv = v[i];
      AdamStep<kNesterov>(fvar, fm, fv, ToF32(grad[i]), p);
      m[i] = fm;
      v[i] = fv;
      for (int q = 0; q < r.world; ++q) r.var[q][lo + i] = fvar;
    }
  }
}

// ---- The same step through an NVSwitch multicast mapping: one `multimem.st`
// per pack writes the new weights into the copy of EVERY replica (the switch
// replicates the store), so the shard leaves the GPU once instead of once per
// peer, and the step is no longer bound by NVLink egress.
__device__ __forceinline__ void MulticastStore4(float* mc, const Pack<float, 4>& p) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc),
               "f"(p.v[0]), "f"(p.v[1]), "f"(p.v[2]), "f"(p.v[3])
               : "memory");
}
__device__ __forceinline__ void MulticastStore1(float* mc, float v) {
  asm volatile("multimem.st.relaxed.sys.global.f32 [%0], %1;" ::"l"(mc), "f"(v) : "memory");
}

__global__ void __launch_bounds__(256)
    AdamShardMulticastKernel(const float* __restrict__ var_local, float* __restrict__ var_mc,
                             float* __restrict__ m, float* __restrict__ v,
                             const float* __restrict__ grad, AdamParams p, int64_t n) {
  GridDepWait();
  GridDepLaunch();
  using SPack = Pack<float, 4>;
  constexpr int kUnroll = 2;
  const int64_t n_packs = n / 4;
  const int64_t tile = static_cast<int64_t>(blockDim.x) * kUnroll;
  const int64_t n_tiles = (n_packs + tile - 1) / tile;
  const SPack* var_p = reinterpret_cast<const SPack*>(var_local);
  SPack* m_p = reinterpret_cast<SPack*>(m);
  SPack* v_p = reinterpret_cast<SPack*>(v);
  const SPack* g_p = reinterpret_cast<const SPack*>(grad);
  for (int64_t t = blockIdx.x; t < n_tiles; t += gridDim.x) {
    const int64_t base = t * tile + threadIdx.x;
    SPack pv[kUnroll], pm[kUnroll], pvv[kUnroll], pg[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const int64_t i = base + static_cast<int64_t>(u) * blockDim.x;
      if (i < n_packs) {
        pg[u] = LoadStream(g_p + i);
        pm[u] = LoadStream(m_p + i);
        pvv[u] = LoadStream(v_p + i);
        pv[u] = LoadStream(var_p + i);
      }
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const int64_t i = base + static_cast<int64_t>(u) * blockDim.x;
      if (i < n_packs) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          AdamStep<false>(pv[u].v[e], pm[u].v[e], pvv[u].v[e], pg[u].v[e], p);
        }
        StoreStream(m_p + i, pm[u]);
        StoreStream(v_p + i, pvv[u]);
        MulticastStore4(var_mc + i * 4, pv[u]);   // all replicas, this one included
      }
    }
  }
  if (blockIdx.x == 0) {
    const int64_t i = n_packs * 4 + threadIdx.x;
    if (threadIdx.x < 4 && i < n) {
      float fvar = var_local[i], fm = m[i], fv = v[i];
      AdamStep<false>(fvar, fm, fv, grad[i], p);
      m[i] = fm;
      v[i] = fv;
      MulticastStore1(var_mc + i, fvar);
    }
  }
}

template <typename GradT>
int AdamShardBroadcast(float* const* var_replicas, int world, int rank, int64_t lo, float* m,
                       float* v, const GradT* grad, float beta1, float beta2, float epsilon,
                       float alpha, int64_t n, bool nesterov, cudaStream_t stream) {
  if (var_replicas == nullptr || world < 1 || world > 16 || rank < 0 || rank >= world ||
      lo < 0 || n < 0) {
    return MUSA_KERNELS_EINVAL;
  }
  MUSA_TRACE("LaunchAdamShardBroadcast", (24 + sizeof(GradT)) * n);
  if (n == 0) return MUSA_KERNELS_OK;
  if (m == nullptr || v == nullptr || grad == nullptr) return MUSA_KERNELS_EINVAL;
  Replicas r{};
  r.world = world;
  r.rank = rank;
  // 128-bit state packs beside a gradient pack of the same four elements.
  bool vec = (lo % 4 == 0) && Aligned16(m) && Aligned16(v) &&
             reinterpret_cast<uintptr_t>(grad) % (4 * sizeof(GradT)) == 0;
  for (int q = 0; q < world; ++q) {
    if (var_replicas[q] == nullptr) return MUSA_KERNELS_EINVAL;
    r.var[q] = var_replicas[q];
    vec = vec && Aligned16(var_replicas[q]);
  }
  AdamParams p;
  p.lr_t = alpha;
  p.beta1 = beta1;
  p.one_minus_b1 = 1.0f - beta1;
  p.beta2 = beta2;
  p.one_minus_b2 = 1.0f - beta2;
  p.epsilon = epsilon;
  const int64_t packs = vec ? n / 4 : n;
  int64_t blocks = CeilDiv(packs, 256 * 2);
  if (blocks < 1) blocks = 1;
  if (blocks > 0x7fffffffLL) blocks = 0x7fffffffLL;
  const dim3 grid(static_cast<unsigned>(blocks));
  cudaError_t err;
  if (vec) {
    err = nesterov ? LaunchChained(true, AdamShardBroadcastKernel<GradT, 4, true>, grid,
                                   dim3(256), 0, stream, r, lo, m, v, grad, p, n)
                   : LaunchChained(true, AdamShardBroadcastKernel<GradT, 4, false>, grid,
                                   dim3(256), 0, stream, r, lo, m, v, grad, p, n);
  } else {
    err = nesterov ? LaunchChained(true, AdamShardBroadcastKernel<GradT, 1, true>, grid,
                                   dim3(256), 0, stream, r, lo, m, v, grad, p, n)
                   : LaunchChained(true, AdamShardBroadcastKernel<GradT, 1, false>, grid,
                                   dim3(256), 0, stream, r, lo, m, v, grad, p, n);
  }
  if (err != cudaSuccess) {
    cudaGetLastError();
    return static_cast<int>(err);
  }
  return static_cast<int>(cudaGetLastError());
}

}  // namespace
}  // namespace musa_b200

using namespace musa_b200;

extern "C" {

void LaunchResourceApplyAdamFloat(float* var, float* m, float* v,
                                  const float* grad, float beta1, float beta2,
                                  float epsilon, float alpha, int64_t total,
                                  cudaStream_t stream) {
  LaunchAdam<float, float>(var, m, v, grad, alpha, beta1, beta2, epsilon, total,
                           /*nesterov=*/false, stream);
}

void LaunchApplyAdamSameType_BFloat16(void* var, void* m, void* v,
                                      const void* grad, float lr_t, float beta1,
                                      float beta2, float epsilon, int64_t n,
                                      bool use_nesterov, cudaStream_t stream) {
  LaunchAdam<__nv_bfloat16, __nv_bfloat16>(
      static_cast<__nv_bfloat16*>(var), static_cast<__nv_bfloat16*>(m),
      static_cast<__nv_bfloat16*>(v), static_cast<const __nv_bfloat16*>(grad),
      lr_t, beta1, beta2, epsilon, n, use_nesterov, stream);
}

void LaunchApplyAdamSameType_Half(void* var, void* m, void* v, const void* grad,
                                  float lr_t, float beta1, float beta2,
                                  float epsilon, int64_t n, bool use_nesterov,
                                  cudaStream_t stream) {
  LaunchAdam<__half, __half>(static_cast<__half*>(var), static_cast<__half*>(m),
                             static_cast<__half*>(v),
                             static_cast<const __half*>(grad), lr_t, beta1,
                             beta2, epsilon, n, use_nesterov, stream);
}

int LaunchAdamShardBroadcastFloat(float* const* var_replicas, int world, int rank,
                                  int64_t lo, float* m, float* v, const float* grad,
                                  float beta1, float beta2, float epsilon, float alpha,
                                  int64_t n, cudaStream_t stream) {
  return AdamShardBroadcast<float>(var_replicas, world, rank, lo, m, v, grad, beta1, beta2,
                                   epsilon, alpha, n, false, stream);
}

int LaunchAdamShardBroadcastMixed(int grad_dtype, float* const* var_replicas, int world,
                                  int rank, int64_t lo, float* m, float* v, const void* grad,
                                  float beta1, float beta2, float epsilon, float alpha,
                                  int64_t n, bool use_nesterov, cudaStream_t stream) {
  switch (grad_dtype) {
    case MUSA_DT_F32:
      return AdamShardBroadcast<float>(var_replicas, world, rank, lo, m, v,
                                       static_cast<const float*>(grad), beta1, beta2, epsilon,
                                       alpha, n, use_nesterov, stream);
    case MUSA_DT_F16:
      return AdamShardBroadcast<__half>(var_replicas, world, rank, lo, m, v,
                                        static_cast<const __half*>(grad), beta1, beta2, epsilon,
                                        alpha, n, use_nesterov, stream);
    case MUSA_DT_BF16:
      return AdamShardBroadcast<__nv_bfloat16>(var_replicas, world, rank, lo, m, v,
                                               static_cast<const __nv_bfloat16*>(grad), beta1,
                                               beta2, epsilon, alpha, n, use_nesterov, stream);
    default:
      return MUSA_KERNELS_EUNSUPPORTED;
  }
}

int LaunchAdamShardMulticastFloat(float* var_local, float* var_multicast, int64_t lo,
                                  float* m, float* v, const float* grad, float beta1,
                                  float beta2, float epsilon, float alpha, int64_t n,
                                  cudaStream_t stream) {
  if (var_local == nullptr || var_multicast == nullptr || lo < 0 || n < 0) {
    return MUSA_KERNELS_EINVAL;
  }
  MUSA_TRACE("LaunchAdamShardMulticast", 28 * n);
  if (n == 0) return MUSA_KERNELS_OK;
  if (m == nullptr || v == nullptr || grad == nullptr) return MUSA_KERNELS_EINVAL;
  // 128-bit packs throughout: the range starts on a pack and every pointer is
  // 16-byte aligned (the multicast store has no element-wise form here).
  if (lo % 4 != 0 || !Aligned16(var_local) || !Aligned16(var_multicast) || !Aligned16(m) ||
      !Aligned16(v) || !Aligned16(grad)) {
    return MUSA_KERNELS_EINVAL;
  }
  AdamParams p;
  p.lr_t = alpha;
  p.beta1 = beta1;
  p.one_minus_b1 = 1.0f - beta1;
  p.beta2 = beta2;
  p.one_minus_b2 = 1.0f - beta2;
  p.epsilon = epsilon;
  int64_t blocks = CeilDiv(n / 4, 256 * 2);
  if (blocks < 1) blocks = 1;
  if (blocks > 0x7fffffffLL) blocks = 0x7fffffffLL;
  const cudaError_t err = LaunchChained(
      true, AdamShardMulticastKernel, dim3(static_cast<unsigned>(blocks)), dim3(256), 0, stream,
      static_cast<const float*>(var_local + lo), var_multicast + lo, m, v, grad, p, n);
  if (err != cudaSuccess) {
    cudaGetLastError();
    return static_cast<int>(err);
  }
  return MUSA_KERNELS_OK;
}

// ---- Range-sharded Adam with the copy engines as the all-gather.  From four
// replicas on, the step is bound by the bytes that leave the GPU over NVLink
// ((world - 1) / world of the vector), and the copy engines move them at the
// peer-copy rate, which stores issued by SMs do not reach.  The local range is
// updated chunk by chunk on the caller's stream; as soon as a chunk is done
// (an event), one cudaMemcpyAsync per peer carries it out on that peer's side
// stream while the next chunk updates.  The caller's stream joins all side
// streams at the end, so the call behaves like one asynchronous operation on
// `stream` and can be captured in a CUDA graph.
struct ShardPipe {
  int world;
  int rank;
  int device;
  cudaStream_t side[16];
  cudaEvent_t done[16];
  cudaEvent_t chunk[8];
};

void* MusaShardPipeCreate(int world, int rank) {
  if (world < 1 || world > 16 || rank < 0 || rank >= world) return nullptr;
  auto* p = new (std::nothrow) ShardPipe();
  if (p == nullptr) return nullptr;
  p->world = world;
  p->rank = rank;
  bool ok = cudaGetDevice(&p->device) == cudaSuccess;
  for (int k = 0; k < world - 1 && ok; ++k) {
    ok = cudaStreamCreateWithFlags(&p->side[k], cudaStreamNonBlocking) == cudaSuccess &&
         cudaEventCreateWithFlags(&p->done[k], cudaEventDisableTiming) == cudaSuccess;
  }
  for (int c = 0; c < 8 && ok; ++c) {
    ok = cudaEventCreateWithFlags(&p->chunk[c], cudaEventDisableTiming) == cudaSuccess;
  }
  if (!ok) {
    cudaGetLastError();
    MusaShardPipeDestroy(p);
    return nullptr;
  }
  return p;
}

void MusaShardPipeDestroy(void* pipe) {
  auto* p = static_cast<ShardPipe*>(pipe);
  if (p == nullptr) return;
  for (int k = 0; k < 16; ++k) {
    if (p->side[k] != nullptr) cudaStreamDestroy(p->side[k]);
    if (p->done[k] != nullptr) cudaEventDestroy(p->done[k]);
  }
  for (int c = 0; c < 8; ++c) {
    if (p->chunk[c] != nullptr) cudaEventDestroy(p->chunk[c]);
  }
  delete p;
}

int LaunchAdamShardCopyFloat(void* pipe, float* const* var_replicas, int64_t lo, float* m,
                             float* v, const float* grad, float beta1, float beta2,
                             float epsilon, float alpha, int64_t n, int chunks,
                             cudaStream_t stream) {
  auto* p = static_cast<ShardPipe*>(pipe);
  if (p == nullptr || var_replicas == nullptr || lo < 0 || n < 0) return MUSA_KERNELS_EINVAL;
  MUSA_TRACE("LaunchAdamShardCopy", 28 * n);
  if (n == 0) return MUSA_KERNELS_OK;
  if (m == nullptr || v == nullptr || grad == nullptr) return MUSA_KERNELS_EINVAL;
  for (int q = 0; q < p->world; ++q) {
    if (var_replicas[q] == nullptr) return MUSA_KERNELS_EINVAL;
  }
  if (chunks < 1) chunks = 1;
  if (chunks > 8) chunks = 8;
  // Chunk boundaries on multiples of 1024 elements (whole 128-bit packs, whole
  // CTAs' tiles), the last chunk taking the remainder.
  int64_t per = (n / chunks + 1023) / 1024 * 1024;
  if (per < 1024) per = 1024;
  float* local = var_replicas[p->rank] + lo;
  int used = 0;
  for (int64_t off = 0; off < n && used < 8; off += per, ++used) {
    const int64_t len = used == 7 || off + per > n ? n - off : per;
    LaunchAdam<float, float>(local + off, m + off, v + off, grad + off, alpha, beta1, beta2,
                             epsilon, len, /*nesterov=*/false, stream);
    cudaError_t err = cudaEventRecord(p->chunk[used], stream);
    for (int k = 1; k < p->world && err == cudaSuccess; ++k) {
      const int q = (p->rank + k) % p->world;   // every replica starts at another peer
      err = cudaStreamWaitEvent(p->side[k - 1], p->chunk[used], 0);
      if (err == cudaSuccess) {
        err = cudaMemcpyAsync(var_replicas[q] + lo + off, local + off,
                              sizeof(float) * static_cast<size_t>(len),
                              cudaMemcpyDeviceToDevice, p->side[k - 1]);
      }
    }
    if (err != cudaSuccess) {
      cudaGetLastError();
      return static_cast<int>(err);
    }
    if (len == n - off) {
      ++used;
      break;
    }
  }
  for (int k = 1; k < p->world; ++k) {
    cudaError_t err = cudaEventRecord(p->done[k - 1], p->side[k - 1]);
    if (err == cudaSuccess) err = cudaStreamWaitEvent(stream, p->done[k - 1], 0);
    if (err != cudaSuccess) {
      cudaGetLastError();
      return static_cast<int>(err);
    }
  }
  return static_cast<int>(cudaGetLastError());
}

void LaunchApplyAdamMixed_Float(float* var, float* m, float* v,
                                const void* grad, float lr_t, float beta1,
                                float beta2, float epsilon, int64_t n,
                                bool use_nesterov, cudaStream_t stream) {
  LaunchAdam<float, float>(var, m, v, static_cast<const float*>(grad), lr_t,
                           beta1, beta2, epsilon, n, use_nesterov, stream);
}

void LaunchApplyAdamMixed_Half(float* var, float* m, float* v, const void* grad,
                               float lr_t, float beta1, float beta2,
                               float epsilon, int64_t n, bool use_nesterov,
                               cudaStream_t stream) {
  LaunchAdam<float, __half>(var, m, v, static_cast<const __half*>(grad), lr_t,
                            beta1, beta2, epsilon, n, use_nesterov, stream);
}

void LaunchApplyAdamMixed_BFloat16(float* var, float* m, float* v,
                                   const void* grad, float lr_t, float beta1,
                                   float beta2, float epsilon, int64_t n,
                                   bool use_nesterov, cudaStream_t stream) {
  LaunchAdam<float, __nv_bfloat16>(var, m, v,
                                   static_cast<const __nv_bfloat16*>(grad),
                                   lr_t, beta1, beta2, epsilon, n, use_nesterov,
                                   stream);
}

}  // extern "C"
