// Shared device helpers for the sm_100a kernels: 128-bit vector packs, dtype
// widening/narrowing, cache-hinted loads and stores, launch sizing.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>

#include "trace.h"

namespace musa_b200 {

// B200: 148 SMs.  Grids of streaming kernels are sized as a multiple of the SM
// count of the device that is current at launch (queried once per device).
int SmCount();

// A pack of N values of T moved with one load/store instruction
// (N * sizeof(T) is 4, 8 or 16 bytes).
template <typename T, int N>
struct alignas(sizeof(T) * N) Pack {
  T v[N];
};

template <typename T>
struct VecWidth {  // elements of T in 128 bits
  static constexpr int value = 16 / sizeof(T);
};

__device__ __forceinline__ float ToF32(float x) { return x; }
__device__ __forceinline__ float ToF32(__half x) { return __half2float(x); }
__device__ __forceinline__ float ToF32(__nv_bfloat16 x) {
  return __bfloat162float(x);
}

template <typename T>
__device__ __forceinline__ T FromF32(float x);
template <>
__device__ __forceinline__ float FromF32<float>(float x) {
  return x;
}
template <>
__device__ __forceinline__ __half FromF32<__half>(float x) {
  return __float2half_rn(x);
}
template <>
__device__ __forceinline__ __nv_bfloat16 FromF32<__nv_bfloat16>(float x) {
  return __float2bfloat16_rn(x);
}

// Streaming (evict-first) accesses for data touched once per launch, and
// default-policy accesses for data that a following pass should find in L2.
template <typename P>
__device__ __forceinline__ P LoadStream(const P* p) {
  if constexpr (sizeof(P) == 16) {
    const float4 t = __ldcs(reinterpret_cast<const float4*>(p));
    return *reinterpret_cast<const P*>(&t);
  } else if constexpr (sizeof(P) == 8) {
    const float2 t = __ldcs(reinterpret_cast<const float2*>(p));
    return *reinterpret_cast<const P*>(&t);
  } else if constexpr (sizeof(P) == 4) {
    const float t = __ldcs(reinterpret_cast<const float*>(p));
    return *reinterpret_cast<const P*>(&t);
  } else {
    return *p;
  }
}

template <typename P>
__device__ __forceinline__ void StoreStream(P* p, const P& val) {
  if constexpr (sizeof(P) == 16) {
    __stcs(reinterpret_cast<float4*>(p), *reinterpret_cast<const float4*>(&val));
  } else if constexpr (sizeof(P) == 8) {
    __stcs(reinterpret_cast<float2*>(p), *reinterpret_cast<const float2*>(&val));
  } else if constexpr (sizeof(P) == 4) {
    __stcs(reinterpret_cast<float*>(p), *reinterpret_cast<const float*>(&val));
  } else {
    *p = val;
  }
}

template <typename P>
__device__ __forceinline__ P LoadKeep(const P* p) {
  if constexpr (sizeof(P) == 16) {
    const float4 t = __ldg(reinterpret_cast<const float4*>(p));
    return *reinterpret_cast<const P*>(&t);
  } else if constexpr (sizeof(P) == 8) {
    const float2 t = __ldg(reinterpret_cast<const float2*>(p));
    return *reinterpret_cast<const P*>(&t);
  } else if constexpr (sizeof(P) == 4) {
    const float t = __ldg(reinterpret_cast<const float*>(p));
    return *reinterpret_cast<const P*>(&t);
  } else {
    return *p;
  }
}

// ---- Packed fp32 pairs.  sm_100 executes add / mul / fma on two fp32 lanes
// per instruction (add.rn.f32x2, fma.rn.f32x2); each lane rounds exactly like
// the scalar instruction, so results are unchanged while the FP instruction
// count of the 16-bit kernels halves.
__device__ __forceinline__ float2 Add2(float2 a, float2 b) {
  return __fadd2_rn(a, b);
}
__device__ __forceinline__ float2 Mul2(float2 a, float2 b) {
  return __fmul2_rn(a, b);
}
__device__ __forceinline__ float2 Fma2(float2 a, float2 b, float2 c) {
  return __ffma2_rn(a, b, c);
}
__device__ __forceinline__ float2 Neg2(float2 a) {
  return make_float2(-a.x, -a.y);
}

// Widen a pack to kVec / 2 float pairs and back (kVec even).
template <int kVec>
__device__ __forceinline__ void WidenPack(const Pack<float, kVec>& p,
                                          float2 (&out)[kVec / 2]) {
#pragma unroll
  for (int i = 0; i < kVec / 2; ++i) out[i] = make_float2(p.v[2 * i], p.v[2 * i + 1]);
}
template <int kVec>
__device__ __forceinline__ void WidenPack(const Pack<__nv_bfloat16, kVec>& p,
                                          float2 (&out)[kVec / 2]) {
  // bf16 is the upper half of an fp32: one shift or mask per element.
  const uint32_t* w = reinterpret_cast<const uint32_t*>(&p);
#pragma unroll
  for (int i = 0; i < kVec / 2; ++i) {
    out[i] = make_float2(__uint_as_float(w[i] << 16),
                         __uint_as_float(w[i] & 0xffff0000u));
  }
}
template <int kVec>
__device__ __forceinline__ void WidenPack(const Pack<__half, kVec>& p,
                                          float2 (&out)[kVec / 2]) {
  const __half2* w = reinterpret_cast<const __half2*>(&p);
#pragma unroll
  for (int i = 0; i < kVec / 2; ++i) out[i] = __half22float2(w[i]);
}
template <int kVec>
__device__ __forceinline__ void NarrowPack(const float2 (&in)[kVec / 2],
                                           Pack<float, kVec>& p) {
#pragma unroll
  for (int i = 0; i < kVec / 2; ++i) {
    p.v[2 * i] = in[i].x;
    p.v[2 * i + 1] = in[i].y;
  }
}
template <int kVec>
__device__ __forceinline__ void NarrowPack(const float2 (&in)[kVec / 2],
                                           Pack<__nv_bfloat16, kVec>& p) {
  __nv_bfloat162* w = reinterpret_cast<__nv_bfloat162*>(&p);
#pragma unroll
  for (int i = 0; i < kVec / 2; ++i) w[i] = __floats2bfloat162_rn(in[i].x, in[i].y);
}
template <int kVec>
__device__ __forceinline__ void NarrowPack(const float2 (&in)[kVec / 2],
                                           Pack<__half, kVec>& p) {
  __half2* w = reinterpret_cast<__half2*>(&p);
#pragma unroll
  for (int i = 0; i < kVec / 2; ++i) w[i] = __floats2half2_rn(in[i].x, in[i].y);
}

// ---- Programmatic dependent launch.  Kernels of one launcher form a chain
// on the stream; launched with the programmatic-serialization attribute, the
// next kernel's CTAs are scheduled while the current kernel drains, and its
// GridDepWait() returns once the previous kernel has completed and its writes
// are visible.  Every kernel calls GridDepWait() before its first global
// access and GridDepLaunch() right after, so a dependent never starts before
// its producer has itself seen all of its inputs.
__device__ __forceinline__ void GridDepWait() {
  asm volatile("griddepcontrol.wait;" ::: "memory");
}
__device__ __forceinline__ void GridDepLaunch() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

template <typename... KArgs, typename... Args>
inline cudaError_t LaunchChained(bool programmatic, void (*kernel)(KArgs...),
                                 dim3 grid, dim3 block, size_t smem,
                                 cudaStream_t stream, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = programmatic ? 1 : 0;
  CountKernelLaunch();
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// Thread-block clusters along grid.y (`cluster_y` CTAs share distributed
// shared memory; grid.y is a multiple of it).  cluster_y == 1 is a plain
// launch.
inline void ClusterConfig(cudaLaunchConfig_t* cfg, cudaLaunchAttribute* attr, bool programmatic,
                          int cluster_y, dim3 grid, dim3 block, size_t smem,
                          cudaStream_t stream) {
  *cfg = cudaLaunchConfig_t{};
  cfg->gridDim = grid;
  cfg->blockDim = block;
  cfg->dynamicSmemBytes = smem;
  cfg->stream = stream;
  int n = 0;
  if (programmatic) {
    attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[n].val.programmaticStreamSerializationAllowed = 1;
    ++n;
  }
  if (cluster_y > 1) {
    attr[n].id = cudaLaunchAttributeClusterDimension;
    attr[n].val.clusterDim.x = 1;
    attr[n].val.clusterDim.y = static_cast<unsigned>(cluster_y);
    attr[n].val.clusterDim.z = 1;
    ++n;
  }
  cfg->attrs = attr;
  cfg->numAttrs = n;
}

template <typename... KArgs, typename... Args>
inline cudaError_t LaunchClustered(bool programmatic, int cluster_y, void (*kernel)(KArgs...),
                                   dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                   Args&&... args) {
  cudaLaunchConfig_t cfg;
  cudaLaunchAttribute attr[2];
  ClusterConfig(&cfg, attr, programmatic, cluster_y, grid, block, smem, stream);
  CountKernelLaunch();
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// Cluster-wide barrier (all threads of all CTAs of the cluster; a superset of
// __syncthreads) and a 32-bit load from the shared memory of CTA `rank` of
// the cluster at the address `local` has in this CTA's window.
__device__ __forceinline__ void ClusterSync() {
  asm volatile(
      "barrier.cluster.arrive.release.aligned;\n"
      "barrier.cluster.wait.acquire.aligned;" ::
          : "memory");
}
__device__ __forceinline__ unsigned ClusterCtaRank() {
  unsigned r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ float LoadClusterF32(const float* local, unsigned rank) {
  const unsigned addr = static_cast<unsigned>(__cvta_generic_to_shared(local));
  unsigned remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(addr), "r"(rank));
  float v;
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(remote) : "memory");
  return v;
}

// One value per device and call site, computed on the first use on that
// device with that device current (function attributes and occupancy are
// per-device state, and one process may drive several GPUs).  The table is a
// zero-initialised static of the call site; 0 means "not computed yet", so
// `init` returns non-zero values.
constexpr int kMaxDevices = 64;
template <typename Init>
inline int PerDevice(std::atomic<int>* table, Init init) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    cudaGetLastError();
    return init();
  }
  int v = table[dev].load(std::memory_order_acquire);
  if (v == 0) {
    v = init();
    table[dev].store(v, std::memory_order_release);
  }
  return v;
}

inline bool Aligned16(const void* p) {
  return (reinterpret_cast<uintptr_t>(p) & 15u) == 0;
}

inline int64_t CeilDiv(int64_t a, int64_t b) { return (a + b - 1) / b; }

}  // namespace musa_b200
