// Shared device helpers for the sm_100a kernels: 128-bit vector packs, dtype
// widening/narrowing, cache-hinted loads and stores, launch sizing.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

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

inline bool Aligned16(const void* p) {
  return (reinterpret_cast<uintptr_t>(p) & 15u) == 0;
}

inline int64_t CeilDiv(int64_t a, int64_t b) { return (a + b - 1) / b; }

}  // namespace musa_b200
