// Device-side pieces of the peer-memory exchange (see exchange.cu for the
// protocol), shared with the kernels that run an exchange inside another
// kernel: the BatchNorm finalize kernel pushes and gathers the per-channel
// values of its own channels, which saves the exchange kernel and its two
// kernel boundaries in every cross-replica BatchNorm pass.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace musa_b200 {

constexpr int kMaxWorld = 16;
constexpr int kExchangeThreads = 512;
// Polls of one cell before a wait gives up (each poll is a load from local
// memory plus a short sleep, about a microsecond: a second in total).
constexpr long long kSpinLimit = 1LL << 20;

struct ExchangeDev {
  int rank;
  int world;
  long long slot_floats;
  unsigned long long* cells[kMaxWorld];  // cell buffer of every replica (peer-mapped)
  unsigned* epoch;          // local
  int* status;              // local: 0 ok, 1 + q when replica q never arrived
};

__device__ __forceinline__ unsigned long long LoadCell(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}

__device__ __forceinline__ void StoreCell(unsigned long long* p, unsigned long long v) {
  asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}

__device__ __forceinline__ unsigned long long MakeCell(float value, unsigned epoch) {
  return (static_cast<unsigned long long>(epoch) << 32) | __float_as_uint(value);
}
__device__ __forceinline__ unsigned CellEpoch(unsigned long long cell) {
  return static_cast<unsigned>(cell >> 32);
}
__device__ __forceinline__ float CellValue(unsigned long long cell) {
  return __uint_as_float(static_cast<unsigned>(cell & 0xffffffffULL));
}

enum ExchangeMode { kExchangeSum = 0, kExchangeMoments = 1 };

// Waits (bounded) until the cell of replica q carries `epoch`.  `dead` is the
// CTA's shared mask of replicas nobody waits for any more.
__device__ __forceinline__ unsigned long long AwaitCell(const unsigned long long* cell,
                                                        unsigned epoch, int q, unsigned* dead,
                                                        int* status) {
  unsigned long long got = LoadCell(cell);
  long long polls = 0;
  while (CellEpoch(got) != epoch) {
    if ((*reinterpret_cast<volatile unsigned*>(dead) >> q) & 1u) break;
    if (++polls > kSpinLimit) {
      atomicOr(dead, 1u << q);
      atomicCAS(status, 0, 1 + q);
      break;
    }
    __nanosleep(40);
    got = LoadCell(cell);
  }
  return got;
}


// One channel's pair of values inside a kernel that owns that channel: pushes
// {v0, v1} (cells c and channels + c; the thread of channel 0 also pushes
// `count` into cell 2 * channels) to every replica, gathers the replicas'
// pairs from local memory (bounded waits) and combines them in rank order:
//   kMoments: v0 = mean, v1 = sum of squared deviations, count = rows ->
//             moments of the union (count-weighted mean, Chan's formula);
//   else    : plain sums (count is neither sent nor read, *total = 0).
// All cells are requested at once (kW replicas: one L2 round trip when every
// replica has already delivered); only the ones that have not arrived are
// polled.
template <bool kMoments, int kW>
__device__ __forceinline__ void ExchangeChannelPairW(const ExchangeDev& x, unsigned epoch,
                                                     int channels, int c, float v0, float v1,
                                                     float count, unsigned* dead, float* r0,
                                                     float* r1, float* total) {
  const int world = x.world;
  const int slot = static_cast<int>(epoch & 1u);
  const long long slot_base = static_cast<long long>(slot) * world * x.slot_floats;
  const long long mine = slot_base + static_cast<long long>(x.rank) * x.slot_floats;
  const unsigned long long c0 = MakeCell(v0, epoch), c1 = MakeCell(v1, epoch);
#pragma unroll
  for (int p = 0; p < kW; ++p) {
    if (p < world && p != x.rank) {   // the own contribution stays in registers
      unsigned long long* dst = x.cells[p] + mine;
      StoreCell(dst + c, c0);
      StoreCell(dst + channels + c, c1);
      if (kMoments && c == 0) StoreCell(dst + 2 * channels, MakeCell(count, epoch));
    }
  }
  const unsigned long long* local = x.cells[x.rank] + slot_base;
  unsigned long long g0[kW], g1[kW], gn[kW];
#pragma unroll
  for (int q = 0; q < kW; ++q) {
    if (q < world) {
      if (q == x.rank) {
        g0[q] = c0;
        g1[q] = c1;
        gn[q] = MakeCell(count, epoch);
      } else {
        const unsigned long long* base = local + static_cast<long long>(q) * x.slot_floats;
        g0[q] = LoadCell(base + c);
        g1[q] = LoadCell(base + channels + c);
        gn[q] = kMoments ? LoadCell(base + 2 * channels) : 0ULL;
      }
    }
  }
#pragma unroll
  for (int q = 0; q < kW; ++q) {
    if (q < world && q != x.rank) {
      const unsigned long long* base = local + static_cast<long long>(q) * x.slot_floats;
      if (CellEpoch(g0[q]) != epoch) g0[q] = AwaitCell(base + c, epoch, q, dead, x.status);
      if (CellEpoch(g1[q]) != epoch) {
        g1[q] = AwaitCell(base + channels + c, epoch, q, dead, x.status);
      }
      if (kMoments && CellEpoch(gn[q]) != epoch) {
        gn[q] = AwaitCell(base + 2 * channels, epoch, q, dead, x.status);
      }
    }
  }
  if (!kMoments) {
    float t0 = 0.0f, t1 = 0.0f;
#pragma unroll
    for (int q = 0; q < kW; ++q) {
      if (q < world) {
        t0 += CellValue(g0[q]);
        t1 += CellValue(g1[q]);
      }
    }
    *r0 = t0;
    *r1 = t1;
    *total = 0.0f;
    return;
  }
  double n_total = 0.0, mean = 0.0;
#pragma unroll
  for (int q = 0; q < kW; ++q) {
    if (q < world) {
      const double n_q = static_cast<double>(CellValue(gn[q]));
      n_total += n_q;
      mean += n_q * static_cast<double>(CellValue(g0[q]));
    }
  }
  mean *= n_total > 0.0 ? 1.0 / n_total : 0.0;
  double m2 = 0.0;
#pragma unroll
  for (int q = 0; q < kW; ++q) {
    if (q < world) {
      const double d = static_cast<double>(CellValue(g0[q])) - mean;
      m2 += static_cast<double>(CellValue(g1[q])) +
            static_cast<double>(CellValue(gn[q])) * d * d;
    }
  }
  *r0 = static_cast<float>(mean);
  *r1 = static_cast<float>(m2);
  *total = static_cast<float>(n_total);
}

template <bool kMoments>
__device__ __forceinline__ void ExchangeChannelPair(const ExchangeDev& x, unsigned epoch,
                                                    int channels, int c, float v0, float v1,
                                                    float count, unsigned* dead, float* r0,
                                                    float* r1, float* total) {
  switch (x.world) {
    case 1:
      ExchangeChannelPairW<kMoments, 1>(x, epoch, channels, c, v0, v1, count, dead, r0, r1, total);
      break;
    case 2:
      ExchangeChannelPairW<kMoments, 2>(x, epoch, channels, c, v0, v1, count, dead, r0, r1, total);
      break;
    case 3:
    case 4:
      ExchangeChannelPairW<kMoments, 4>(x, epoch, channels, c, v0, v1, count, dead, r0, r1, total);
      break;
    case 5:
    case 6:
    case 7:
    case 8:
      ExchangeChannelPairW<kMoments, 8>(x, epoch, channels, c, v0, v1, count, dead, r0, r1, total);
      break;
    default:
      ExchangeChannelPairW<kMoments, kMaxWorld>(x, epoch, channels, c, v0, v1, count, dead, r0, r1,
                                                total);
  }
}

// Device context of an exchange handle (exchange.cu): the table that kernels
// take, the capacity of a slot in floats, and the device address of the epoch
// counter (a kernel that precedes an in-kernel exchange advances it).
const ExchangeDev* ExchangeDeviceContext(void* handle, long long* slot_floats,
                                         unsigned** epoch);

}  // namespace musa_b200
