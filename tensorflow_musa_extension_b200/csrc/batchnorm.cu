// FusedBatchNorm forward / gradient for sm_100a.
//
// Data layout.  x, y, dy, dx are [outer, channels, inner]; NHWC is
// (outer = N*H*W, inner = 1), NCHW is (outer = N, inner = H*W).  Statistics
// are fp32 [channels] for every x dtype.
//
// Structure.  Both directions are "two per-channel sums over all rows, then an
// element-wise pass":
//   forward : S1 = sum(x - K), S2 = sum((x - K)^2)      (K: per-channel shift)
//   gradient: S1 = sum(dy),    S2 = sum(dy * (x - mean))
// Level 1 (stats kernel): each thread owns one 128-bit channel pack and walks
// rows, keeping 2 * kVec fp32 partials in registers; a CTA folds its row
// lanes through shared memory and writes one partial row [2, C] to the
// workspace.  Level 2 (finalize kernel): 8 channels x 128 partial-lanes per
// CTA, fp64 accumulation, then the per-channel outputs.  The apply kernel
// re-reads x (and dy) with the default L2 policy, walking the rows in the
// opposite order of the stats kernel so that it meets the most recently read
// lines first, and streams y / dx out with evict-first stores.
//
// The forward sums are taken about a per-channel shift K (the channel's first
// element) so that the variance does not cancel when |mean| >> std; the
// gradient sums are centred on the batch mean by construction.
//
// Output conventions follow the op this replaces
// (musa_ext/kernels/nn/musa_fused_batchnorm_op.cc:126-170: batch_var is
// Bessel-corrected, saved_var is the population variance, no correction when
// there is one value per channel; :265-277: the gradient receives a variance
// and turns it into 1/sqrt(var + eps)).
#include <atomic>
#include <mutex>

#include "common.cuh"
#include "exchange_dev.cuh"
#include "trace.h"
#include "tuning.h"
#include "../../include/musa_plugin_kernels.h"

namespace musa_b200 {
namespace {

constexpr int kThreads = 256;
// Upper bound of fp32 partials in the workspace (level-1 output).
constexpr int64_t kMaxPartialFloats = 1 << 20;
constexpr int64_t kMaxSplits = 4096;

// ------------------------------------------------------------- planning --

inline int Pow2Ceil(int64_t v) {
  int p = 1;
  while (p < v && p < kThreads) p <<= 1;
  return p;
}

// Largest number of row splits the workspace has to hold for `rows` rows of
// `channels` channels, whatever vector width or grid the launch picks.
inline int64_t MaxSplits(int64_t rows, int64_t channels) {
  int64_t by_ws = kMaxPartialFloats / (2 * channels);
  if (by_ws < 1) by_ws = 1;
  int64_t s = rows < 1 ? 1 : rows;
  if (s > kMaxSplits) s = kMaxSplits;
  if (s > by_ws) s = by_ws;
  return s;
}

struct Plan {
  int tx, ty;      // thread block = tx channel packs x ty row lanes
  int gx;          // column blocks
  int gy;          // row splits (= partial rows written by the stats kernel)
  int64_t rows_per_cta;
};

// Channel packs per column block of a channels-last launch.
inline int PlanTx(int64_t cv, int max_tx) {
  const int tx = Pow2Ceil(cv);
  return tx > max_tx ? max_tx : tx;
}

// Channels-last plan.  `cv` = channel packs per row.
// `resident`: CTAs of this kernel that fit on one SM; the grid is one full
// wave of them (a second, partly filled wave would idle SMs at the end).
inline Plan PlanLast(int64_t rows, int64_t channels, int64_t cv, int unroll,
                     bool cap_by_workspace, int resident, int max_tx = kThreads) {
  Plan p;
  p.tx = PlanTx(cv, max_tx);
  p.ty = kThreads / p.tx;
  p.gx = static_cast<int>(CeilDiv(cv, p.tx));
  int per_sm = GetTuning(cap_by_workspace ? kTuneBnCtasPerSm : kTuneBnApplyCtasPerSm);
  if (per_sm < 1) per_sm = resident > 0 ? resident : 4;
  int64_t target = static_cast<int64_t>(SmCount()) * per_sm / p.gx;
  if (target < 1) target = 1;
  // Do not split below one unrolled sweep of the row lanes.
  int64_t max_useful = CeilDiv(rows, static_cast<int64_t>(p.ty) * unroll);
  if (max_useful < 1) max_useful = 1;
  int64_t gy = target < max_useful ? target : max_useful;
  if (cap_by_workspace) {
    const int64_t cap = MaxSplits(rows, channels);
    if (gy > cap) gy = cap;
  }
  if (gy > 65535) gy = 65535;
  p.rows_per_cta = CeilDiv(rows, gy);
  // Keep CTA row ranges a multiple of ty so that lanes stay aligned.
  p.rows_per_cta = CeilDiv(p.rows_per_cta, p.ty) * p.ty;
  p.gy = static_cast<int>(CeilDiv(rows, p.rows_per_cta));
  if (p.gy < 1) p.gy = 1;
  // Interleaved row tiles do not need whole row ranges per CTA (the kernels
  // take the number of row splits from the grid): keep the full wave.
  if (GetTuning(kTuneBnFullWave) != 0 && GetTuning(kTuneBnInterleave) != 0) {
    p.gy = static_cast<int>(gy);
  }
  return p;
}

// ------------------------------------------------------------ level 1 ----

// Cross-replica passes: the finalize kernel that follows a statistics kernel
// runs a peer-memory exchange whose cells are tagged with an epoch.  The
// statistics kernel advances the device-side epoch counter (one thread, once
// it may touch memory), so that every CTA of the finalize kernel reads the
// same, already advanced value and nothing has to count CTAs afterwards.
__device__ __forceinline__ void BumpEpoch(unsigned* epoch, int linear_tid) {
  if (epoch != nullptr && blockIdx.x == 0 && blockIdx.y == 0 && linear_tid == 0) {
    *epoch = *epoch + 1u;
  }
}

enum Mode { kFwd = 0, kGrad = 1 };

// Channels-last stats.  Grid (gx, gy), block (tx, ty).
template <typename T, int kVec, int kUnroll, int kMode>
__global__ void __launch_bounds__(kThreads)
    BnStatsLastKernel(const T* __restrict__ x, const T* __restrict__ dy,
                      const float* __restrict__ mean,
                      float* __restrict__ partial, int64_t rows, int64_t cv,
                      int64_t channels, int64_t rows_per_cta, bool keep,
                      unsigned* epoch_bump) {
  using P = Pack<T, kVec>;
  GridDepWait();
  GridDepLaunch();
  BumpEpoch(epoch_bump, threadIdx.y * blockDim.x + threadIdx.x);
  const int tx = threadIdx.x, ty = threadIdx.y;
  const int TX = blockDim.x, TY = blockDim.y;
  const int64_t col = static_cast<int64_t>(blockIdx.x) * TX + tx;
  const bool active = col < cv;
  const int64_t r0 = static_cast<int64_t>(blockIdx.y) * rows_per_cta;
  int64_t r1 = r0 + rows_per_cta;
  if (r1 > rows) r1 = rows;

  float shift[kVec];
  float s1[kVec], s2[kVec];
#pragma unroll
  for (int e = 0; e < kVec; ++e) {
    s1[e] = 0.0f;
    s2[e] = 0.0f;
    shift[e] = 0.0f;
  }

  if (active) {
    if constexpr (kMode == kFwd) {
      const P first = LoadKeep(reinterpret_cast<const P*>(x) + col);
#pragma unroll
      for (int e = 0; e < kVec; ++e) shift[e] = ToF32(first.v[e]);
    } else {
#pragma unroll
      for (int e = 0; e < kVec; ++e) shift[e] = mean[col * kVec + e];
    }
    const P* xp = reinterpret_cast<const P*>(x) + col;
    const P* dp = reinterpret_cast<const P*>(dy) + col;
    int64_t r = r0 + ty;
    const int64_t step = static_cast<int64_t>(TY) * kUnroll;
    // Full sweeps: kUnroll independent loads per stream in flight.
    for (; r + static_cast<int64_t>(kUnroll - 1) * TY < r1; r += step) {
      P px[kUnroll];
      P pd[kUnroll];
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        const int64_t off = (r + static_cast<int64_t>(u) * TY) * cv;
        px[u] = keep ? LoadKeep(xp + off) : LoadStream(xp + off);
        if constexpr (kMode == kGrad) {
          pd[u] = keep ? LoadKeep(dp + off) : LoadStream(dp + off);
        }
      }
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
#pragma unroll
        for (int e = 0; e < kVec; ++e) {
          const float d = ToF32(px[u].v[e]) - shift[e];
          if constexpr (kMode == kFwd) {
            s1[e] += d;
            s2[e] = fmaf(d, d, s2[e]);
          } else {
            const float g = ToF32(pd[u].v[e]);
            s1[e] += g;
            s2[e] = fmaf(g, d, s2[e]);
          }
        }
      }
    }
    for (; r < r1; r += TY) {
      const int64_t off = r * cv;
      const P px = keep ? LoadKeep(xp + off) : LoadStream(xp + off);
      P pd;
      if constexpr (kMode == kGrad) {
        pd = keep ? LoadKeep(dp + off) : LoadStream(dp + off);
      }
#pragma unroll
      for (int e = 0; e < kVec; ++e) {
        const float d = ToF32(px.v[e]) - shift[e];
        if constexpr (kMode == kFwd) {
          s1[e] += d;
          s2[e] = fmaf(d, d, s2[e]);
        } else {
          const float g = ToF32(pd.v[e]);
          s1[e] += g;
          s2[e] = fmaf(g, d, s2[e]);
        }
      }
    }
  }

  // Fold the ty row lanes.  red[(s * kVec + e)][ty][tx]
  __shared__ float red[2 * kVec * kThreads];
  if (TY > 1) {
#pragma unroll
    for (int e = 0; e < kVec; ++e) {
      red[((0 * kVec + e) * TY + ty) * TX + tx] = s1[e];
      red[((1 * kVec + e) * TY + ty) * TX + tx] = s2[e];
    }
    __syncthreads();
    const int tid = ty * TX + tx;
    const int n_out = 2 * kVec * TX;
    for (int o = tid; o < n_out; o += kThreads) {
      const int otx = o % TX;
      const int se = o / TX;  // s * kVec + e
      float acc = 0.0f;
      for (int j = 0; j < TY; ++j) acc += red[(se * TY + j) * TX + otx];
      const int64_t ocol = static_cast<int64_t>(blockIdx.x) * TX + otx;
      if (ocol < cv) {
        const int s = se / kVec, e = se % kVec;
        partial[(static_cast<int64_t>(blockIdx.y) * 2 + s) * channels +
                ocol * kVec + e] = acc;
      }
    }
  } else if (active) {
#pragma unroll
    for (int e = 0; e < kVec; ++e) {
      partial[(static_cast<int64_t>(blockIdx.y) * 2 + 0) * channels +
              col * kVec + e] = s1[e];
      partial[(static_cast<int64_t>(blockIdx.y) * 2 + 1) * channels +
              col * kVec + e] = s2[e];
    }
  }
}

// ---- Per-channel epilogues shared by the finalize kernel and the in-kernel
// finalize of the pipelined statistics kernel.
struct FinalizeArgs {
  const float* partial;  // [splits, 2, C] level-1 output (or NULL with sums)
  int splits;
  int64_t channels;
  double count;          // values per channel behind the sums (all replicas)
  double inv_count;      // 1 / count
  double bessel;         // count / (count - 1), or 1 when count <= 1
  // forward
  const void* x_first;   // tensor base: the shift K is re-read from it
  int x_dtype;
  int64_t shift_stride;  // elements between consecutive channels' K
  const float* est_mean;
  const float* est_var;
  float* batch_mean;
  float* batch_var;
  float* saved_mean;
  float* saved_var;
  float exp_avg_factor;
  // gradient
  const float* variance;
  float* dscale;
  float* doffset;
  float epsilon;
  // both: totals for the apply pass / the all-reduce
  float* sums;           // [2, C] or NULL
  float* count_out;      // optional: receives `count` (rides in the all-reduce)
  // Cross-replica: when set, the finalize kernel exchanges its channels' pair
  // with the other replicas itself (moments are merged, gradient sums added)
  // and everything it writes is the result over all replicas.
  const ExchangeDev* xchg;
  unsigned* xchg_epoch;   // the exchange's epoch counter (advanced by the statistics kernel)
};

__device__ __forceinline__ float LoadAsF32(const void* base, int dtype,
                                           int64_t i) {
  if (dtype == MUSA_DT_F32) return static_cast<const float*>(base)[i];
  if (dtype == MUSA_DT_F16) return __half2float(static_cast<const __half*>(base)[i]);
  return __bfloat162float(static_cast<const __nv_bfloat16*>(base)[i]);
}

__device__ __forceinline__ void WriteFwdStats(const FinalizeArgs& a, int64_t c,
                                              double mean, double var) {
  if (var < 0.0) var = 0.0;
  // bessel = R / (R - 1), or 1 when there is one value per channel; taken on
  // the host (an fp64 divide per thread is not free on the device).
  const double unbiased = var * a.bessel;
  if (a.saved_mean) a.saved_mean[c] = static_cast<float>(mean);
  if (a.saved_var) a.saved_var[c] = static_cast<float>(var);
  const double f = static_cast<double>(a.exp_avg_factor);
  double bm = mean, bv = unbiased;
  if (a.exp_avg_factor != 1.0f && a.est_mean != nullptr &&
      a.est_var != nullptr) {
    bm = (1.0 - f) * static_cast<double>(a.est_mean[c]) + f * mean;
    bv = (1.0 - f) * static_cast<double>(a.est_var[c]) + f * unbiased;
  }
  if (a.batch_mean) a.batch_mean[c] = static_cast<float>(bm);
  if (a.batch_var) a.batch_var[c] = static_cast<float>(bv);
}

inline void SetCount(FinalizeArgs* f, double count) {
  f->count = count;
  f->inv_count = 1.0 / count;
  f->bessel = count > 1.0 ? count / (count - 1.0) : 1.0;
}


// What the second level of the reduction writes.
enum TailKind {
  kTailFwdStats = 0,    // mean / variance outputs of the training forward
  kTailFwdSums = 1,     // raw [sum x, sum x^2] (+ count)
  kTailGrad = 2,        // [sum dy, sum dy (x - mean)], dscale, doffset
  kTailFwdMoments = 3,  // [mean, sum (x - mean)^2] (+ count) of the local rows
};

// ---- Pipelined channels-last stats (128-bit packs only).
//
// Same mapping as BnStatsLastKernel, but the row stream is staged through
// shared memory with per-thread asynchronous 16-byte copies (cp.async): every
// thread owns kStages * kStreams * kU private 16-byte slots, keeps
// (kStages - 1) * kStreams * kU copies in flight and reads back only its own
// slots, so no barrier is needed in the loop and the bytes in flight per SM
// (~150 KB at 3 CTAs) no longer depend on registers.  With register-held loads
// the kernel was latency-bound at about half of the HBM rate.
__device__ __forceinline__ void CpAsync16(void* smem_dst, const void* gmem_src) {
  const unsigned dst = static_cast<unsigned>(__cvta_generic_to_shared(smem_dst));
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(dst),
               "l"(gmem_src)
               : "memory");
}
// L2 eviction-priority policies.  The statistics pass marks the lines it
// brings in "evict last" when the tensor is small enough to stay in L2 until
// the element-wise pass re-reads it; that pass marks them "evict first" as it
// consumes them.
__device__ __forceinline__ uint64_t PolicyEvictLast() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(p));
  return p;
}
__device__ __forceinline__ uint64_t PolicyEvictNormal() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_normal.b64 %0, 1.0;" : "=l"(p));
  return p;
}
__device__ __forceinline__ uint64_t PolicyEvictFirst() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
  return p;
}
__device__ __forceinline__ void CpAsync16Hint(void* smem_dst,
                                              const void* gmem_src,
                                              uint64_t policy) {
  const unsigned dst = static_cast<unsigned>(__cvta_generic_to_shared(smem_dst));
  asm volatile(
      "cp.async.cg.shared.global.L2::cache_hint [%0], [%1], 16, %2;\n" ::"r"(dst),
      "l"(gmem_src), "l"(policy)
      : "memory");
}
template <typename P>
__device__ __forceinline__ P LoadHint16(const P* p, uint64_t policy) {
  static_assert(sizeof(P) == 16, "128-bit packs only");
  uint4 r;
  asm volatile("ld.global.nc.L2::cache_hint.v4.u32 {%0, %1, %2, %3}, [%4], %5;"
               : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
               : "l"(p), "l"(policy));
  return *reinterpret_cast<const P*>(&r);
}
__device__ __forceinline__ void CpAsyncCommit() {
  asm volatile("cp.async.commit_group;\n" ::: "memory");
}
template <int kPending>
__device__ __forceinline__ void CpAsyncWait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(kPending) : "memory");
}

template <int kMode, int kStagesT>
struct StatsPipe {
  static constexpr int kStages = kStagesT;
  static constexpr int kStreams = kMode == 0 ? 1 : 2;
  static constexpr int kU = kMode == 0 ? 4 : 2;  // rows per stage and stream
  static constexpr int kSlots = kStages * kStreams * kU;
  static constexpr int kSmemBytes = kSlots * 256 * 16;
};

// The loop is written for instruction count: measured, the forward form needs
// about 2.7 instructions per clock and SM to keep up with HBM, so every
// instruction per 16-byte pack beyond the arithmetic (convert, shift, two
// accumulations) costs bandwidth.  Whole stages run without bounds checks
// (the stage loop is not unrolled over the ring: the slot is a run-time
// offset), source pointers advance by additions, and the rows that do not
// fill a stage are read with plain loads at the end.
template <typename T, int kMode, int kStagesT>
__global__ void __launch_bounds__(kThreads)
    BnStatsPipeKernel(const T* __restrict__ x, const T* __restrict__ dy,
                      const float* __restrict__ mean,
                      float* __restrict__ partial, int64_t rows, int64_t cv,
                      int64_t channels, int64_t rows_per_cta, float keep_fraction,
                      bool drop_rest, bool interleave, unsigned* epoch_bump, int fold) {
  constexpr int kVec = VecWidth<T>::value;
  using P = Pack<T, kVec>;
  GridDepWait();
  GridDepLaunch();
  BumpEpoch(epoch_bump, threadIdx.y * blockDim.x + threadIdx.x);
  using Cfg = StatsPipe<kMode, kStagesT>;
  constexpr int kStages = Cfg::kStages, kU = Cfg::kU, kStreams = Cfg::kStreams;
  constexpr int kStageSlots = kStreams * kU;           // 16-byte slots per thread and stage
  extern __shared__ uint4 pipe_smem[];
  const int tx = threadIdx.x, ty = threadIdx.y;
  const int TX = blockDim.x, TY = blockDim.y;
  const int tid = ty * TX + tx;
  const int64_t col = static_cast<int64_t>(blockIdx.x) * TX + tx;
  const bool active = col < cv;
  const int64_t r0 = static_cast<int64_t>(blockIdx.y) * rows_per_cta;
  int64_t r1 = r0 + rows_per_cta;
  if (r1 > rows) r1 = rows;

  // Channel pairs: accumulators and the negated shift as packed fp32 pairs.
  constexpr int kPairs = kVec / 2;
  float2 nshift[kPairs], a1[kPairs], a2[kPairs];
#pragma unroll
  for (int q = 0; q < kPairs; ++q) {
    a1[q] = make_float2(0.0f, 0.0f);
    a2[q] = make_float2(0.0f, 0.0f);
    nshift[q] = make_float2(0.0f, 0.0f);
  }

  auto accumulate = [&](const uint4& rx, const uint4& rd) {
    float2 xv[kPairs], gv[kPairs];
    WidenPack<kVec>(*reinterpret_cast<const P*>(&rx), xv);
    if constexpr (kMode == kGrad) WidenPack<kVec>(*reinterpret_cast<const P*>(&rd), gv);
#pragma unroll
    for (int q = 0; q < kPairs; ++q) {
      const float2 d = Add2(xv[q], nshift[q]);
      if constexpr (kMode == kFwd) {
        a1[q] = Add2(a1[q], d);
        a2[q] = Fma2(d, d, a2[q]);
      } else {
        a1[q] = Add2(a1[q], gv[q]);
        a2[q] = Fma2(gv[q], d, a2[q]);
      }
    }
  };

  if (active) {
    if constexpr (kMode == kFwd) {
      const P first = LoadKeep(reinterpret_cast<const P*>(x) + col);
      WidenPack<kVec>(first, nshift);
#pragma unroll
      for (int q = 0; q < kPairs; ++q) nshift[q] = Neg2(nshift[q]);
    } else {
#pragma unroll
      for (int q = 0; q < kPairs; ++q) {
        nshift[q] = make_float2(-mean[col * kVec + 2 * q],
                                -mean[col * kVec + 2 * q + 1]);
      }
    }
    // This thread's rows: r0 + ty + j * TY, j = 0 .. n_j - 1 (32-bit counters:
    // a CTA never owns 2^31 rows), in n_full whole stages of kU rows and a
    // remainder.
    // Two row maps.  Contiguous: CTA b owns rows [r0, r1).  Interleaved: the
    // rows are cut into tiles of kU * TY rows (one stage of one CTA) and CTA b
    // takes tiles b, b + G, b + 2G ...: at any moment all CTAs read inside one
    // window of G tiles that moves through the tensor, instead of G streams
    // spread over all of it (fewer DRAM pages open at once).
    const int64_t row_bytes = static_cast<int64_t>(TY) * cv * 16;   // one row step
    int n_full, rem;
    int64_t stage_bytes, first_row;
    int keep_from_tile = 0, tile_step = 1, tile_first = 0;   // global tile of stage s: first + s * step
    if (interleave) {
      const int64_t tile_rows = static_cast<int64_t>(kU) * TY;
      const int64_t tiles = (rows + tile_rows - 1) / tile_rows;
      const int64_t G = gridDim.y, b = blockIdx.y;
      const int64_t mine = b < tiles ? (tiles - 1 - b) / G + 1 : 0;
      const bool owns_last = mine > 0 && b + (mine - 1) * G == tiles - 1;
      const int64_t last_rows = rows - (tiles - 1) * tile_rows;     // rows of the last tile
      if (owns_last && last_rows != tile_rows) {
        n_full = static_cast<int>(mine - 1);
        rem = last_rows > ty ? static_cast<int>((last_rows - ty + TY - 1) / TY) : 0;
      } else {
        n_full = static_cast<int>(mine);
        rem = 0;
      }
      stage_bytes = row_bytes * kU * G;
      first_row = b * tile_rows + ty;
      tile_first = static_cast<int>(b);
      tile_step = static_cast<int>(G);
      keep_from_tile =
          keep_fraction >= 1.0f ? 0
          : keep_fraction <= 0.0f
              ? static_cast<int>(tiles) + 1
              : static_cast<int>(tiles) -
                    static_cast<int>(static_cast<float>(tiles) * keep_fraction);
    } else {
      const int n_rows = static_cast<int>(r1 - r0);
      const int n_j = n_rows > ty ? (n_rows - ty + TY - 1) / TY : 0;
      n_full = n_j / kU;
      rem = n_j - n_full * kU;
      stage_bytes = row_bytes * kU;
      first_row = r0 + ty;
      keep_from_tile =
          keep_fraction >= 1.0f ? 0
          : keep_fraction <= 0.0f
              ? n_full + 1
              : n_full - static_cast<int>(static_cast<float>(n_full) * keep_fraction);
    }
    const char* xi =
        reinterpret_cast<const char*>(reinterpret_cast<const P*>(x) + col + first_row * cv);
    const char* di =
        reinterpret_cast<const char*>(reinterpret_cast<const P*>(dy) + col + first_row * cv);
    const unsigned my = static_cast<unsigned>(__cvta_generic_to_shared(pipe_smem + tid));
    constexpr unsigned kSlotBytes = kThreads * 16;                  // between a thread's slots
    constexpr unsigned kStageBytes = kStageSlots * kSlotBytes;
    // L2 retention for the element-wise pass that follows: the LAST
    // keep_fraction of this thread's stages (contiguous map) or of the tensor's
    // tiles (interleaved map) is read with the evict-last priority, everything before it with evict-first (or the default), so
    // that what stays in L2 is chosen by this kernel (about as much as L2 can
    // hold back) instead of whatever the replacement policy happens to keep of
    // a tensor that is larger than the cache.
    const uint64_t keep_policy = PolicyEvictLast();
    const uint64_t drop_policy = drop_rest ? PolicyEvictFirst() : PolicyEvictNormal();
    auto policy_of = [&](int stage) {
      return tile_first + stage * tile_step >= keep_from_tile ? keep_policy : drop_policy;
    };
    auto issue = [&](unsigned dst, uint64_t policy) {
#pragma unroll
      for (int u = 0; u < kU; ++u) {
        asm volatile(
            "cp.async.cg.shared.global.L2::cache_hint [%0], [%1], 16, %2;\n" ::"r"(
                dst + u * kSlotBytes),
            "l"(xi + u * row_bytes), "l"(policy)
            : "memory");
        if constexpr (kMode == kGrad) {
          asm volatile(
              "cp.async.cg.shared.global.L2::cache_hint [%0], [%1], 16, %2;\n" ::"r"(
                  dst + (kU + u) * kSlotBytes),
              "l"(di + u * row_bytes), "l"(policy)
              : "memory");
        }
      }
      xi += stage_bytes;
      di += stage_bytes;
    };
    // Prologue: kStages - 1 stages in flight (empty groups keep the count
    // uniform when the thread has fewer).
    int s_issue = 0;
#pragma unroll
    for (int st = 0; st < kStages - 1; ++st) {
      if (s_issue < n_full) {
        issue(my + st * kStageBytes, policy_of(s_issue));
        ++s_issue;
      }
      CpAsyncCommit();
    }
    unsigned fill = (kStages - 1) * kStageBytes;   // ring offset of the next stage to fill
    unsigned drain = 0;                            // ring offset of the next stage to read
    for (int s = 0; s < n_full; ++s) {
      if (s_issue < n_full) {
        issue(my + fill, policy_of(s_issue));
        ++s_issue;
      }
      CpAsyncCommit();
      fill = fill + kStageBytes == kStages * kStageBytes ? 0u : fill + kStageBytes;
      CpAsyncWait<kStages - 1>();
#pragma unroll
      for (int u = 0; u < kU; ++u) {
        uint4 rx, rd;
        asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];"
                     : "=r"(rx.x), "=r"(rx.y), "=r"(rx.z), "=r"(rx.w)
                     : "r"(my + drain + u * kSlotBytes));
        if constexpr (kMode == kGrad) {
          asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];"
                       : "=r"(rd.x), "=r"(rd.y), "=r"(rd.z), "=r"(rd.w)
                       : "r"(my + drain + (kU + u) * kSlotBytes));
        } else {
          rd = rx;
        }
        accumulate(rx, rd);
      }
      drain = drain + kStageBytes == kStages * kStageBytes ? 0u : drain + kStageBytes;
    }
    // Remainder rows (at most kU: a thread's share of a last, partial tile):
    // plain loads; xi / di stand at the first of them.
#pragma unroll
    for (int u = 0; u < kU; ++u) {
      if (u < rem) {
        const P px = LoadKeep(reinterpret_cast<const P*>(xi + u * row_bytes));
        P pd = px;
        if constexpr (kMode == kGrad) {
          pd = LoadKeep(reinterpret_cast<const P*>(di + u * row_bytes));
        }
        accumulate(*reinterpret_cast<const uint4*>(&px), *reinterpret_cast<const uint4*>(&pd));
      }
    }
  }
  CpAsyncWait<0>();
  __syncthreads();  // every thread is done with its slots: reuse the buffer

  float s1[kVec], s2[kVec];
#pragma unroll
  for (int q = 0; q < kPairs; ++q) {
    s1[2 * q] = a1[q].x;
    s1[2 * q + 1] = a1[q].y;
    s2[2 * q] = a2[q].x;
    s2[2 * q + 1] = a2[q].y;
  }
  float* red = reinterpret_cast<float*>(pipe_smem);
  if (TY > 1) {
#pragma unroll
    for (int e = 0; e < kVec; ++e) {
      red[((0 * kVec + e) * TY + ty) * TX + tx] = s1[e];
      red[((1 * kVec + e) * TY + ty) * TX + tx] = s2[e];
    }
    __syncthreads();
    const int n_out = 2 * kVec * TX;
    if (fold <= 1) {
      for (int o = tid; o < n_out; o += kThreads) {
        const int otx = o % TX;
        const int se = o / TX;
        float acc = 0.0f;
        for (int j = 0; j < TY; ++j) acc += red[(se * TY + j) * TX + otx];
        const int64_t ocol = static_cast<int64_t>(blockIdx.x) * TX + otx;
        if (ocol < cv) {
          const int sidx = se / kVec, e = se % kVec;
          partial[(static_cast<int64_t>(blockIdx.y) * 2 + sidx) * channels +
                  ocol * kVec + e] = acc;
        }
      }
    } else {
      // The launch put `fold` CTAs that are neighbours along y into one
      // cluster: their partial rows are added through distributed shared
      // memory (CTA r of the cluster adds its share of the columns, in CTA
      // order) and ONE row per cluster goes to memory, so few enough rows are
      // left for the element-wise kernel to add them itself.
      float* crow = red + 2 * kVec * kThreads;
      for (int o = tid; o < n_out; o += kThreads) {
        const int otx = o % TX;
        const int se = o / TX;
        float acc = 0.0f;
        for (int j = 0; j < TY; ++j) acc += red[(se * TY + j) * TX + otx];
        crow[o] = acc;
      }
      ClusterSync();
      const int rank = static_cast<int>(ClusterCtaRank());
      const int chunk = (n_out + fold - 1) / fold;
      for (int t = tid; t < chunk; t += kThreads) {
        const int o = rank * chunk + t;
        if (o < n_out) {
          double acc = 0.0;
          for (int q = 0; q < fold; ++q) {
            acc += static_cast<double>(LoadClusterF32(crow + o, static_cast<unsigned>(q)));
          }
          const int otx = o % TX;
          const int se = o / TX;
          const int64_t ocol = static_cast<int64_t>(blockIdx.x) * TX + otx;
          if (ocol < cv) {
            const int sidx = se / kVec, e = se % kVec;
            partial[(static_cast<int64_t>(blockIdx.y / fold) * 2 + sidx) * channels +
                    ocol * kVec + e] = static_cast<float>(acc);
          }
        }
      }
      ClusterSync();   // nobody leaves while a neighbour still reads its row
    }
  } else if (active) {
#pragma unroll
    for (int e = 0; e < kVec; ++e) {
      partial[(static_cast<int64_t>(blockIdx.y) * 2 + 0) * channels +
              col * kVec + e] = s1[e];
      partial[(static_cast<int64_t>(blockIdx.y) * 2 + 1) * channels +
              col * kVec + e] = s2[e];
    }
  }
}

// Channel-major layouts ([outer, C, inner], inner > 1): a plane (n, c) is a run
// of `inner` contiguous elements.  A WARP owns one channel: it walks the planes
// of its CTA's split of the outer axis as one flattened sequence of packs
// (lane l takes packs l, l + 32, ... of that sequence, whatever the plane
// length), with kPlaneUnroll loads in flight per lane.  Planes of any length
// keep all lanes busy - 7x7 planes as well as 112x112 ones - and the pack
// width is the widest that divides the plane (down to single elements), so no
// access ever straddles a plane.  A CTA covers 8 neighbouring channels.
constexpr int kPlaneUnroll = 8;
constexpr int kPlaneWarps = kThreads / 32;

struct PlaneCursor {
  int64_t n, i;       // plane index on the outer axis, pack inside the plane
  int64_t ip;         // packs per plane
  int64_t dn, di;     // 32 packs further: n += dn, i += di (+ carry)
  __device__ __forceinline__ void Init(int64_t n0, int lane, int64_t packs) {
    ip = packs;
    n = n0 + lane / ip;
    i = lane % ip;
    dn = 32 / ip;
    di = 32 % ip;
  }
  __device__ __forceinline__ void Advance() {
    n += dn;
    i += di;
    if (i >= ip) {
      i -= ip;
      ++n;
    }
  }
};

template <typename T, int kVec, int kMode>
__global__ void __launch_bounds__(kThreads)
    BnStatsPlaneKernel(const T* __restrict__ x, const T* __restrict__ dy,
                       const float* __restrict__ mean,
                       float* __restrict__ partial, int64_t outer,
                       int64_t channels, int64_t inner, int64_t outer_per_cta,
                       unsigned* epoch_bump) {
  using P = Pack<T, kVec>;
  GridDepWait();
  GridDepLaunch();
  BumpEpoch(epoch_bump, threadIdx.x);
  const int lane = threadIdx.x & 31;
  const int64_t c = static_cast<int64_t>(blockIdx.x) * kPlaneWarps + (threadIdx.x >> 5);
  if (c >= channels) return;  // whole warp; nothing below synchronises the CTA
  const int64_t n0 = static_cast<int64_t>(blockIdx.y) * outer_per_cta;
  int64_t n1 = n0 + outer_per_cta;
  if (n1 > outer) n1 = outer;
  const float shift = kMode == kFwd ? ToF32(x[c * inner]) : mean[c];
  const int64_t plane_stride = channels * inner;
  const T* xc = x + c * inner;
  const T* dc = dy + c * inner;
  PlaneCursor cur;
  cur.Init(n0, lane, inner / kVec);
  float s1 = 0.0f, s2 = 0.0f;
  float2 a1 = make_float2(0.0f, 0.0f), a2 = make_float2(0.0f, 0.0f);  // packed lanes
  const float2 nshift = make_float2(-shift, -shift);
  while (cur.n < n1) {
    P px[kPlaneUnroll];
    P pd[kPlaneUnroll];
    bool have[kPlaneUnroll];
#pragma unroll
    for (int u = 0; u < kPlaneUnroll; ++u) {
      have[u] = cur.n < n1;
      if (have[u]) {
        const int64_t at = cur.n * plane_stride + cur.i * kVec;
        px[u] = LoadKeep(reinterpret_cast<const P*>(xc + at));
        if constexpr (kMode == kGrad) pd[u] = LoadKeep(reinterpret_cast<const P*>(dc + at));
      }
      cur.Advance();
    }
#pragma unroll
    for (int u = 0; u < kPlaneUnroll; ++u) {
      if (have[u]) {
        if constexpr (kVec >= 2) {
          float2 xv[kVec / 2], gv[kVec / 2];
          WidenPack<kVec>(px[u], xv);
          if constexpr (kMode == kGrad) WidenPack<kVec>(pd[u], gv);
#pragma unroll
          for (int q = 0; q < kVec / 2; ++q) {
            const float2 d = Add2(xv[q], nshift);
            if constexpr (kMode == kFwd) {
              a1 = Add2(a1, d);
              a2 = Fma2(d, d, a2);
            } else {
              a1 = Add2(a1, gv[q]);
              a2 = Fma2(gv[q], d, a2);
            }
          }
        } else {
          const float d = ToF32(px[u].v[0]) - shift;
          if constexpr (kMode == kFwd) {
            s1 += d;
            s2 = fmaf(d, d, s2);
          } else {
            const float g = ToF32(pd[u].v[0]);
            s1 += g;
            s2 = fmaf(g, d, s2);
          }
        }
      }
    }
  }
  s1 += a1.x + a1.y;
  s2 += a2.x + a2.y;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    s1 += __shfl_xor_sync(0xffffffffu, s1, o);
    s2 += __shfl_xor_sync(0xffffffffu, s2, o);
  }
  if (lane == 0) {
    partial[(static_cast<int64_t>(blockIdx.y) * 2 + 0) * channels + c] = s1;
    partial[(static_cast<int64_t>(blockIdx.y) * 2 + 1) * channels + c] = s2;
  }
}

// Channel-major planes whose length is not a whole number of packs (7x7,
// 5x5, 3x3 ...): single planes cannot be read with 128-bit accesses, but a
// GROUP of kVec neighbouring channels can - its kVec * inner elements are
// `inner` whole packs, and the group starts on a 16-byte boundary for every n.
// A CTA owns one group and a split of the outer axis; thread t reads pack t of
// the group's run for n = n0, n0 + 1, ... (independent addresses: several in
// flight).  The position of a pack inside the run is the same for every n, so
// a thread's pack always covers the same one or two channels: the first
// `before` elements belong to channel lo, the rest to lo + 1.
constexpr int kGroupSlots = 4;   // packs of a run per thread (inner <= 4 * 256)
constexpr int kGroupUnroll = 4;  // values of n in flight per thread

__device__ __forceinline__ void GroupSlot(int p, int inner, int group, int* lo,
                                          int* before) {
  const int first = p * group;
  *lo = first / inner;
  *before = (*lo + 1) * inner - first;  // >= 1 elements of channel lo
}

template <typename T, int kMode>
__global__ void __launch_bounds__(kThreads)
    BnStatsGroupKernel(const T* __restrict__ x, const T* __restrict__ dy,
                       const float* __restrict__ mean,
                       float* __restrict__ partial, int64_t outer,
                       int64_t channels, int inner, int64_t outer_per_cta,
                       unsigned* epoch_bump) {
  constexpr int kG = VecWidth<T>::value;
  using P = Pack<T, kG>;
  extern __shared__ float4 contrib[];  // [inner]: (s1, s2) of lo, (s1, s2) of lo + 1
  __shared__ float shift_s[kG + 1];
  GridDepWait();
  GridDepLaunch();
  BumpEpoch(epoch_bump, threadIdx.x);
  const int64_t c0 = static_cast<int64_t>(blockIdx.x) * kG;
  const int64_t n0 = static_cast<int64_t>(blockIdx.y) * outer_per_cta;
  int64_t n1 = n0 + outer_per_cta;
  if (n1 > outer) n1 = outer;
  if (threadIdx.x < kG) {
    shift_s[threadIdx.x] = kMode == kFwd ? ToF32(x[(c0 + threadIdx.x) * inner])
                                         : mean[c0 + threadIdx.x];
  }
  if (threadIdx.x == 0) shift_s[kG] = 0.0f;
  __syncthreads();
  const int64_t run_stride = channels * inner;
  const T* xg = x + c0 * inner;
  const T* dg = dy + c0 * inner;
#pragma unroll 1
  for (int slot = 0; slot < kGroupSlots; ++slot) {
    const int p = threadIdx.x + slot * blockDim.x;
    if (p >= inner) break;
    int lo, before;
    GroupSlot(p, inner, kG, &lo, &before);
    const float sh_lo = shift_s[lo], sh_hi = shift_s[lo + 1];
    float s1l = 0.0f, s2l = 0.0f, s1h = 0.0f, s2h = 0.0f;
    for (int64_t n = n0; n < n1; n += kGroupUnroll) {
      P px[kGroupUnroll];
      P pd[kGroupUnroll];
#pragma unroll
      for (int u = 0; u < kGroupUnroll; ++u) {
        if (n + u < n1) {
          const int64_t at = (n + u) * run_stride;
          px[u] = LoadKeep(reinterpret_cast<const P*>(xg + at) + p);
          if constexpr (kMode == kGrad) pd[u] = LoadKeep(reinterpret_cast<const P*>(dg + at) + p);
        }
      }
#pragma unroll
      for (int u = 0; u < kGroupUnroll; ++u) {
        if (n + u < n1) {
#pragma unroll
          for (int e = 0; e < kG; ++e) {
            const bool in_lo = e < before;
            const float d = ToF32(px[u].v[e]) - (in_lo ? sh_lo : sh_hi);
            float a, b;
            if constexpr (kMode == kFwd) {
              a = d;
              b = d * d;
            } else {
              a = ToF32(pd[u].v[e]);
              b = a * d;
            }
            if (in_lo) {
              s1l += a;
              s2l += b;
            } else {
              s1h += a;
              s2h += b;
            }
          }
        }
      }
    }
    contrib[p] = make_float4(s1l, s2l, s1h, s2h);
  }
  __syncthreads();
  // Channel k of the group: its packs in run order, a fixed order of adds.
  if (threadIdx.x < kG) {
    const int k = threadIdx.x;
    const int p_first = (k * inner) / kG;
    const int p_last = ((k + 1) * inner - 1) / kG;
    float t1 = 0.0f, t2 = 0.0f;
    for (int p = p_first; p <= p_last; ++p) {
      int lo, before;
      GroupSlot(p, inner, kG, &lo, &before);
      const float4 v = contrib[p];
      if (lo == k) {
        t1 += v.x;
        t2 += v.y;
      } else {  // lo == k - 1: the pack crosses into this channel
        t1 += v.z;
        t2 += v.w;
      }
    }
    partial[(static_cast<int64_t>(blockIdx.y) * 2 + 0) * channels + c0 + k] = t1;
    partial[(static_cast<int64_t>(blockIdx.y) * 2 + 1) * channels + c0 + k] = t2;
  }
}

// ------------------------------------------------------------ level 2 ----

// kOut (a TailKind): forward statistics, forward raw sums (sum x, sum x^2),
// gradient (dscale, doffset and/or sums), or the local moments (mean,
// sum (x - mean)^2) for the cross-replica merge.
// Block (8 channels, kLanes partial lanes): 128 lanes (1024 threads) by
// default; 32 lanes make a 256-thread CTA that fits beside the draining
// statistics CTAs (measured the same to 1 % slower over the ResNet-50 step).
template <int kOut, int kLanes>
__global__ void __launch_bounds__(8 * kLanes) BnFinalizeKernel(FinalizeArgs a) {
  // Dependents first: the element-wise kernel that follows may take its place
  // on the SMs (and request its first rows of x, which do not depend on this
  // kernel) while the statistics kernel drains.  Its own wait still covers this
  // kernel, and this kernel's wait covers the statistics kernel.
  GridDepLaunch();
  GridDepWait();
  const int cx = threadIdx.x;  // 0..7
  const int py = threadIdx.y;  // 0..kLanes-1
  const int tid = py * 8 + cx;
  const int64_t c = static_cast<int64_t>(blockIdx.x) * 8 + cx;
  // The threads that finish a channel (first 8 of the CTA) fetch the shift
  // now, so that its latency overlaps the partial-sum loads.
  float shift_k = 0.0f;
  if (kOut != 2 && tid < 8 && c < a.channels) {
    shift_k = LoadAsF32(a.x_first, a.x_dtype, c * a.shift_stride);
  }
  // In-kernel exchange: the epoch of this exchange, and the replicas an
  // earlier exchange gave up on (not waited for again).
  __shared__ unsigned dead;
  unsigned epoch = 0;
  if (a.xchg != nullptr && tid < 32) {
    epoch = *reinterpret_cast<volatile unsigned*>(a.xchg_epoch);   // advanced by the statistics kernel
    if (tid == 0) {
      const int st = *reinterpret_cast<volatile int*>(a.xchg->status);
      dead = st > 0 && st <= kMaxWorld ? 1u << (st - 1) : 0u;
    }
  }
  double t1 = 0.0, t2 = 0.0;
  if (c < a.channels) {
    // kU independent loads per sum in flight: the loop is a chain of L2 round
    // trips otherwise.
    constexpr int kU = 8;
    int p = py;
    for (; p + (kU - 1) * kLanes < a.splits; p += kU * kLanes) {
      float u1[kU], u2[kU];
#pragma unroll
      for (int q = 0; q < kU; ++q) {
        const int64_t row = static_cast<int64_t>(p + q * kLanes) * 2;
        u1[q] = a.partial[(row + 0) * a.channels + c];
        u2[q] = a.partial[(row + 1) * a.channels + c];
      }
#pragma unroll
      for (int q = 0; q < kU; ++q) {
        t1 += static_cast<double>(u1[q]);
        t2 += static_cast<double>(u2[q]);
      }
    }
    float v1[kU - 1], v2[kU - 1];
#pragma unroll
    for (int q = 0; q < kU - 1; ++q) {
      v1[q] = 0.0f;
      v2[q] = 0.0f;
      if (p + q * kLanes < a.splits) {
        const int64_t row = static_cast<int64_t>(p + q * kLanes) * 2;
        v1[q] = a.partial[(row + 0) * a.channels + c];
        v2[q] = a.partial[(row + 1) * a.channels + c];
      }
    }
#pragma unroll
    for (int q = 0; q < kU - 1; ++q) {
      t1 += static_cast<double>(v1[q]);
      t2 += static_cast<double>(v2[q]);
    }
  }
  // A warp holds 4 partial lanes x 8 channels: fold lanes 8 and 16 apart.
  t1 += __shfl_xor_sync(0xffffffffu, t1, 8);
  t2 += __shfl_xor_sync(0xffffffffu, t2, 8);
  t1 += __shfl_xor_sync(0xffffffffu, t1, 16);
  t2 += __shfl_xor_sync(0xffffffffu, t2, 16);
  constexpr int kWarps = kLanes / 4;
  __shared__ double red[2][kWarps][8];
  const int warp = tid >> 5, lane = tid & 31;
  if (lane < 8) {
    red[0][warp][lane] = t1;
    red[1][warp][lane] = t2;
  }
  __syncthreads();
  if (warp == 0) {
    // Lane l folds warps {l/8, l/8 + 4, ...} of channel l % 8, then the four
    // lane groups fold with two shuffles: a fixed order, so the result does
    // not depend on scheduling.
    const int ch = lane & 7, grp = lane >> 3;
    double S1 = 0.0, S2 = 0.0;
#pragma unroll
    for (int w = 0; w < kWarps / 4; ++w) {
      S1 += red[0][grp + 4 * w][ch];
      S2 += red[1][grp + 4 * w][ch];
    }
    S1 += __shfl_xor_sync(0xffffffffu, S1, 8);
    S2 += __shfl_xor_sync(0xffffffffu, S2, 8);
    S1 += __shfl_xor_sync(0xffffffffu, S1, 16);
    S2 += __shfl_xor_sync(0xffffffffu, S2, 16);
    if (lane < 8 && c < a.channels) {
      const double inv_count = a.inv_count;
      if constexpr (kOut == 0) {
        const double K = static_cast<double>(shift_k);
        const double md = S1 * inv_count;
        WriteFwdStats(a, c, K + md, S2 * inv_count - md * md);
      } else if constexpr (kOut == 1) {
        if (a.count_out != nullptr && c == 0) {
          *a.count_out = static_cast<float>(a.count);
        }
        const double K = static_cast<double>(shift_k);
        // Local rows only: count is this replica's.
        a.sums[c] = static_cast<float>(S1 + a.count * K);
        a.sums[a.channels + c] =
            static_cast<float>(S2 + 2.0 * K * S1 + a.count * K * K);
      } else if constexpr (kOut == kTailFwdMoments) {
        const double md = S1 * inv_count;
        double m2 = S2 - md * S1;
        if (m2 < 0.0) m2 = 0.0;
        float mean_f = static_cast<float>(static_cast<double>(shift_k) + md);
        float m2_f = static_cast<float>(m2);
        float count_f = static_cast<float>(a.count);
        if (a.xchg != nullptr) {
          ExchangeChannelPair<true>(*a.xchg, epoch, static_cast<int>(a.channels),
                                    static_cast<int>(c), mean_f, m2_f, count_f, &dead, &mean_f,
                                    &m2_f, &count_f);
        }
        if (a.count_out != nullptr && c == 0) *a.count_out = count_f;
        a.sums[c] = mean_f;
        a.sums[a.channels + c] = m2_f;
      } else {
        float s1_f = static_cast<float>(S1), s2_f = static_cast<float>(S2);
        if (a.xchg != nullptr) {
          float unused;
          ExchangeChannelPair<false>(*a.xchg, epoch, static_cast<int>(a.channels),
                                     static_cast<int>(c), s1_f, s2_f, 0.0f, &dead, &s1_f, &s2_f,
                                     &unused);
        }
        if (a.sums) {
          a.sums[c] = s1_f;
          a.sums[a.channels + c] = s2_f;
        }
        if (a.doffset) a.doffset[c] = s1_f;
        if (a.dscale) {
          const float inv = 1.0f / sqrtf(a.variance[c] + a.epsilon);
          a.dscale[c] = s2_f * inv;
        }
      }
    }
  }
}

// Per-channel epilogues when the sums already exist (after an all-reduce).
// `moments`: sums = [mean, sum (x - mean)^2] instead of [sum x, sum x^2].
__global__ void BnFinalizeFromSumsKernel(FinalizeArgs a, const float* sums,
                                         bool moments) {
  GridDepWait();
  GridDepLaunch();
  const int64_t c = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (c >= a.channels) return;
  double mean, var;
  if (moments) {
    mean = static_cast<double>(sums[c]);
    var = static_cast<double>(sums[a.channels + c]) * a.inv_count;
  } else {
    mean = static_cast<double>(sums[c]) * a.inv_count;
    var = static_cast<double>(sums[a.channels + c]) * a.inv_count - mean * mean;
  }
  WriteFwdStats(a, c, mean, var);
}

// Merge of `world` per-replica moment vectors [mean[C], M2[C], count]
// (gathered back to back) into the moments of all rows together, in rank
// order and fp64: N = sum n_q, mean = sum n_q mean_q / N,
// M2 = sum M2_q + sum n_q (mean_q - mean)^2.
__global__ void BnMergeMomentsKernel(const float* gathered, int world,
                                     int64_t channels, float* out) {
  GridDepWait();
  GridDepLaunch();
  const int64_t c = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (c >= channels) return;
  const int64_t stride = 2 * channels + 1;
  double total = 0.0;
  for (int q = 0; q < world; ++q) {
    total += static_cast<double>(gathered[q * stride + 2 * channels]);
  }
  const double inv_total = total > 0.0 ? 1.0 / total : 0.0;
  double mean = 0.0;
  for (int q = 0; q < world; ++q) {
    mean += static_cast<double>(gathered[q * stride + 2 * channels]) *
            static_cast<double>(gathered[q * stride + c]);
  }
  mean *= inv_total;
  double m2 = 0.0;
  for (int q = 0; q < world; ++q) {
    const double d = static_cast<double>(gathered[q * stride + c]) - mean;
    m2 += static_cast<double>(gathered[q * stride + channels + c]) +
          static_cast<double>(gathered[q * stride + 2 * channels]) * d * d;
  }
  out[c] = static_cast<float>(mean);
  out[channels + c] = static_cast<float>(m2);
  if (c == 0) out[2 * channels] = static_cast<float>(total);
}

__global__ void BnGradScalesFromSumsKernel(const float* sums,
                                           const float* variance, float epsilon,
                                           float* dscale, float* doffset,
                                           int64_t channels) {
  GridDepWait();
  GridDepLaunch();
  const int64_t c = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (c >= channels) return;
  doffset[c] = sums[c];
  dscale[c] = sums[channels + c] * (1.0f / sqrtf(variance[c] + epsilon));
}

__global__ void ScaleKernel(float* data, float factor, int count) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < count) data[i] *= factor;
}

__global__ void InvStdKernel(const float* variance, float* inv_std,
                             float epsilon, int count) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < count) inv_std[i] = 1.0f / sqrtf(variance[i] + epsilon);
}

// ---------------------------------------------------------- apply pass ----

// Per-channel coefficients of the element-wise pass.
//   forward : y  = (x - mean) * a + b          a = scale*inv, b = offset
//   gradient: dx = a * (dy - c1 - (x - mean) * c2)
//             training : a = scale*inv, c1 = S1/R, c2 = S2*inv*inv/R
//             inference: a = scale*inv, c1 = c2 = 0
struct ApplyArgs {
  const float* scale;
  const float* offset;    // forward only
  const float* mean;
  const float* variance;
  const float* sums;      // gradient: [2, C] totals (NULL for inference grad)
  float inv_count;        // gradient: 1 / R over all replicas
  float epsilon;
  // Forward from all-reduced sums: when stat_sums is set, mean / variance are
  // derived from [sum x, sum x^2] over `count` values in the kernel prologue
  // and the first row of CTAs writes the four statistic outputs.
  const float* stat_sums;
  bool stat_moments;      // stat_sums = [mean, sum (x - mean)^2] (merged moments)
  double count;
  FinalizeArgs stat_out;  // est_*, batch_*, saved_*, exp_avg_factor
  // Gradient: the first row of CTAs writes dscale / doffset when set.
  float* dscale;
  float* doffset;
  // The statistics kernel of the same op left `fold_n` partial rows
  // ([fold_n, 2, C], folded on chip per cluster): every CTA adds the rows of
  // its own channels in its prologue (fp64, row order) and there is no
  // finalize kernel.  Forward: shifted sums (shift = first row of x), the
  // first row of CTAs writes the statistics outputs (stat_out); gradient:
  // [sum dy, sum dy (x - mean)], `fold_use` tells whether dx uses them
  // (training) or only dscale / doffset are written.
  const float* fold_rows;
  int fold_n;
  bool fold_use;
};

template <typename T, int kVec, int kUnroll, int kMode>
__global__ void __launch_bounds__(kThreads)
    BnApplyLastKernel(const T* __restrict__ x, const T* __restrict__ dy,
                      T* __restrict__ out, ApplyArgs a, int64_t rows,
                      int64_t cv, int64_t channels, int64_t rows_per_cta,
                      bool reverse, bool last_use, bool early_loads, bool interleave) {
  using P = Pack<T, kVec>;
  const int tx = threadIdx.x, ty = threadIdx.y;
  const int TX = blockDim.x, TY = blockDim.y;
  const int64_t col = static_cast<int64_t>(blockIdx.x) * TX + tx;
  const int64_t step = static_cast<int64_t>(TY) * kUnroll;
  // Two row maps (see BnStatsPipeKernel).  Contiguous: CTA b owns one range of
  // rows_per_cta rows, walked in batches of `step` rows.  Interleaved: the
  // rows are cut into tiles of `step` rows and CTA b takes tiles b, b + G ...
  // Either way the CTA sees "local rows" 0 .. n_rows - 1, batch k being local
  // rows [k * step, (k + 1) * step), mapped to global rows below; `reverse`
  // walks them from the end.
  int64_t r0, r1, n_rows, batch_stride;
  if (interleave) {
    const int64_t tiles = (rows + step - 1) / step;
    const int64_t G = gridDim.y, b = blockIdx.y;
    const int64_t mine = b < tiles ? (tiles - 1 - b) / G + 1 : 0;
    r0 = b * step;                 // global row of local row 0
    batch_stride = G * step;       // global rows between consecutive batches
    n_rows = mine * step;          // the last tile may stick out: checked per row
    r1 = rows;
  } else {
    const int64_t chunk = reverse ? (gridDim.y - 1 - blockIdx.y) : blockIdx.y;
    r0 = chunk * rows_per_cta;
    r1 = r0 + rows_per_cta;
    if (r1 > rows) r1 = rows;
    n_rows = r1 > r0 ? r1 - r0 : 0;
    batch_stride = step;
  }
  const P* xp = reinterpret_cast<const P*>(x) + col;
  const P* dp = reinterpret_cast<const P*>(dy) + col;
  const uint64_t drop_policy = PolicyEvictFirst();
  P px[kUnroll];
  P pd[kUnroll];
  int64_t off[kUnroll];
  // Loads of one batch of rows (local row l and the kUnroll - 1 after it).
  const int64_t n_batches = interleave ? n_rows / step : 0;
  // `k`: the batch, l = ty + k * step its first local row for this thread.
  auto load_batch = [&](int64_t l, int64_t k) {
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const int64_t li = l + static_cast<int64_t>(u) * TY;
      const int64_t in_batch = ty + static_cast<int64_t>(u) * TY;
      const int64_t kk = reverse ? (n_batches - 1 - k) : k;
      int64_t r;
      bool ok;
      if (interleave) {
        r = r0 + kk * batch_stride + in_batch;
        ok = li < n_rows && r < rows;
      } else {
        ok = li < n_rows;
        r = reverse ? (r1 - 1 - li) : (r0 + li);
      }
      off[u] = ok ? r * cv : -1;
      if (ok) {
        if constexpr (sizeof(P) == 16) {
          if (last_use) {
            px[u] = LoadHint16(xp + off[u], drop_policy);
            if constexpr (kMode == kGrad) pd[u] = LoadHint16(dp + off[u], drop_policy);
          } else {
            px[u] = LoadKeep(xp + off[u]);
            if constexpr (kMode == kGrad) pd[u] = LoadKeep(dp + off[u]);
          }
        } else {
          px[u] = LoadKeep(xp + off[u]);
          if constexpr (kMode == kGrad) pd[u] = LoadKeep(dp + off[u]);
        }
      }
    }
  };
  // `early_loads`: x and dy are inputs of the whole op, final before the
  // statistics kernel of the same launcher call started, and only the
  // per-channel statistics come from the kernel this one depends on.  The
  // first batch of rows is then requested BEFORE the wait for that kernel, so
  // its latency (and the tail of the reduction) is hidden behind it.  A
  // stand-alone element-wise launch cannot know who produced x and waits
  // first.
  const bool active = col < cv;
  if (early_loads && active) load_batch(ty, 0);
  // The shift of the shifted sums (first row of x: an input of the op, like
  // the early rows).
  P first_row;
  if (kMode == kFwd && a.fold_rows != nullptr && active) first_row = LoadKeep(xp);
  GridDepWait();
  GridDepLaunch();
  // Second level of the reduction when no finalize kernel ran (fold_rows):
  // the CTA fetches the partial rows of its own channels into shared memory
  // with one round of 16-byte copies and adds them in fp64, in row order.
  extern __shared__ __align__(16) float fold_smem[];   // [fold_n][2][TX * kVec]
  __shared__ double s_tot[2][kThreads];     // TX * kVec <= kThreads (the launcher sees to it)
  if (a.fold_rows != nullptr) {
    const int tid = ty * TX + tx;
    const int nch = TX * kVec;
    const int64_t c0 = static_cast<int64_t>(blockIdx.x) * nch;
    const int seg = channels - c0 < nch ? static_cast<int>(channels - c0) : nch;
    if constexpr (kVec >= 4) {
      const int per_seg = seg / 4;                       // 16-byte copies per row segment
      const int copies = a.fold_n * 2 * per_seg;
      for (int i = tid; i < copies; i += kThreads) {
        const int r2 = i / per_seg, j = i - r2 * per_seg;
        CpAsync16(fold_smem + r2 * nch + j * 4,
                  a.fold_rows + static_cast<int64_t>(r2) * channels + c0 + j * 4);
      }
      CpAsyncCommit();
      CpAsyncWait<0>();
    }
    __syncthreads();
    for (int o = tid; o < 2 * nch; o += kThreads) {
      const int which = o / nch, ch = o - which * nch;
      double acc = 0.0;
      if (ch < seg) {
        for (int r = 0; r < a.fold_n; ++r) {
          acc += static_cast<double>(fold_smem[(r * 2 + which) * nch + ch]);
        }
      }
      s_tot[which][ch] = acc;
    }
    __syncthreads();
  }
  if (!active) return;

  // 16-bit outputs round to 8 or 11 bits, so the per-channel affine forms are
  // folded to two (forward) or three (gradient) coefficients and one or two
  // FMAs per element; fp32 keeps the centred form (x - mean) to the end.
  constexpr bool kFold = sizeof(T) == 2;
  const bool writer = blockIdx.y == 0 && ty == 0;
  float mean[kVec], ca[kVec], cb[kVec], cc[kVec];
#pragma unroll
  for (int e = 0; e < kVec; ++e) {
    const int64_t c = col * kVec + e;
    float var_c;
    if (kMode == kFwd && a.fold_rows != nullptr) {
      // Shifted sums (the statistics kernel subtracted the first row).
      const double K = static_cast<double>(ToF32(first_row.v[e]));
      const double md = s_tot[0][tx * kVec + e] * a.stat_out.inv_count;
      const double m = K + md;
      double v = s_tot[1][tx * kVec + e] * a.stat_out.inv_count - md * md;
      if (v < 0.0) v = 0.0;
      mean[e] = static_cast<float>(m);
      var_c = static_cast<float>(v);
      if (writer) WriteFwdStats(a.stat_out, c, m, v);
    } else if (kMode == kFwd && a.stat_sums != nullptr) {
      double m, v;
      if (a.stat_moments) {
        m = static_cast<double>(a.stat_sums[c]);
        v = static_cast<double>(a.stat_sums[channels + c]) * a.stat_out.inv_count;
      } else {
        m = static_cast<double>(a.stat_sums[c]) * a.stat_out.inv_count;
        v = static_cast<double>(a.stat_sums[channels + c]) * a.stat_out.inv_count - m * m;
      }
      if (v < 0.0) v = 0.0;
      mean[e] = static_cast<float>(m);
      var_c = static_cast<float>(v);
      if (writer) WriteFwdStats(a.stat_out, c, m, v);
    } else {
      mean[e] = a.mean[c];
      var_c = a.variance[c];
    }
    const float inv = 1.0f / sqrtf(var_c + a.epsilon);
    ca[e] = a.scale[c] * inv;
    if constexpr (kMode == kFwd) {
      cb[e] = a.offset[c];
      cc[e] = 0.0f;
    } else {
      if (a.fold_rows != nullptr) {
        const float t1 = static_cast<float>(s_tot[0][tx * kVec + e]);
        const float t2 = static_cast<float>(s_tot[1][tx * kVec + e]);
        cb[e] = a.fold_use ? t1 * a.inv_count : 0.0f;
        cc[e] = a.fold_use ? t2 * inv * inv * a.inv_count : 0.0f;
        if (writer && a.dscale != nullptr) {
          a.doffset[c] = t1;
          a.dscale[c] = t2 * inv;
        }
      } else if (a.sums != nullptr) {
        cb[e] = a.sums[c] * a.inv_count;
        cc[e] = a.sums[channels + c] * inv * inv * a.inv_count;
      } else {
        cb[e] = 0.0f;
        cc[e] = 0.0f;
      }
      if (writer && a.dscale != nullptr && a.sums != nullptr) {
        a.doffset[c] = a.sums[c];
        a.dscale[c] = a.sums[channels + c] * inv;
      }
    }
    if constexpr (kFold) {
      if constexpr (kMode == kFwd) {
        // y = x * ca + (offset - mean * ca)
        cb[e] = fmaf(-mean[e], ca[e], cb[e]);
      } else {
        // dx = dy * ca + x * (-ca * cc) + ca * (cc * mean - cb)
        const float fb = -ca[e] * cc[e];
        const float fc = ca[e] * fmaf(cc[e], mean[e], -cb[e]);
        cb[e] = fb;
        cc[e] = fc;
      }
    }
  }

  P* op = reinterpret_cast<P*>(out) + col;
  // Row lane ty visits local rows ty, ty + TY, ...; in reverse mode the local
  // index is mirrored.
  int64_t batch = 0;
  for (int64_t l = ty; l < n_rows; l += step, ++batch) {
    if (!(early_loads && batch == 0)) load_batch(l, batch);
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      if (off[u] >= 0) {
        P o;
        if constexpr (kVec >= 2) {
          // Packed fp32 pairs (same roundings as the scalar forms below).
          constexpr int kPairs = kVec / 2;
          float2 xv[kPairs], gv[kPairs], rv[kPairs];
          WidenPack<kVec>(px[u], xv);
          if constexpr (kMode == kGrad) WidenPack<kVec>(pd[u], gv);
#pragma unroll
          for (int q = 0; q < kPairs; ++q) {
            const float2 A = make_float2(ca[2 * q], ca[2 * q + 1]);
            const float2 B = make_float2(cb[2 * q], cb[2 * q + 1]);
            const float2 C = make_float2(cc[2 * q], cc[2 * q + 1]);
            if constexpr (kFold) {
              if constexpr (kMode == kFwd) {
                rv[q] = Fma2(xv[q], A, B);
              } else {
                rv[q] = Fma2(gv[q], A, Fma2(xv[q], B, C));
              }
            } else {
              const float2 d =
                  Add2(xv[q], make_float2(-mean[2 * q], -mean[2 * q + 1]));
              if constexpr (kMode == kFwd) {
                rv[q] = Fma2(d, A, B);
              } else {
                // ca * ((g - cb) - d * cc)
                rv[q] = Mul2(A, Fma2(Neg2(d), C, Add2(gv[q], Neg2(B))));
              }
            }
          }
          NarrowPack<kVec>(rv, o);
        } else {
#pragma unroll
        for (int e = 0; e < kVec; ++e) {
          float r;
          if constexpr (kFold) {
            const float xv = ToF32(px[u].v[e]);
            if constexpr (kMode == kFwd) {
              r = fmaf(xv, ca[e], cb[e]);
            } else {
              r = fmaf(ToF32(pd[u].v[e]), ca[e], fmaf(xv, cb[e], cc[e]));
            }
          } else {
            const float d = ToF32(px[u].v[e]) - mean[e];
            if constexpr (kMode == kFwd) {
              r = fmaf(d, ca[e], cb[e]);
            } else {
              const float g = ToF32(pd[u].v[e]);
              r = ca[e] * (g - cb[e] - d * cc[e]);
            }
          }
          o.v[e] = FromF32<T>(r);
        }
        }
        StoreStream(op + off[u], o);
      }
    }
  }
}

// Channel-major element-wise pass: the warp-per-channel walk of
// BnStatsPlaneKernel; the channel's coefficients are formed once per warp.
template <typename T, int kVec, int kMode>
__global__ void __launch_bounds__(kThreads)
    BnApplyPlaneKernel(const T* __restrict__ x, const T* __restrict__ dy,
                       T* __restrict__ out, ApplyArgs a, int64_t outer,
                       int64_t channels, int64_t inner, int64_t outer_per_cta) {
  using P = Pack<T, kVec>;
  GridDepWait();
  GridDepLaunch();
  const int lane = threadIdx.x & 31;
  const int64_t c = static_cast<int64_t>(blockIdx.x) * kPlaneWarps + (threadIdx.x >> 5);
  if (c >= channels) return;
  const int64_t n0 = static_cast<int64_t>(blockIdx.y) * outer_per_cta;
  int64_t n1 = n0 + outer_per_cta;
  if (n1 > outer) n1 = outer;
  const float inv = 1.0f / sqrtf(a.variance[c] + a.epsilon);
  const float mean = a.mean[c];
  const float ca = a.scale[c] * inv;
  float cb, cc = 0.0f;
  if constexpr (kMode == kFwd) {
    cb = a.offset[c];
  } else {
    cb = a.sums ? a.sums[c] * a.inv_count : 0.0f;
    cc = a.sums ? a.sums[channels + c] * inv * inv * a.inv_count : 0.0f;
  }
  const float2 nmean2 = make_float2(-mean, -mean), ca2 = make_float2(ca, ca);
  const float2 cb2 = make_float2(cb, cb), ncb2 = make_float2(-cb, -cb);
  const float2 ncc2 = make_float2(-cc, -cc);
  const int64_t plane_stride = channels * inner;
  const T* xc = x + c * inner;
  const T* dc = dy + c * inner;
  T* oc = out + c * inner;
  PlaneCursor cur;
  cur.Init(n0, lane, inner / kVec);
  constexpr int kU = kMode == kFwd ? kPlaneUnroll : kPlaneUnroll / 2;
  while (cur.n < n1) {
    P px[kU];
    P pd[kU];
    int64_t at[kU];
#pragma unroll
    for (int u = 0; u < kU; ++u) {
      at[u] = cur.n < n1 ? cur.n * plane_stride + cur.i * kVec : -1;
      if (at[u] >= 0) {
        px[u] = LoadStream(reinterpret_cast<const P*>(xc + at[u]));
        if constexpr (kMode == kGrad) pd[u] = LoadStream(reinterpret_cast<const P*>(dc + at[u]));
      }
      cur.Advance();
    }
#pragma unroll
    for (int u = 0; u < kU; ++u) {
      if (at[u] >= 0) {
        P o;
        if constexpr (kVec >= 2) {
          float2 xv[kVec / 2], gv[kVec / 2], rv[kVec / 2];
          WidenPack<kVec>(px[u], xv);
          if constexpr (kMode == kGrad) WidenPack<kVec>(pd[u], gv);
#pragma unroll
          for (int q = 0; q < kVec / 2; ++q) {
            const float2 d = Add2(xv[q], nmean2);
            if constexpr (kMode == kFwd) {
              rv[q] = Fma2(d, ca2, cb2);
            } else {
              // ca * (dy - cb - d * cc)
              rv[q] = Mul2(ca2, Fma2(d, ncc2, Add2(gv[q], ncb2)));
            }
          }
          NarrowPack<kVec>(rv, o);
        } else {
          const float d = ToF32(px[u].v[0]) - mean;
          float r;
          if constexpr (kMode == kFwd) {
            r = fmaf(d, ca, cb);
          } else {
            r = ca * (ToF32(pd[u].v[0]) - cb - d * cc);
          }
          o.v[0] = FromF32<T>(r);
        }
        StoreStream(reinterpret_cast<P*>(oc + at[u]), o);
      }
    }
  }
}

// Element-wise pass of the channel-group form (see BnStatsGroupKernel): the
// group's coefficients sit in shared memory, a pack picks those of channel lo
// for its first `before` elements and those of lo + 1 for the rest.
template <typename T, int kMode>
__global__ void __launch_bounds__(kThreads)
    BnApplyGroupKernel(const T* __restrict__ x, const T* __restrict__ dy,
                       T* __restrict__ out, ApplyArgs a, int64_t outer,
                       int64_t channels, int inner, int64_t outer_per_cta) {
  constexpr int kG = VecWidth<T>::value;
  using P = Pack<T, kG>;
  __shared__ float4 coef[kG + 1];  // mean, ca, cb, cc
  GridDepWait();
  GridDepLaunch();
  const int64_t c0 = static_cast<int64_t>(blockIdx.x) * kG;
  const int64_t n0 = static_cast<int64_t>(blockIdx.y) * outer_per_cta;
  int64_t n1 = n0 + outer_per_cta;
  if (n1 > outer) n1 = outer;
  if (threadIdx.x < kG) {
    const int64_t c = c0 + threadIdx.x;
    const float inv = 1.0f / sqrtf(a.variance[c] + a.epsilon);
    float cb, cc = 0.0f;
    if constexpr (kMode == kFwd) {
      cb = a.offset[c];
    } else {
      cb = a.sums ? a.sums[c] * a.inv_count : 0.0f;
      cc = a.sums ? a.sums[channels + c] * inv * inv * a.inv_count : 0.0f;
    }
    coef[threadIdx.x] = make_float4(a.mean[c], a.scale[c] * inv, cb, cc);
  }
  if (threadIdx.x == 0) coef[kG] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
  __syncthreads();
  const int64_t run_stride = channels * inner;
  const T* xg = x + c0 * inner;
  const T* dg = dy + c0 * inner;
  T* og = out + c0 * inner;
#pragma unroll 1
  for (int slot = 0; slot < kGroupSlots; ++slot) {
    const int p = threadIdx.x + slot * blockDim.x;
    if (p >= inner) break;
    int lo, before;
    GroupSlot(p, inner, kG, &lo, &before);
    const float4 cl = coef[lo], ch = coef[lo + 1];
    for (int64_t n = n0; n < n1; n += kGroupUnroll) {
      P px[kGroupUnroll];
      P pd[kGroupUnroll];
#pragma unroll
      for (int u = 0; u < kGroupUnroll; ++u) {
        if (n + u < n1) {
          const int64_t at = (n + u) * run_stride;
          px[u] = LoadStream(reinterpret_cast<const P*>(xg + at) + p);
          if constexpr (kMode == kGrad) pd[u] = LoadStream(reinterpret_cast<const P*>(dg + at) + p);
        }
      }
#pragma unroll
      for (int u = 0; u < kGroupUnroll; ++u) {
        if (n + u < n1) {
          P o;
#pragma unroll
          for (int e = 0; e < kG; ++e) {
            const float4 k = e < before ? cl : ch;
            const float d = ToF32(px[u].v[e]) - k.x;
            float r;
            if constexpr (kMode == kFwd) {
              r = fmaf(d, k.y, k.z);
            } else {
              r = k.y * (ToF32(pd[u].v[e]) - k.z - d * k.w);
            }
            o.v[e] = FromF32<T>(r);
          }
          StoreStream(reinterpret_cast<P*>(og + (n + u) * run_stride) + p, o);
        }
      }
    }
  }
}

// ------------------------------------------------------------ host side --

template <typename T>
struct DtypeCode;
template <>
struct DtypeCode<float> {
  static constexpr int value = MUSA_DT_F32;
};
template <>
struct DtypeCode<__half> {
  static constexpr int value = MUSA_DT_F16;
};
template <>
struct DtypeCode<__nv_bfloat16> {
  static constexpr int value = MUSA_DT_BF16;
};

struct Geom {
  int64_t outer, channels, inner;
  int64_t rows() const { return outer * inner; }  // values per channel
};

inline int CheckGeom(const Geom& g) {
  if (g.outer < 0 || g.channels < 0 || g.inner < 0) return MUSA_KERNELS_EINVAL;
  return MUSA_KERNELS_OK;
}

inline bool IsEmpty(const Geom& g) {
  return g.outer == 0 || g.channels == 0 || g.inner == 0;
}

// Workspace layout: [partial rows: MaxSplits * 2 * C floats][totals: 2 * C
// floats], rounded up to 256 bytes.
inline size_t WorkspaceBytes(const Geom& g) {
  if (IsEmpty(g)) return 0;
  const int64_t floats =
      MaxSplits(g.outer, g.channels) * 2 * g.channels + 2 * g.channels;
  return static_cast<size_t>((floats + 63) / 64 * 64) * sizeof(float);
}

// Launch errors travel as -(1000 + cudaError_t) beside the negative
// MUSA_KERNELS_E* codes and come back out as the positive cudaError_t.
inline int EncodeCuda(cudaError_t e) { return -(1000 + static_cast<int>(e)); }
inline int DecodeError(int rc) { return rc <= -1000 ? -rc - 1000 : rc; }

// Pipelined channels-last statistics.  Returns the number of partial rows
// written, or a negative error.
template <typename T, int kMode, int kStagesT>
int LaunchStatsPipe(const T* x, const T* dy, const float* mean, float* workspace,
                    const Geom& g, int64_t cv, unsigned* epoch_bump, cudaStream_t stream,
                    int* fold_io = nullptr) {
  using Cfg = StatsPipe<kMode, kStagesT>;
  auto kernel = BnStatsPipeKernel<T, kMode, kStagesT>;
  static std::atomic<int> resident_by_device[kMaxDevices];
  const int resident = PerDevice(resident_by_device, [&] {
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             Cfg::kSmemBytes) != cudaSuccess) {
      cudaGetLastError();
      return -1;
    }
    int n = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kernel, kThreads,
                                                      Cfg::kSmemBytes) != cudaSuccess) {
      cudaGetLastError();
      return -1;
    }
    return n > 0 ? n : -1;
  });
  if (resident < 0) return EncodeCuda(cudaErrorInvalidValue);
  // Column blocks of at most 16 packs (256-byte row segments; the tuning
  // table holds the width): measured 3 % faster over the ResNet-50 step than
  // blocks as wide as the row, which leave one row lane per CTA for the wide
  // layers.
  int max_tx = GetTuning(kTuneBnStatsMaxTx);
  if (max_tx <= 0) max_tx = kThreads;
  const Plan p = PlanLast(g.outer, g.channels, cv, Cfg::kU, true, resident, max_tx);
  // What the element-wise pass that follows can find in L2: the budget over
  // the bytes this pass reads (all streams), as the fraction of every
  // thread's rows that is read with the evict-last priority.
  const double bytes = static_cast<double>(g.outer) * static_cast<double>(g.channels) *
                       sizeof(T) * (kMode == kFwd ? 1 : 2);
  const double budget = static_cast<double>(GetTuning(kTuneBnL2KeepMb)) * 1048576.0;
  float keep_fraction = 0.0f;
  if (budget > 0.0) {
    keep_fraction = budget >= bytes ? 1.0f : static_cast<float>(budget / bytes);
    if (GetTuning(kTuneBnL2KeepPartial) == 0 && keep_fraction < 1.0f) keep_fraction = 0.0f;
  }
  // Clusters of `fold` CTAs along y add their partial rows on chip (the
  // caller asked for it and the block has row lanes to fold): grid.y becomes a
  // multiple of `fold` within what is resident at once, and gy / fold rows are
  // written.
  int fold = fold_io != nullptr ? *fold_io : 1;
  if (fold != 2 && fold != 4 && fold != 8) fold = 1;   // portable cluster sizes
  if (p.ty == 1) fold = 1;
  int gy = p.gy;
  int64_t rows_per_cta = p.rows_per_cta;
  if (fold > 1) {
    static std::atomic<int> clusters_by_device[4][kMaxDevices];   // fold 2, 4, 8
    const int max_clusters = PerDevice(clusters_by_device[fold == 2 ? 0 : fold == 4 ? 1 : 2], [&] {
      cudaLaunchConfig_t cfg;
      cudaLaunchAttribute attr[2];
      ClusterConfig(&cfg, attr, false, fold, dim3(1, fold), dim3(kThreads), Cfg::kSmemBytes,
                    nullptr);
      int n = 0;
      if (cudaOccupancyMaxActiveClusters(&n, kernel, &cfg) != cudaSuccess) {
        cudaGetLastError();
        return -1;
      }
      return n > 0 ? n : -1;
    });
    int64_t per_column = max_clusters > 0 ? max_clusters / p.gx : 0;
    if (per_column < 1) {
      fold = 1;
    } else {
      int64_t clusters = CeilDiv(static_cast<int64_t>(gy), static_cast<int64_t>(fold));
      if (clusters > per_column) clusters = per_column;
      gy = static_cast<int>(clusters) * fold;
      rows_per_cta = CeilDiv(CeilDiv(g.outer, static_cast<int64_t>(gy)), p.ty) * p.ty;
    }
  }
  if (fold_io != nullptr) *fold_io = fold;
  const cudaError_t err = LaunchClustered(
      GetTuning(kTuneBnPdl) != 0, fold, kernel, dim3(p.gx, gy), dim3(p.tx, p.ty),
      Cfg::kSmemBytes, stream, x, dy, mean, workspace, g.outer, cv, g.channels,
      rows_per_cta, keep_fraction, GetTuning(kTuneBnStatsDropRest) != 0,
      GetTuning(kTuneBnInterleave) != 0, epoch_bump, fold);
  if (err != cudaSuccess) {
    cudaGetLastError();
    return EncodeCuda(err);
  }
  return gy / fold;
}

// Grid of the channel-major kernels: 8 channels per CTA along x, the outer
// axis cut into gy pieces so that about 8 CTAs per SM exist.
struct PlanePlan {
  int64_t gx, gy, per;
};
inline PlanePlan PlanPlanes(const Geom& g) {
  PlanePlan p;
  p.gx = CeilDiv(g.channels, kPlaneWarps);
  if (p.gx > 0x7fffffffLL) {
    p.gx = -1;
    return p;
  }
  int64_t target = static_cast<int64_t>(SmCount()) * 8 / p.gx;
  if (target < 1) target = 1;
  int64_t gy = target < g.outer ? target : g.outer;
  const int64_t cap = MaxSplits(g.outer, g.channels);
  if (gy > cap) gy = cap;
  if (gy > 65535) gy = 65535;
  if (gy < 1) gy = 1;
  p.per = CeilDiv(g.outer, gy);
  p.gy = CeilDiv(g.outer, p.per);
  return p;
}

// Widest pack (in elements, at most 16 bytes) that divides a plane, given
// 16-byte aligned tensors; single elements otherwise.
template <typename T>
inline int PlaneVec(int64_t inner, bool aligned) {
  if (!aligned) return 1;
  for (int v = VecWidth<T>::value; v > 1; v >>= 1) {
    if (inner % v == 0) return v;
  }
  return 1;
}

// The channel-group form applies to planes that are not whole packs, when the
// groups tile the channel axis and a thread has at most kGroupSlots packs.
template <typename T>
inline bool UseChannelGroups(const Geom& g, bool aligned) {
  constexpr int kG = VecWidth<T>::value;
  return aligned && g.inner % kG != 0 && g.inner >= kG &&
         g.inner <= static_cast<int64_t>(kGroupSlots) * kThreads && g.channels % kG == 0;
}
struct GroupPlan {
  int64_t gx, gy, per;
  int threads;
};
template <typename T>
inline GroupPlan PlanGroups(const Geom& g) {
  constexpr int kG = VecWidth<T>::value;
  GroupPlan p;
  p.gx = g.channels / kG;
  int64_t target = static_cast<int64_t>(SmCount()) * 8 / (p.gx > 0 ? p.gx : 1);
  if (target < 1) target = 1;
  int64_t gy = target < g.outer ? target : g.outer;
  const int64_t cap = MaxSplits(g.outer, g.channels);
  if (gy > cap) gy = cap;
  if (gy > 65535) gy = 65535;
  if (gy < 1) gy = 1;
  p.per = CeilDiv(g.outer, gy);
  p.gy = CeilDiv(g.outer, p.per);
  const int64_t t = (g.inner + 31) / 32 * 32;
  p.threads = static_cast<int>(t < kThreads ? t : kThreads);
  return p;
}

// Stats launch: fills partial[splits][2][C]; returns splits or a negative
// error.
template <typename T, int kMode>
int LaunchStats(const T* x, const T* dy, const float* mean, float* partial,
                const Geom& g, unsigned* epoch_bump, cudaStream_t stream,
                int* fold_io = nullptr) {
  constexpr int kVec = VecWidth<T>::value;
  constexpr int kUnroll = 4;
  // Only the pipelined channels-last kernel folds partial rows on chip.
  int fold_none = 1;
  int* const fold_pipe = fold_io != nullptr ? fold_io : &fold_none;
  const int fold_wanted = *fold_pipe;
  *fold_pipe = 1;
  const bool keep = GetTuning(kTuneBnStatsKeep) != 0;
  const bool aligned = Aligned16(x) && (kMode == kFwd || Aligned16(dy));
  if (g.inner == 1) {
    if (g.channels % kVec == 0 && aligned) {
      const int64_t cv = g.channels / kVec;
      const int stages = GetTuning(kTuneBnStatsPipe);
      if (stages == 3) {
        *fold_pipe = fold_wanted;
        return LaunchStatsPipe<T, kMode, 3>(x, dy, mean, partial, g, cv, epoch_bump, stream,
                                            fold_pipe);
      }
      if (stages != 0) {
        *fold_pipe = fold_wanted;
        return LaunchStatsPipe<T, kMode, 4>(x, dy, mean, partial, g, cv, epoch_bump, stream,
                                            fold_pipe);
      }
      const Plan p = PlanLast(g.outer, g.channels, cv, kUnroll, true, 3);
      BnStatsLastKernel<T, kVec, kUnroll, kMode>
          <<<dim3(p.gx, p.gy), dim3(p.tx, p.ty), 0, stream>>>(
              x, dy, mean, partial, g.outer, cv, g.channels, p.rows_per_cta,
              keep, epoch_bump);
      CountKernelLaunch();
      return p.gy;
    }
    const Plan p = PlanLast(g.outer, g.channels, g.channels, kUnroll, true, 4);
    BnStatsLastKernel<T, 1, kUnroll, kMode>
        <<<dim3(p.gx, p.gy), dim3(p.tx, p.ty), 0, stream>>>(
            x, dy, mean, partial, g.outer, g.channels, g.channels,
            p.rows_per_cta, keep, epoch_bump);
    CountKernelLaunch();
    return p.gy;
  }
  if (UseChannelGroups<T>(g, aligned) && g.channels / kVec <= 0x7fffffffLL) {
    const GroupPlan gp = PlanGroups<T>(g);
    BnStatsGroupKernel<T, kMode>
        <<<dim3(static_cast<unsigned>(gp.gx), static_cast<unsigned>(gp.gy)), gp.threads,
           static_cast<size_t>(g.inner) * sizeof(float4), stream>>>(
            x, dy, mean, partial, g.outer, g.channels, static_cast<int>(g.inner), gp.per,
            epoch_bump);
    CountKernelLaunch();
    return static_cast<int>(gp.gy);
  }
  // [outer, C, inner]: a warp per channel, the outer axis split over grid.y.
  const PlanePlan pp = PlanPlanes(g);
  if (pp.gx < 0) return MUSA_KERNELS_ETOOLARGE;
  const dim3 grid(static_cast<unsigned>(pp.gx), static_cast<unsigned>(pp.gy));
  switch (PlaneVec<T>(g.inner, aligned)) {
    case 8:
      if constexpr (kVec >= 8) {
        BnStatsPlaneKernel<T, 8, kMode><<<grid, kThreads, 0, stream>>>(
            x, dy, mean, partial, g.outer, g.channels, g.inner, pp.per, epoch_bump);
        CountKernelLaunch();
      }
      break;
    case 4:
      BnStatsPlaneKernel<T, 4, kMode><<<grid, kThreads, 0, stream>>>(
          x, dy, mean, partial, g.outer, g.channels, g.inner, pp.per, epoch_bump);
      CountKernelLaunch();
      break;
    case 2:
      BnStatsPlaneKernel<T, 2, kMode><<<grid, kThreads, 0, stream>>>(
          x, dy, mean, partial, g.outer, g.channels, g.inner, pp.per, epoch_bump);
      CountKernelLaunch();
      break;
    default:
      BnStatsPlaneKernel<T, 1, kMode><<<grid, kThreads, 0, stream>>>(
          x, dy, mean, partial, g.outer, g.channels, g.inner, pp.per, epoch_bump);
      CountKernelLaunch();
  }
  return static_cast<int>(pp.gy);
}

template <int kLanes>
void LaunchFinalizeAs(int kind, const FinalizeArgs& a, cudaStream_t stream) {
  const int grid = static_cast<int>(CeilDiv(a.channels, 8));
  const bool pdl = GetTuning(kTuneBnPdl) != 0;
  const dim3 block(8, kLanes);
  switch (kind) {
    case kTailFwdStats:
      LaunchChained(pdl, BnFinalizeKernel<kTailFwdStats, kLanes>, dim3(grid), block, 0, stream, a);
      break;
    case kTailFwdSums:
      LaunchChained(pdl, BnFinalizeKernel<kTailFwdSums, kLanes>, dim3(grid), block, 0, stream, a);
      break;
    case kTailFwdMoments:
      LaunchChained(pdl, BnFinalizeKernel<kTailFwdMoments, kLanes>, dim3(grid), block, 0, stream,
                    a);
      break;
    default:
      LaunchChained(pdl, BnFinalizeKernel<kTailGrad, kLanes>, dim3(grid), block, 0, stream, a);
  }
}

void LaunchFinalize(int kind, const FinalizeArgs& a, cudaStream_t stream) {
  if (GetTuning(kTuneBnFinalizeLanes) == 128) {
    LaunchFinalizeAs<128>(kind, a, stream);
  } else {
    LaunchFinalizeAs<32>(kind, a, stream);
  }
}

// Both levels of the reduction: the statistics kernel, then the finalize
// kernel.  `f.partial` / `f.splits` are filled in here.  0 or an error code.
template <typename T, int kMode>
int RunStats(const T* x, const T* dy, const float* mean, float* workspace,
             const Geom& g, FinalizeArgs f, int kind, cudaStream_t stream) {
  f.partial = workspace;
  const int splits = LaunchStats<T, kMode>(x, dy, mean, workspace, g, f.xchg_epoch, stream);
  if (splits < 0) return DecodeError(splits);
  f.splits = splits;
  LaunchFinalize(kind, f, stream);
  return MUSA_KERNELS_OK;
}

// Column blocks of the element-wise kernels, in channel packs (measured on the
// ResNet-50 step: 16 packs 7.21 ms, whole rows 7.25 ms).
inline int ApplyMaxTx() {
  const int t = GetTuning(kTuneBnApplyMaxTx);
  return t > 0 ? t : kThreads;
}

// Dynamic shared memory of an element-wise launch that adds `fold_n` partial
// rows itself, or -1 when its column blocks are wider than a CTA has threads
// (the prologue gives every channel of the block one thread).
constexpr int64_t kApplyFoldSmemMax = 64 * 1024;
template <typename T>
inline int64_t ApplyFoldBytes(int64_t cv, int fold_n) {
  constexpr int kVec = VecWidth<T>::value;
  const int tx = PlanTx(cv, ApplyMaxTx());   // the column block PlanLast will choose
  if (tx * kVec > kThreads) return -1;
  return static_cast<int64_t>(fold_n) * 2 * tx * kVec * static_cast<int64_t>(sizeof(float));
}

template <typename T, int kVec, int kU, int kMode>
void LaunchApplyLast(const T* x, const T* dy, T* out, const ApplyArgs& a, const Geom& g,
                     int64_t cv, bool reverse, bool last_use, bool early_loads,
                     cudaStream_t stream) {
  auto kernel = BnApplyLastKernel<T, kVec, kU, kMode>;
  static std::atomic<int> resident_by_device[kMaxDevices];
  int resident = PerDevice(resident_by_device, [&] {
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             static_cast<int>(kApplyFoldSmemMax)) != cudaSuccess) {
      cudaGetLastError();
    }
    int n = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kernel, kThreads, 0) !=
        cudaSuccess) {
      cudaGetLastError();
    }
    return n > 0 ? n : 1;
  });
  size_t smem = 0;
  if (a.fold_rows != nullptr) {
    smem = static_cast<size_t>(ApplyFoldBytes<T>(cv, a.fold_n));
    // Shared memory of an SM over a CTA's dynamic + static + reserved bytes.
    const int by_smem = static_cast<int>(233472 / (smem + 4096 + 1024));
    if (by_smem < resident) resident = by_smem > 0 ? by_smem : 1;
  }
  const Plan p = PlanLast(g.outer, g.channels, cv, kU, false, resident, ApplyMaxTx());
  LaunchChained(GetTuning(kTuneBnPdl) != 0, kernel, dim3(p.gx, p.gy), dim3(p.tx, p.ty), smem,
                stream, x, dy, out, a, g.outer, cv, g.channels, p.rows_per_cta, reverse,
                last_use, early_loads, GetTuning(kTuneBnInterleave) != 0);
}

// `early_loads`: the caller launched the statistics kernel of the same op on
// `stream` just before (see BnApplyLastKernel).
template <typename T, int kMode>
void LaunchApply(const T* x, const T* dy, T* out, const ApplyArgs& a,
                 const Geom& g, cudaStream_t stream, bool early_loads = false) {
  constexpr int kVec = VecWidth<T>::value;
  constexpr int kUnroll = 4;
  const bool reverse = GetTuning(kTuneBnApplyReverse) != 0;
  // Evict-first loads pay off while the tensor is of the order of L2 (what the
  // statistics pass left there is not pushed out); on larger ones they cost.
  const int64_t in_bytes = g.outer * g.channels * g.inner *
                           static_cast<int64_t>(sizeof(T)) *
                           (kMode == kFwd ? 1 : 2);
  // (measured: up to four times the L2 budget the hinted loads pay - the
  // config-2 gradient, 205 MB of inputs, 83 against 87 us - beyond that they
  // cost: the gradient pass alone on 822 MB, 0.94 against 0.99 of peak.)
  const bool last_use =
      GetTuning(kTuneBnApplyDropAll) != 0 ||
      in_bytes <= (static_cast<int64_t>(GetTuning(kTuneBnL2KeepMb)) << 22);
  const bool aligned =
      Aligned16(x) && Aligned16(out) && (kMode == kFwd || Aligned16(dy));
  if (g.inner == 1) {
    if (g.channels % kVec == 0 && aligned) {
      const int64_t cv = g.channels / kVec;
      // The forward pass has one input stream: twice the rows in flight.
      const bool deep = kMode == kFwd && GetTuning(kTuneBnApplyDeep) != 0;
      const bool early = early_loads && GetTuning(kTuneBnApplyEarlyLoads) != 0;
      if (deep) {
        constexpr int kDeep = kMode == kFwd ? 8 : kUnroll;
        LaunchApplyLast<T, kVec, kDeep, kMode>(x, dy, out, a, g, cv, reverse, last_use, early,
                                               stream);
      } else {
        LaunchApplyLast<T, kVec, kUnroll, kMode>(x, dy, out, a, g, cv, reverse, last_use, early,
                                                 stream);
      }
    } else {
      const Plan p =
          PlanLast(g.outer, g.channels, g.channels, kUnroll, false, 4);
      BnApplyLastKernel<T, 1, kUnroll, kMode>
          <<<dim3(p.gx, p.gy), dim3(p.tx, p.ty), 0, stream>>>(
              x, dy, out, a, g.outer, g.channels, g.channels, p.rows_per_cta,
              reverse, false, false, false);
      CountKernelLaunch();
    }
    return;
  }
  const bool pdl = GetTuning(kTuneBnPdl) != 0;
  if (UseChannelGroups<T>(g, aligned) && g.channels / kVec <= 0x7fffffffLL) {
    const GroupPlan gp = PlanGroups<T>(g);
    LaunchChained(pdl, BnApplyGroupKernel<T, kMode>,
                  dim3(static_cast<unsigned>(gp.gx), static_cast<unsigned>(gp.gy)),
                  dim3(gp.threads), 0, stream, x, dy, out, a, g.outer, g.channels,
                  static_cast<int>(g.inner), gp.per);
    return;
  }
  const PlanePlan pp = PlanPlanes(g);
  if (pp.gx < 0) return;
  const dim3 grid(static_cast<unsigned>(pp.gx), static_cast<unsigned>(pp.gy));
  switch (PlaneVec<T>(g.inner, aligned)) {
    case 8:
      if constexpr (kVec >= 8) {
        LaunchChained(pdl, BnApplyPlaneKernel<T, 8, kMode>, grid, dim3(kThreads), 0, stream, x,
                      dy, out, a, g.outer, g.channels, g.inner, pp.per);
      }
      break;
    case 4:
      LaunchChained(pdl, BnApplyPlaneKernel<T, 4, kMode>, grid, dim3(kThreads), 0, stream, x, dy,
                    out, a, g.outer, g.channels, g.inner, pp.per);
      break;
    case 2:
      LaunchChained(pdl, BnApplyPlaneKernel<T, 2, kMode>, grid, dim3(kThreads), 0, stream, x, dy,
                    out, a, g.outer, g.channels, g.inner, pp.per);
      break;
    default:
      LaunchChained(pdl, BnApplyPlaneKernel<T, 1, kMode>, grid, dim3(kThreads), 0, stream, x, dy,
                    out, a, g.outer, g.channels, g.inner, pp.per);
  }
}

inline int LastError() { return static_cast<int>(cudaGetLastError()); }

// Whether the op has the geometry in which the element-wise kernel can add
// the partial rows itself (channels-last whole packs, 16-byte aligned
// tensors: the vector form of BnApplyLastKernel).
template <typename T>
inline bool VectorChain(const Geom& g, const void* x, const void* out, const void* dy) {
  constexpr int kVec = VecWidth<T>::value;
  return g.inner == 1 && g.channels % kVec == 0 && Aligned16(x) && Aligned16(out) &&
         (dy == nullptr || Aligned16(dy));
}
// ... and whether it does, given the rows the statistics kernel left: few
// enough (the tuning table holds the limit) and within the shared memory the
// element-wise kernel may take.  The finalize kernel costs a kernel boundary
// and, for wide layers, hundreds of CTAs; a few dozen rows are added faster by
// every CTA for its own channels.
template <typename T>
inline bool ApplyAddsRows(const Geom& g, int rows) {
  if (rows > GetTuning(kTuneBnApplyAddsRows)) return false;
  const int64_t bytes = ApplyFoldBytes<T>(g.channels / VecWidth<T>::value, rows);
  return bytes >= 0 && bytes <= kApplyFoldSmemMax;
}

template <typename T>
int FwdTrain(const void* x, const float* scale, const float* offset,
             const float* est_mean, const float* est_var, void* y,
             float* batch_mean, float* batch_var, float* saved_mean,
             float* saved_var, int64_t outer, int64_t channels, int64_t inner,
             float epsilon, float exp_avg_factor, void* workspace,
             size_t workspace_bytes, cudaStream_t stream) {
  const Geom g{outer, channels, inner};
  if (int rc = CheckGeom(g)) return rc;
  MUSA_TRACE("LaunchBnFwdTrain", 2 * sizeof(T) * outer * channels * inner);
  if (IsEmpty(g)) return MUSA_KERNELS_OK;
  if (!x || !y || !scale || !offset || !saved_mean || !saved_var) {
    return MUSA_KERNELS_EINVAL;
  }
  if (exp_avg_factor != 1.0f && (!est_mean || !est_var)) {
    return MUSA_KERNELS_EINVAL;
  }
  if (!workspace || workspace_bytes < WorkspaceBytes(g) ||
      !Aligned16(workspace)) {
    return MUSA_KERNELS_EWORKSPACE;
  }
  float* partial = static_cast<float*>(workspace);
  const T* xt = static_cast<const T*>(x);
  FinalizeArgs f{};
  f.partial = partial;
  f.channels = channels;
  SetCount(&f, static_cast<double>(g.rows()));
  f.x_first = x;
  f.x_dtype = DtypeCode<T>::value;
  f.shift_stride = inner == 1 ? 1 : inner;
  f.est_mean = est_mean;
  f.est_var = est_var;
  f.batch_mean = batch_mean;
  f.batch_var = batch_var;
  f.saved_mean = saved_mean;
  f.saved_var = saved_var;
  f.exp_avg_factor = exp_avg_factor;
  ApplyArgs a{};
  a.scale = scale;
  a.offset = offset;
  a.mean = saved_mean;
  a.variance = saved_var;
  a.epsilon = epsilon;
  // (An in-place call, y == x, keeps the finalize kernel: the element-wise
  // kernel would otherwise re-read the first row of x, the shift of the sums,
  // while other CTAs already overwrite it.)
  const bool vector_chain = x != y && VectorChain<T>(g, x, y, nullptr);
  int fold = vector_chain ? GetTuning(kTuneBnClusterFold) : 1;
  const int splits = LaunchStats<T, kFwd>(xt, nullptr, nullptr, partial, g, nullptr, stream,
                                          &fold);
  if (splits < 0) return DecodeError(splits);
  if (vector_chain && ApplyAddsRows<T>(g, splits)) {
    // The element-wise kernel adds the few rows that are left and writes the
    // statistics outputs: no finalize kernel.
    a.fold_rows = partial;
    a.fold_n = splits;
    a.stat_out = f;
  } else {
    f.splits = splits;
    LaunchFinalize(kTailFwdStats, f, stream);
  }
  LaunchApply<T, kFwd>(xt, nullptr, static_cast<T*>(y), a, g, stream, true);
  return LastError();
}

template <typename T>
int FwdInfer(const void* x, const float* scale, const float* offset,
             const float* est_mean, const float* est_var, void* y,
             int64_t outer, int64_t channels, int64_t inner, float epsilon,
             cudaStream_t stream) {
  const Geom g{outer, channels, inner};
  if (int rc = CheckGeom(g)) return rc;
  MUSA_TRACE("LaunchBnApply", 2 * sizeof(T) * outer * channels * inner);
  if (IsEmpty(g)) return MUSA_KERNELS_OK;
  if (!x || !y || !scale || !offset || !est_mean || !est_var) {
    return MUSA_KERNELS_EINVAL;
  }
  ApplyArgs a{};
  a.scale = scale;
  a.offset = offset;
  a.mean = est_mean;
  a.variance = est_var;
  a.epsilon = epsilon;
  LaunchApply<T, kFwd>(static_cast<const T*>(x), nullptr, static_cast<T*>(y), a,
                       g, stream);
  return LastError();
}

template <typename T>
int Grad(const void* dy, const void* x, const float* scale, const float* mean,
         const float* variance, void* dx, float* dscale, float* doffset,
         int64_t outer, int64_t channels, int64_t inner, float epsilon,
         bool is_training, void* workspace, size_t workspace_bytes,
         cudaStream_t stream) {
  const Geom g{outer, channels, inner};
  if (int rc = CheckGeom(g)) return rc;
  MUSA_TRACE("LaunchBnGrad", 3 * sizeof(T) * outer * channels * inner);
  if (IsEmpty(g)) return MUSA_KERNELS_OK;
  if (!dy || !x || !scale || !mean || !variance || !dx || !dscale || !doffset) {
    return MUSA_KERNELS_EINVAL;
  }
  if (!workspace || workspace_bytes < WorkspaceBytes(g) ||
      !Aligned16(workspace)) {
    return MUSA_KERNELS_EWORKSPACE;
  }
  float* partial = static_cast<float*>(workspace);
  float* sums = partial + MaxSplits(g.outer, g.channels) * 2 * g.channels;
  const T* xt = static_cast<const T*>(x);
  const T* dyt = static_cast<const T*>(dy);
  FinalizeArgs f{};
  f.partial = partial;
  f.channels = channels;
  SetCount(&f, static_cast<double>(g.rows()));
  f.variance = variance;
  f.dscale = dscale;
  f.doffset = doffset;
  f.epsilon = epsilon;
  f.sums = sums;
  ApplyArgs a{};
  a.scale = scale;
  a.mean = mean;
  a.variance = variance;
  a.epsilon = epsilon;
  a.sums = is_training ? sums : nullptr;
  a.inv_count = static_cast<float>(1.0 / static_cast<double>(g.rows()));
  const bool vector_chain = VectorChain<T>(g, x, dx, dy);
  int fold = vector_chain ? GetTuning(kTuneBnClusterFold) : 1;
  const int splits = LaunchStats<T, kGrad>(xt, dyt, mean, partial, g, nullptr, stream, &fold);
  if (splits < 0) return DecodeError(splits);
  if (vector_chain && ApplyAddsRows<T>(g, splits)) {
    a.sums = nullptr;
    a.fold_rows = partial;
    a.fold_n = splits;
    a.fold_use = is_training;
    a.dscale = dscale;
    a.doffset = doffset;
  } else {
    f.splits = splits;
    LaunchFinalize(kTailGrad, f, stream);
  }
  LaunchApply<T, kGrad>(xt, dyt, static_cast<T*>(dx), a, g, stream, true);
  return LastError();
}

template <typename T>
int StatsSums(const void* x, float* sums, float* count_out, const Geom& g,
              void* workspace, size_t workspace_bytes, int kind,
              cudaStream_t stream, const ExchangeDev* xchg = nullptr,
              unsigned* xchg_epoch = nullptr) {
  MUSA_TRACE("LaunchBnStats", sizeof(T) * g.outer * g.channels * g.inner);
  if (!x || !sums) return MUSA_KERNELS_EINVAL;
  if (!workspace || workspace_bytes < WorkspaceBytes(g) ||
      !Aligned16(workspace)) {
    return MUSA_KERNELS_EWORKSPACE;
  }
  float* partial = static_cast<float*>(workspace);
  FinalizeArgs f{};
  f.channels = g.channels;
  SetCount(&f, static_cast<double>(g.rows()));
  f.x_first = x;
  f.x_dtype = DtypeCode<T>::value;
  f.shift_stride = g.inner == 1 ? 1 : g.inner;
  f.sums = sums;
  f.count_out = count_out;
  f.xchg = xchg;
  f.xchg_epoch = xchg_epoch;
  if (int rc = RunStats<T, kFwd>(static_cast<const T*>(x), nullptr, nullptr, partial, g,
                                 f, kind, stream)) {
    return rc;
  }
  return LastError();
}

template <typename T>
int GradStatsSums(const void* dy, const void* x, const float* mean, float* sums,
                  const Geom& g, void* workspace, size_t workspace_bytes,
                  cudaStream_t stream, const ExchangeDev* xchg = nullptr,
                  unsigned* xchg_epoch = nullptr) {
  MUSA_TRACE("LaunchBnGradStats", 2 * sizeof(T) * g.outer * g.channels * g.inner);
  if (!dy || !x || !mean || !sums) return MUSA_KERNELS_EINVAL;
  if (!workspace || workspace_bytes < WorkspaceBytes(g) ||
      !Aligned16(workspace)) {
    return MUSA_KERNELS_EWORKSPACE;
  }
  float* partial = static_cast<float*>(workspace);
  FinalizeArgs f{};
  f.channels = g.channels;
  SetCount(&f, static_cast<double>(g.rows()));
  f.sums = sums;
  f.xchg = xchg;
  f.xchg_epoch = xchg_epoch;
  if (int rc = RunStats<T, kGrad>(static_cast<const T*>(x), static_cast<const T*>(dy),
                                  mean, partial, g, f, kTailGrad, stream)) {
    return rc;
  }
  return LastError();
}

template <typename T>
int GradApplyFromSums(const void* dy, const void* x, const float* scale,
                      const float* mean, const float* variance,
                      const float* sums, double total_count, void* dx,
                      float* dscale, float* doffset, const Geom& g,
                      float epsilon, cudaStream_t stream) {
  MUSA_TRACE("LaunchBnGradApply", 3 * sizeof(T) * g.outer * g.channels * g.inner);
  if (!dy || !x || !scale || !mean || !variance || !sums || !dx) {
    return MUSA_KERNELS_EINVAL;
  }
  ApplyArgs a{};
  if (dscale && doffset) {
    if (g.inner == 1) {
      a.dscale = dscale;  // written by the element-wise kernel's first CTA row
      a.doffset = doffset;
    } else {
      const int grid = static_cast<int>(CeilDiv(g.channels, 256));
      BnGradScalesFromSumsKernel<<<grid, 256, 0, stream>>>(
          sums, variance, epsilon, dscale, doffset, g.channels);
      CountKernelLaunch();
    }
  }
  a.scale = scale;
  a.mean = mean;
  a.variance = variance;
  a.epsilon = epsilon;
  a.sums = sums;
  a.inv_count = static_cast<float>(1.0 / total_count);
  // dy and x were read by the preceding LaunchBnGradStatsSums* call on this
  // stream: final before it (see ApplyFromSums).
  LaunchApply<T, kGrad>(static_cast<const T*>(x), static_cast<const T*>(dy),
                        static_cast<T*>(dx), a, g, stream, true);
  return LastError();
}

// ---- Scratch that lives in the library image, for callers that cannot
// allocate device memory (see LaunchBnFwdTrainNoAlloc below).
//
// 4 MiB of level-1 partial sums plus the [2, C] totals for up to 8192
// channels.  Every GPU that loads the library carries this array until the
// process exits.  In host code the array's NAME is only a handle of the
// runtime, not a device address: the address a kernel may use is obtained
// with cudaGetSymbolAddress, once per device, with that device current.
constexpr int64_t kStaticScratchMaxChannels = 8192;
constexpr size_t kStaticScratchBytes =
    sizeof(float) * (kMaxPartialFloats + 2 * kStaticScratchMaxChannels) + 512;
static __device__ __align__(256) unsigned char
    g_bn_static_scratch[kStaticScratchBytes];

constexpr int kScratchMaxDevices = kMaxDevices;
std::mutex g_scratch_mutex;
void* g_scratch_addr[kScratchMaxDevices] = {};

// Device address of g_bn_static_scratch on the current device; resolves it on
// the first call per device.  Returns a cudaError_t (0 on success).
int StaticScratchAddress(void** out) {
  int dev = -1;
  cudaError_t err = cudaGetDevice(&dev);
  if (err != cudaSuccess) return static_cast<int>(err);
  if (dev < 0 || dev >= kScratchMaxDevices) {
    return static_cast<int>(cudaErrorInvalidDevice);
  }
  std::lock_guard<std::mutex> lock(g_scratch_mutex);
  if (g_scratch_addr[dev] == nullptr) {
    void* ptr = nullptr;
    err = cudaGetSymbolAddress(&ptr, g_bn_static_scratch);
    if (err != cudaSuccess) return static_cast<int>(err);
    if (ptr == nullptr) return static_cast<int>(cudaErrorInvalidSymbol);
    g_scratch_addr[dev] = ptr;
  }
  *out = g_scratch_addr[dev];
  return 0;
}

}  // namespace
}  // namespace musa_b200

using namespace musa_b200;

#define MUSA_BY_DTYPE(dtype, CALL)                      \
  switch (dtype) {                                      \
    case MUSA_DT_F32: {                                 \
      using T = float;                                  \
      return CALL;                                      \
    }                                                   \
    case MUSA_DT_F16: {                                 \
      using T = __half;                                 \
      return CALL;                                      \
    }                                                   \
    case MUSA_DT_BF16: {                                \
      using T = __nv_bfloat16;                          \
      return CALL;                                      \
    }                                                   \
    default:                                            \
      return MUSA_KERNELS_EUNSUPPORTED;                 \
  }

extern "C" {

size_t BnWorkspaceBytes(int64_t outer, int64_t channels, int64_t inner) {
  const Geom g{outer, channels, inner};
  if (CheckGeom(g) != MUSA_KERNELS_OK) return 0;
  return WorkspaceBytes(g);
}

#define MUSA_DEFINE_BN(SUFFIX, TYPE)                                           \
  int LaunchBnFwdTrain_##SUFFIX(                                               \
      const void* x, const float* scale, const float* offset,                  \
      const float* est_mean, const float* est_var, void* y, float* batch_mean, \
      float* batch_var, float* saved_mean, float* saved_var, int64_t outer,    \
      int64_t channels, int64_t inner, float epsilon, float exp_avg_factor,    \
      void* workspace, size_t workspace_bytes, cudaStream_t stream) {          \
    return FwdTrain<TYPE>(x, scale, offset, est_mean, est_var, y, batch_mean,  \
                          batch_var, saved_mean, saved_var, outer, channels,   \
                          inner, epsilon, exp_avg_factor, workspace,           \
                          workspace_bytes, stream);                            \
  }                                                                            \
  int LaunchBnFwdInfer_##SUFFIX(                                               \
      const void* x, const float* scale, const float* offset,                  \
      const float* est_mean, const float* est_var, void* y, int64_t outer,     \
      int64_t channels, int64_t inner, float epsilon, cudaStream_t stream) {   \
    return FwdInfer<TYPE>(x, scale, offset, est_mean, est_var, y, outer,       \
                          channels, inner, epsilon, stream);                   \
  }                                                                            \
  int LaunchBnGrad_##SUFFIX(                                                   \
      const void* dy, const void* x, const float* scale, const float* mean,    \
      const float* variance, void* dx, float* dscale, float* doffset,          \
      int64_t outer, int64_t channels, int64_t inner, float epsilon,           \
      bool is_training, void* workspace, size_t workspace_bytes,               \
      cudaStream_t stream) {                                                   \
    return Grad<TYPE>(dy, x, scale, mean, variance, dx, dscale, doffset,       \
                      outer, channels, inner, epsilon, is_training, workspace, \
                      workspace_bytes, stream);                                \
  }

MUSA_DEFINE_BN(F32, float)
MUSA_DEFINE_BN(F16, __half)
MUSA_DEFINE_BN(BF16, __nv_bfloat16)
#undef MUSA_DEFINE_BN

size_t BnNoAllocMaxChannels(void) {
  return static_cast<size_t>(kStaticScratchMaxChannels);
}

int LaunchBnFwdTrainNoAlloc(int dtype, const void* x, const float* scale,
                            const float* offset, const float* est_mean,
                            const float* est_var, void* y, float* batch_mean,
                            float* batch_var, float* saved_mean,
                            float* saved_var, int64_t outer, int64_t channels,
                            int64_t inner, float epsilon, float exp_avg_factor,
                            cudaStream_t stream) {
  const Geom g{outer, channels, inner};
  if (int rc = CheckGeom(g)) return rc;
  if (IsEmpty(g)) return MUSA_KERNELS_OK;
  if (channels > kStaticScratchMaxChannels ||
      WorkspaceBytes(g) > kStaticScratchBytes) {
    return MUSA_KERNELS_ETOOLARGE;
  }
  void* scratch = nullptr;
  if (int rc = StaticScratchAddress(&scratch)) return rc;
  MUSA_BY_DTYPE(dtype,
                FwdTrain<T>(x, scale, offset, est_mean, est_var, y, batch_mean,
                            batch_var, saved_mean, saved_var, outer, channels,
                            inner, epsilon, exp_avg_factor, scratch,
                            kStaticScratchBytes, stream));
}

void LaunchBesselCorrection(float* data, float factor, int count,
                            cudaStream_t stream) {
  if (count <= 0) return;
  ScaleKernel<<<(count + 255) / 256, 256, 0, stream>>>(data, factor, count);
  CountKernelLaunch();
}

void LaunchVarianceToInvStd(const float* variance, float* inv_std,
                            float epsilon, int count, cudaStream_t stream) {
  if (count <= 0) return;
  InvStdKernel<<<(count + 255) / 256, 256, 0, stream>>>(variance, inv_std,
                                                       epsilon, count);
  CountKernelLaunch();
}

int LaunchBnStatsSums(int dtype, const void* x, float* sums, int64_t outer,
                      int64_t channels, int64_t inner, void* workspace,
                      size_t workspace_bytes, cudaStream_t stream) {
  const Geom g{outer, channels, inner};
  if (int rc = CheckGeom(g)) return rc;
  if (channels == 0) return MUSA_KERNELS_OK;
  if (!sums) return MUSA_KERNELS_EINVAL;
  if (IsEmpty(g)) {
    // A replica with no rows contributes zeros to the all-reduce.
    return static_cast<int>(
        cudaMemsetAsync(sums, 0, sizeof(float) * 2 * channels, stream));
  }
  MUSA_BY_DTYPE(dtype, StatsSums<T>(x, sums, nullptr, g, workspace,
                                    workspace_bytes, kTailFwdSums, stream));
}

int LaunchBnStatsSumsCount(int dtype, const void* x, float* sums, int64_t outer,
                           int64_t channels, int64_t inner, void* workspace,
                           size_t workspace_bytes, cudaStream_t stream) {
  const Geom g{outer, channels, inner};
  if (int rc = CheckGeom(g)) return rc;
  if (channels == 0) return MUSA_KERNELS_OK;
  if (!sums) return MUSA_KERNELS_EINVAL;
  if (IsEmpty(g)) {
    return static_cast<int>(
        cudaMemsetAsync(sums, 0, sizeof(float) * (2 * channels + 1), stream));
  }
  MUSA_BY_DTYPE(dtype, StatsSums<T>(x, sums, sums + 2 * channels, g, workspace,
                                    workspace_bytes, kTailFwdSums, stream));
}

namespace {
int FinalizeFromSums(const float* sums, bool moments, double total_count,
                     const float* est_mean, const float* est_var, float* batch_mean,
                     float* batch_var, float* saved_mean, float* saved_var,
                     int64_t channels, float exp_avg_factor, cudaStream_t stream) {
  if (channels < 0 || !(total_count > 0.0)) return MUSA_KERNELS_EINVAL;
  if (channels == 0) return MUSA_KERNELS_OK;
  if (!sums || !saved_mean || !saved_var) return MUSA_KERNELS_EINVAL;
  if (exp_avg_factor != 1.0f && (!est_mean || !est_var)) {
    return MUSA_KERNELS_EINVAL;
  }
  FinalizeArgs f{};
  f.channels = channels;
  SetCount(&f, total_count);
  f.est_mean = est_mean;
  f.est_var = est_var;
  f.batch_mean = batch_mean;
  f.batch_var = batch_var;
  f.saved_mean = saved_mean;
  f.saved_var = saved_var;
  f.exp_avg_factor = exp_avg_factor;
  const int grid = static_cast<int>(CeilDiv(channels, 256));
  BnFinalizeFromSumsKernel<<<grid, 256, 0, stream>>>(f, sums, moments);
  CountKernelLaunch();
  return LastError();
}

int ApplyFromSums(int dtype, const void* x, const float* scale, const float* offset,
                  const float* sums, bool moments, double total_count,
                  const float* est_mean, const float* est_var, float exp_avg_factor,
                  void* y, float* batch_mean, float* batch_var, float* saved_mean,
                  float* saved_var, int64_t outer, int64_t channels, int64_t inner,
                  float epsilon, cudaStream_t stream) {
  const Geom g{outer, channels, inner};
  if (int rc = CheckGeom(g)) return rc;
  if (!(total_count > 0.0)) return MUSA_KERNELS_EINVAL;
  if (channels == 0) return MUSA_KERNELS_OK;
  if (!sums || !scale || !offset || !saved_mean || !saved_var) {
    return MUSA_KERNELS_EINVAL;
  }
  if (exp_avg_factor != 1.0f && (!est_mean || !est_var)) {
    return MUSA_KERNELS_EINVAL;
  }
  if (g.inner != 1 || IsEmpty(g)) {
    // General layout (or a replica without rows): statistics first, then the
    // element-wise pass.
    if (int rc = FinalizeFromSums(sums, moments, total_count, est_mean, est_var,
                                  batch_mean, batch_var, saved_mean, saved_var, channels,
                                  exp_avg_factor, stream)) {
      return rc;
    }
    if (IsEmpty(g)) return MUSA_KERNELS_OK;
    return LaunchBnApply(dtype, x, scale, offset, saved_mean, saved_var, y,
                         outer, channels, inner, epsilon, stream);
  }
  if (!x || !y) return MUSA_KERNELS_EINVAL;
  ApplyArgs a{};
  a.scale = scale;
  a.offset = offset;
  a.epsilon = epsilon;
  a.stat_sums = sums;
  a.stat_moments = moments;
  a.count = total_count;
  a.stat_out.channels = channels;
  SetCount(&a.stat_out, total_count);
  a.stat_out.est_mean = est_mean;
  a.stat_out.est_var = est_var;
  a.stat_out.batch_mean = batch_mean;
  a.stat_out.batch_var = batch_var;
  a.stat_out.saved_mean = saved_mean;
  a.stat_out.saved_var = saved_var;
  a.stat_out.exp_avg_factor = exp_avg_factor;
  // x is the tensor whose statistics the preceding launcher call on this
  // stream took: it was final before that call, so the first rows may be
  // requested before the wait for the kernel that delivers the statistics.
  MUSA_BY_DTYPE(dtype, (LaunchApply<T, kFwd>(static_cast<const T*>(x), nullptr,
                                             static_cast<T*>(y), a, g, stream, true),
                        LastError()));
}
}  // namespace

int LaunchBnApplyFromSums(int dtype, const void* x, const float* scale,
                          const float* offset, const float* sums,
                          double total_count, const float* est_mean,
                          const float* est_var, float exp_avg_factor, void* y,
                          float* batch_mean, float* batch_var,
                          float* saved_mean, float* saved_var, int64_t outer,
                          int64_t channels, int64_t inner, float epsilon,
                          cudaStream_t stream) {
  return ApplyFromSums(dtype, x, scale, offset, sums, false, total_count, est_mean,
                       est_var, exp_avg_factor, y, batch_mean, batch_var, saved_mean,
                       saved_var, outer, channels, inner, epsilon, stream);
}

int LaunchBnApplyFromMoments(int dtype, const void* x, const float* scale,
                             const float* offset, const float* moments,
                             double total_count, const float* est_mean,
                             const float* est_var, float exp_avg_factor, void* y,
                             float* batch_mean, float* batch_var,
                             float* saved_mean, float* saved_var, int64_t outer,
                             int64_t channels, int64_t inner, float epsilon,
                             cudaStream_t stream) {
  return ApplyFromSums(dtype, x, scale, offset, moments, true, total_count, est_mean,
                       est_var, exp_avg_factor, y, batch_mean, batch_var, saved_mean,
                       saved_var, outer, channels, inner, epsilon, stream);
}

int LaunchBnStatsMoments(int dtype, const void* x, float* moments, int64_t outer,
                         int64_t channels, int64_t inner, void* workspace,
                         size_t workspace_bytes, cudaStream_t stream) {
  const Geom g{outer, channels, inner};
  if (int rc = CheckGeom(g)) return rc;
  if (channels == 0) return MUSA_KERNELS_OK;
  if (!moments) return MUSA_KERNELS_EINVAL;
  if (IsEmpty(g)) {
    // A replica with no rows: count 0, nothing to merge.
    return static_cast<int>(
        cudaMemsetAsync(moments, 0, sizeof(float) * (2 * channels + 1), stream));
  }
  MUSA_BY_DTYPE(dtype, StatsSums<T>(x, moments, moments + 2 * channels, g, workspace,
                                    workspace_bytes, kTailFwdMoments, stream));
}

// The cross-replica forms: statistics kernel, then a finalize kernel that
// also runs the peer-memory exchange for its own channels, so that `moments`
// / `sums` hold the result over all replicas when the call's work is done and
// no separate exchange kernel sits in the chain.
int LaunchBnStatsMomentsExchange(int dtype, const void* x, float* moments, int64_t outer,
                                 int64_t channels, int64_t inner, void* workspace,
                                 size_t workspace_bytes, void* exchange,
                                 cudaStream_t stream) {
  const Geom g{outer, channels, inner};
  if (int rc = CheckGeom(g)) return rc;
  if (channels == 0) return MUSA_KERNELS_OK;
  if (!moments || !exchange) return MUSA_KERNELS_EINVAL;
  long long slot_floats = 0;
  unsigned* xchg_epoch = nullptr;
  const ExchangeDev* xchg = ExchangeDeviceContext(exchange, &slot_floats, &xchg_epoch);
  if (2 * channels + 1 > slot_floats) return MUSA_KERNELS_ETOOLARGE;
  if (IsEmpty(g)) {
    // A replica with no rows still takes part: zeros through the stand-alone
    // exchange kernel.
    const cudaError_t err =
        cudaMemsetAsync(moments, 0, sizeof(float) * (2 * channels + 1), stream);
    if (err != cudaSuccess) return static_cast<int>(err);
    return LaunchExchangeMoments(exchange, moments, channels, stream);
  }
  MUSA_BY_DTYPE(dtype, StatsSums<T>(x, moments, moments + 2 * channels, g, workspace,
                                    workspace_bytes, kTailFwdMoments, stream, xchg, xchg_epoch));
}

int LaunchBnGradStatsSumsExchange(int dtype, const void* dy, const void* x,
                                  const float* mean, float* sums, int64_t outer,
                                  int64_t channels, int64_t inner, void* workspace,
                                  size_t workspace_bytes, void* exchange,
                                  cudaStream_t stream) {
  const Geom g{outer, channels, inner};
  if (int rc = CheckGeom(g)) return rc;
  if (channels == 0) return MUSA_KERNELS_OK;
  if (!sums || !exchange) return MUSA_KERNELS_EINVAL;
  long long slot_floats = 0;
  unsigned* xchg_epoch = nullptr;
  const ExchangeDev* xchg = ExchangeDeviceContext(exchange, &slot_floats, &xchg_epoch);
  if (2 * channels + 1 > slot_floats) return MUSA_KERNELS_ETOOLARGE;
  if (IsEmpty(g)) {
    const cudaError_t err = cudaMemsetAsync(sums, 0, sizeof(float) * 2 * channels, stream);
    if (err != cudaSuccess) return static_cast<int>(err);
    return LaunchExchangeSums(exchange, sums, 2 * channels, stream);
  }
  MUSA_BY_DTYPE(dtype, GradStatsSums<T>(dy, x, mean, sums, g, workspace, workspace_bytes,
                                        stream, xchg, xchg_epoch));
}

int LaunchBnMergeMoments(const float* gathered, int world, int64_t channels,
                         float* merged, cudaStream_t stream) {
  if (world < 1 || channels < 0) return MUSA_KERNELS_EINVAL;
  if (channels == 0) return MUSA_KERNELS_OK;
  if (!gathered || !merged) return MUSA_KERNELS_EINVAL;
  const int grid = static_cast<int>(CeilDiv(channels, 256));
  BnMergeMomentsKernel<<<grid, 256, 0, stream>>>(gathered, world, channels, merged);
  CountKernelLaunch();
  return LastError();
}

int LaunchBnFinalizeFromSums(const float* sums, double total_count,
                             const float* est_mean, const float* est_var,
                             float* batch_mean, float* batch_var,
                             float* saved_mean, float* saved_var,
                             int64_t channels, float exp_avg_factor,
                             cudaStream_t stream) {
  return FinalizeFromSums(sums, false, total_count, est_mean, est_var, batch_mean,
                          batch_var, saved_mean, saved_var, channels, exp_avg_factor,
                          stream);
}

int LaunchBnApply(int dtype, const void* x, const float* scale,
                  const float* offset, const float* mean, const float* variance,
                  void* y, int64_t outer, int64_t channels, int64_t inner,
                  float epsilon, cudaStream_t stream) {
  MUSA_BY_DTYPE(dtype, FwdInfer<T>(x, scale, offset, mean, variance, y, outer,
                                   channels, inner, epsilon, stream));
}

int LaunchBnGradStatsSums(int dtype, const void* dy, const void* x,
                          const float* mean, float* sums, int64_t outer,
                          int64_t channels, int64_t inner, void* workspace,
                          size_t workspace_bytes, cudaStream_t stream) {
  const Geom g{outer, channels, inner};
  if (int rc = CheckGeom(g)) return rc;
  if (channels == 0) return MUSA_KERNELS_OK;
  if (!sums) return MUSA_KERNELS_EINVAL;
  if (IsEmpty(g)) {
    return static_cast<int>(
        cudaMemsetAsync(sums, 0, sizeof(float) * 2 * channels, stream));
  }
  MUSA_BY_DTYPE(dtype, GradStatsSums<T>(dy, x, mean, sums, g, workspace,
                                        workspace_bytes, stream));
}

int LaunchBnGradApplyFromSums(int dtype, const void* dy, const void* x,
                              const float* scale, const float* mean,
                              const float* variance, const float* sums,
                              double total_count, void* dx, float* dscale,
                              float* doffset, int64_t outer, int64_t channels,
                              int64_t inner, float epsilon,
                              cudaStream_t stream) {
  const Geom g{outer, channels, inner};
  if (int rc = CheckGeom(g)) return rc;
  if (IsEmpty(g)) return MUSA_KERNELS_OK;
  if (!(total_count > 0.0)) return MUSA_KERNELS_EINVAL;
  MUSA_BY_DTYPE(dtype, GradApplyFromSums<T>(dy, x, scale, mean, variance, sums,
                                            total_count, dx, dscale, doffset,
                                            g, epsilon, stream));
}

}  // extern "C"
