// Row-wise normalisations over the last axis: LayerNorm (forward, gradient)
// and RMSNorm (forward, gradient with respect to x).
//
//   MusaLayerNorm      y = (x - mean) * rsqrt(var + eps) * gamma + beta
//                      (musa_ext/kernels/fusion/musa_layernorm_op.cc:26-100)
//   MusaLayerNormGrad  dx, dgamma, dbeta from dy, x, gamma
//                      (musa_ext/kernels/fusion/musa_layernorm_grad_op.cc)
//   MusaRmsNorm        inv = rsqrt(mean(x^2) + eps); normalized = x * inv;
//                      y = normalized * gamma
//                      (musa_ext/kernels/nn/musa_rmsnorm_kernel.mu:58-92)
//   MusaRmsNormGradDx  dx = dy*gamma*inv - x * (sum(x*dy*gamma) * inv^3 / n)
//                      (musa_ext/kernels/nn/musa_rmsnorm_kernel.mu:171-204)
//
// A row is read from HBM once: a group of kGroup threads holds it in registers
// (up to kMaxPacks 128-bit packs per thread), reduces with shuffles (and shared
// memory across warps) and writes the results.  The reference kernels walk the
// row two or three times.  Statistics are fp32; the variance is taken from the
// residuals around a first mean (second in-register pass), so it does not
// cancel.  Rows that do not fit the register form (very long, or not a whole
// number of aligned packs) take a CTA-per-row kernel with element accesses.
#include "common.cuh"
#include "trace.h"
#include "tuning.h"
#include "../../include/musa_plugin_kernels.h"

namespace musa_b200 {
namespace {

constexpr int kOpLnFwd = 0;
constexpr int kOpLnGrad = 1;
constexpr int kOpRmsFwd = 2;
constexpr int kOpRmsGrad = 3;

struct RowArgs {
  const void* x;
  const void* dy;        // gradients (grad ops)
  const void* gamma;
  const void* beta;      // LayerNorm forward
  const void* inv_in;    // RMSNorm gradient: inv_rms from the forward, type T
  void* out;             // y (forward) / dx (gradient)
  void* out2;            // RMSNorm forward: normalized
  void* stat_t;          // RMSNorm forward: inv_rms, type T
  float* mean_out;       // LayerNorm forward, optional fp32 [rows]
  float* inv_std_out;    // LayerNorm forward, optional fp32 [rows]
  float* partial;        // LayerNorm gradient: [ctas][2][row_size]
  int64_t rows;
  int row_size;
  float epsilon;
};

// Sums over the kGroup threads that share a row; every thread of the group
// gets the totals.  Groups are aligned runs of threads, so a group of 32 or
// fewer lives inside one warp (shuffles only); larger groups go through shared
// memory and meet at a barrier - a named one per group when the CTA holds
// several (ids 1 .., barrier 0 stays with __syncthreads).  Successive sums
// alternate between two scratch rows (`parity`), which makes one barrier per
// sum enough: a warp that writes row A for sum k + 2 has passed the barrier of
// sum k + 1, which every warp of the group reaches only after reading row A of
// sum k.  All threads of a group must make the same sequence of calls.
template <int kGroup, int kThreads>
__device__ __forceinline__ void GroupMeet() {
  if constexpr (kGroup == kThreads) {
    __syncthreads();
  } else {
    asm volatile("bar.sync %0, %1;" ::"r"(1 + (threadIdx.x >> 5) / (kGroup / 32)), "n"(kGroup)
                 : "memory");
  }
}

template <int kGroup, int kThreads>
__device__ __forceinline__ float2 GroupSum2(float2 v, float2* smem, int& parity) {
  constexpr int kWarpSpan = kGroup < 32 ? kGroup : 32;
#pragma unroll
  for (int m = kWarpSpan / 2; m > 0; m >>= 1) {
    v.x += __shfl_xor_sync(0xffffffffu, v.x, m);
    v.y += __shfl_xor_sync(0xffffffffu, v.y, m);
  }
  if constexpr (kGroup > 32) {
    constexpr int kWarps = kGroup / 32;
    const int warp = threadIdx.x >> 5;
    const int first = (warp / kWarps) * kWarps;  // first warp of this group
    float2* row = smem + parity * (kThreads / 32);
    parity ^= 1;
    if ((threadIdx.x & 31) == 0) row[warp] = v;
    GroupMeet<kGroup, kThreads>();
    float2 t = make_float2(0.0f, 0.0f);
#pragma unroll
    for (int w = 0; w < kWarps; ++w) {
      const float2 o = row[first + w];
      t.x += o.x;
      t.y += o.y;
    }
    v = t;
  }
  return v;
}

template <int kGroup, int kThreads>
__device__ __forceinline__ float GroupSum(float v, float2* smem, int& parity) {
  constexpr int kWarpSpan = kGroup < 32 ? kGroup : 32;
#pragma unroll
  for (int m = kWarpSpan / 2; m > 0; m >>= 1) v += __shfl_xor_sync(0xffffffffu, v, m);
  if constexpr (kGroup > 32) {
    constexpr int kWarps = kGroup / 32;
    const int warp = threadIdx.x >> 5;
    const int first = (warp / kWarps) * kWarps;
    float2* row = smem + parity * (kThreads / 32);
    parity ^= 1;
    if ((threadIdx.x & 31) == 0) row[warp].x = v;
    GroupMeet<kGroup, kThreads>();
    float t = 0.0f;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) t += row[first + w].x;
    v = t;
  }
  return v;
}

// Per-thread asynchronous 16-byte copies global -> shared.  A thread only ever
// reads back the slots that it filled itself, so waiting for its own copy
// groups is all the synchronisation the ring needs.
__device__ __forceinline__ void AsyncCopy16(void* smem_dst, const void* gmem_src) {
  const unsigned dst = static_cast<unsigned>(__cvta_generic_to_shared(smem_dst));
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(dst), "l"(gmem_src)
               : "memory");
}
__device__ __forceinline__ void AsyncCommit() {
  asm volatile("cp.async.commit_group;\n" ::: "memory");
}
template <int kPending>
__device__ __forceinline__ void AsyncWait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(kPending) : "memory");
}

// Threads per CTA: one group when it is wider than 256, else 256 - except the
// LayerNorm gradient of groups up to 128 threads: it keeps its column sums in
// registers, and 128-thread CTAs then fill an SM in finer steps.  Warp-sized
// groups run two such CTAs per SM at about 190 registers (capping them at 160
// for three CTAs measured 3-6 % slower), groups of 64 and 128 threads three
// at 160 (bf16 rows of 4096: +9 %), groups of 256 threads two 256-thread CTAs
// at 128 where that needs no spills (bf16 rows of 5120: +19 %; with four
// 16-bit packs a thread it spills and runs at 0.6 of the one-CTA form).
// 64-thread CTAs for warp-sized groups (five per SM) measured slower (bf16
// rows of 768: 4.7 against 5.6 TB/s).
__host__ __device__ constexpr int RowThreads(int group, int op) {
  return group > 256 ? group : (op == 1 /* kOpLnGrad */ && group <= 128) ? 128 : 256;
}

template <int kOp>
struct RowPipe {
  static constexpr bool kGrad = kOp == kOpLnGrad || kOp == kOpRmsGrad;
  static constexpr int kInputs = kGrad ? 2 : 1;
};

// Ring stages: three, with two exceptions of two.  The two-input ring of a
// 512-thread LayerNorm-gradient group is 64 KB a stage.  And 16-bit rows of a
// 256-thread group outside the LayerNorm gradient (for which two, three and
// four stages measured alike): their fp32 copies of gamma / beta take 20-64 KB,
// and the shorter ring fits a third CTA per SM (bf16 rows of 5120: LayerNorm
// +12 %, rows of 8192: RMSNorm gradient +32 %; fp32 rows of 4096 measured 7 %
// slower that way and keep three).
__host__ __device__ constexpr int RowStages(int op, int group, int elem_bytes) {
  if (op == 1 /* kOpLnGrad */) return group > 256 ? 2 : 3;
  return (group >= 256 && elem_bytes == 2) ? 2 : 3;
}

// One launch handles all rows; CTA = RowThreads() threads = kRows rows at
// a time, grid-stride over blocks of kRows rows.  The rows travel through a
// ring of shared-memory stages filled by per-thread asynchronous copies:
// while a row block is being worked on, the copies of the CTA's next
// kStages - 1 blocks are in flight, whatever the register budget.  A thread
// keeps its packs of the current row in registers in stored form and widens
// them on each use.
// The single-input forms fit three 256-thread CTAs per SM (56 KB of shared
// memory each) when the compiler keeps them to 85 registers, the RMSNorm
// gradient two (100 KB each, 128 registers).
// The LayerNorm gradient keeps the column sums (dgamma, dbeta) of a thread's
// packs in registers: a thread meets the same columns in every row.  When the
// rows are done the sums go to shared memory (over the ring, which is free by
// then), the row lanes of the CTA are added in lane order and the CTA writes
// one partial row.
// CTAs per SM that the register allocation aims at (see RowThreads for the
// LayerNorm gradient).
constexpr int RowMinCtas(int group, int op, int max_packs, int elem_bytes) {
  if (group > 256) return 1;
  if (op == kOpLnFwd || op == kOpRmsFwd) return 3;
  if (op == kOpRmsGrad) return 2;
  if (group >= 64 && group <= 128) return 3;
  if (group == 256 && (max_packs <= 3 || elem_bytes == 4)) return 2;
  return 1;
}

template <typename T, int kGroup, int kMaxPacks, int kOp, bool kFull>
__global__ void __launch_bounds__(RowThreads(kGroup, kOp),
                                  RowMinCtas(kGroup, kOp, kMaxPacks, sizeof(T)))
    RowNormKernel(RowArgs a) {
  constexpr int kThreads = RowThreads(kGroup, kOp);
  constexpr int kRows = kThreads / kGroup;
  constexpr int kVec = VecWidth<T>::value;
  constexpr bool kGrad = RowPipe<kOp>::kGrad;
  constexpr int kInputs = RowPipe<kOp>::kInputs;
  constexpr int kStages = RowStages(kOp, kGroup, sizeof(T));
  constexpr int kPairs = kVec / 2;
  constexpr int kQuads = kVec / 4;
  using P = Pack<T, kVec>;
  __shared__ float2 red[2 * (kThreads / 32)];
  int parity = 0;
  // Ring: [stage][input][pack j][thread], 16 bytes each.  After the ring:
  // gamma (and beta for the LayerNorm forward) widened to fp32 once per CTA,
  // in quads (see Quad below).
  extern __shared__ uint4 ring[];
  float* gsm = reinterpret_cast<float*>(ring + kStages * kInputs * kMaxPacks * kThreads);
  float* bsm = gsm + a.row_size;
  // LayerNorm gradient, after the last row: one slab [2][kVec / 4][packs][4]
  // of column sums per row lane, laid over the ring.
  float* slab = reinterpret_cast<float*>(ring);

  const int t = threadIdx.x % kGroup;
  const int lane_row = threadIdx.x / kGroup;
  const int packs = a.row_size / kVec;
  const float inv_n = 1.0f / static_cast<float>(a.row_size);
  float* my_slab = slab + static_cast<size_t>(lane_row) * 2 * a.row_size;
  uint4* const mine = ring + threadIdx.x;
  // Pack j of this thread exists; known at compile time for rows that fill the
  // layout (kFull: row_size == kGroup * kMaxPacks packs).
  const auto Has = [&](int j) { return kFull || t + j * kGroup < packs; };
  // Quad h of pack p (elements 4h .. 4h+3) sits at ((h * packs + p) * 4): the
  // 128-bit accesses of neighbouring lanes are 16 bytes apart.
  const auto Quad = [&](const float* base, int h, int p) {
    return *reinterpret_cast<const float4*>(base + (h * packs + p) * 4);
  };
  const auto LoadRowVector = [&](const float* base, int p, float2 (&out)[kPairs]) {
#pragma unroll
    for (int h = 0; h < kQuads; ++h) {
      const float4 v = Quad(base, h, p);
      out[2 * h] = make_float2(v.x, v.y);
      out[2 * h + 1] = make_float2(v.z, v.w);
    }
  };

  // Column sums of this thread's packs (dgamma, dbeta), kept in registers.
  float2 ag[kOp == kOpLnGrad ? kMaxPacks : 1][kPairs];
  float2 ab[kOp == kOpLnGrad ? kMaxPacks : 1][kPairs];
  if constexpr (kOp == kOpLnGrad) {
#pragma unroll
    for (int j = 0; j < kMaxPacks; ++j)
#pragma unroll
      for (int q = 0; q < kPairs; ++q) {
        ag[j][q] = make_float2(0.0f, 0.0f);
        ab[j][q] = make_float2(0.0f, 0.0f);
      }
  }

  GridDepWait();
  GridDepLaunch();

  for (int c = threadIdx.x; c < a.row_size; c += kThreads) {
    const int e = c % kVec;
    const int at = ((e / 4) * packs + c / kVec) * 4 + (e & 3);
    gsm[at] = ToF32(static_cast<const T*>(a.gamma)[c]);
    if constexpr (kOp == kOpLnFwd) bsm[at] = ToF32(static_cast<const T*>(a.beta)[c]);
  }
  __syncthreads();

  const int64_t n_blocks = (a.rows + kRows - 1) / kRows;
  // Queues the copies of row block `rb` into ring stage `stage`; always one
  // commit group, empty when there is nothing to copy.
  auto request = [&](int64_t rb, int stage) {
    const int64_t row = rb * kRows + lane_row;
    if (rb < n_blocks && row < a.rows) {
      const P* xp = reinterpret_cast<const P*>(a.x) + row * packs;
      const P* dp = reinterpret_cast<const P*>(a.dy) + row * packs;
#pragma unroll
      for (int j = 0; j < kMaxPacks; ++j) {
        const int p = t + j * kGroup;
        if (Has(j)) {
          AsyncCopy16(mine + ((stage * kInputs + 0) * kMaxPacks + j) * kThreads, xp + p);
          if constexpr (kGrad) {
            AsyncCopy16(mine + ((stage * kInputs + 1) * kMaxPacks + j) * kThreads, dp + p);
          }
        }
      }
    }
    AsyncCommit();
  };
#pragma unroll
  for (int s = 0; s < kStages - 1; ++s) {
    request(static_cast<int64_t>(blockIdx.x) + static_cast<int64_t>(s) * gridDim.x, s);
  }

  int stage = 0;
  for (int64_t rb = blockIdx.x; rb < n_blocks; rb += gridDim.x) {
    const int64_t row = rb * kRows + lane_row;
    const bool live = row < a.rows;
    {
      int ahead = stage + kStages - 1;
      if (ahead >= kStages) ahead -= kStages;
      request(rb + static_cast<int64_t>(kStages - 1) * gridDim.x, ahead);
    }
    AsyncWait<kStages - 1>();
    P cx[kMaxPacks];
    P cd[kGrad ? kMaxPacks : 1];
#pragma unroll
    for (int j = 0; j < kMaxPacks; ++j) {
      if (live && Has(j)) {
        const uint4 rx = mine[((stage * kInputs + 0) * kMaxPacks + j) * kThreads];
        cx[j] = *reinterpret_cast<const P*>(&rx);
        if constexpr (kGrad) {
          const uint4 rd = mine[((stage * kInputs + 1) * kMaxPacks + j) * kThreads];
          cd[j] = *reinterpret_cast<const P*>(&rd);
        }
      }
    }
    stage = stage + 1 == kStages ? 0 : stage + 1;
    // Widened once; packs that the row does not have read as zeros.
    float2 xv[kMaxPacks][kPairs];
#pragma unroll
    for (int j = 0; j < kMaxPacks; ++j) {
      if (live && Has(j)) {
        WidenPack<kVec>(cx[j], xv[j]);
      } else {
#pragma unroll
        for (int q = 0; q < kPairs; ++q) xv[j][q] = make_float2(0.0f, 0.0f);
      }
    }
    const auto Dup = [](float v) { return make_float2(v, v); };

    if constexpr (kOp == kOpLnFwd || kOp == kOpLnGrad) {
      // A plain fp32 sum of the row can be off by a few ulps of |mean|, which
      // matters when |mean| >> std.  So: a first mean from the plain sum, then
      // one pass over the residuals r = x - mean0 that gives both the
      // correction mean1 = mean(r) and the variance mean(r^2) - mean1^2
      // (mean1 is of rounding size, nothing cancels).  Two group sums a row.
      float2 s2 = make_float2(0.0f, 0.0f);
#pragma unroll
      for (int j = 0; j < kMaxPacks; ++j)
#pragma unroll
        for (int q = 0; q < kPairs; ++q) s2 = Add2(s2, xv[j][q]);
      const float mean0 = GroupSum<kGroup, kThreads>(s2.x + s2.y, red, parity) * inv_n;
      const float2 nmean0 = Dup(-mean0);
      float2 r2 = make_float2(0.0f, 0.0f), q2 = make_float2(0.0f, 0.0f);
#pragma unroll
      for (int j = 0; j < kMaxPacks; ++j) {
        if (live && Has(j)) {
#pragma unroll
          for (int q = 0; q < kPairs; ++q) {
            xv[j][q] = Add2(xv[j][q], nmean0);
            r2 = Add2(r2, xv[j][q]);
            q2 = Fma2(xv[j][q], xv[j][q], q2);
          }
        }
      }
      const float2 rq = GroupSum2<kGroup, kThreads>(
          make_float2(r2.x + r2.y, q2.x + q2.y), red, parity);
      const float mean1 = rq.x * inv_n;
      const float mean = mean0 + mean1;
      const float var = fmaxf(fmaf(-mean1, mean1, rq.y * inv_n), 0.0f);
      const float inv_std = 1.0f / sqrtf(var + a.epsilon);
      const float2 inv2 = Dup(inv_std);
      // x_hat = (r - mean1) * inv_std = r * inv_std + shift
      const float2 shift2 = Dup(-mean1 * inv_std);

      if constexpr (kOp == kOpLnFwd) {
        if (live && t == 0) {
          if (a.mean_out != nullptr) a.mean_out[row] = mean;
          if (a.inv_std_out != nullptr) a.inv_std_out[row] = inv_std;
        }
        P* yp = reinterpret_cast<P*>(a.out) + row * packs;
#pragma unroll
        for (int j = 0; j < kMaxPacks; ++j) {
          const int p = t + j * kGroup;
          if (live && Has(j)) {
            float2 gm[kPairs], bt[kPairs], o2[kPairs];
            LoadRowVector(gsm, p, gm);
            LoadRowVector(bsm, p, bt);
#pragma unroll
            for (int q = 0; q < kPairs; ++q) {
              o2[q] = Fma2(Fma2(xv[j][q], inv2, shift2), gm[q], bt[q]);
            }
            P o;
            NarrowPack<kVec>(o2, o);
            StoreStream(yp + p, o);
          }
        }
      } else {
        // x_hat = (x - mean) * inv_std; g = dy * gamma
        // dx = inv_std * (g - mean(g) - x_hat * mean(g * x_hat))
        float2 sg2 = make_float2(0.0f, 0.0f), sgx2 = make_float2(0.0f, 0.0f);
#pragma unroll
        for (int j = 0; j < kMaxPacks; ++j) {
          const int p = t + j * kGroup;
          if (live && Has(j)) {
            float2 gm[kPairs], dv[kPairs];
            LoadRowVector(gsm, p, gm);
            WidenPack<kVec>(cd[j], dv);
#pragma unroll
            for (int q = 0; q < kPairs; ++q) {
              xv[j][q] = Fma2(xv[j][q], inv2, shift2);  // x_hat from here on
              const float2 g = Mul2(dv[q], gm[q]);
              sg2 = Add2(sg2, g);
              sgx2 = Fma2(g, xv[j][q], sgx2);
            }
          }
        }
        const float2 gs = GroupSum2<kGroup, kThreads>(
            make_float2(sg2.x + sg2.y, sgx2.x + sgx2.y), red, parity);
        const float mg = gs.x * inv_n, mgx = gs.y * inv_n;
        const float2 nmg = Dup(-mg), nmgx = Dup(-mgx);
        P* op = reinterpret_cast<P*>(a.out) + row * packs;
#pragma unroll
        for (int j = 0; j < kMaxPacks; ++j) {
          const int p = t + j * kGroup;
          if (live && Has(j)) {
            float2 gm[kPairs], dv[kPairs], o2[kPairs];
            LoadRowVector(gsm, p, gm);
            WidenPack<kVec>(cd[j], dv);
#pragma unroll
            for (int q = 0; q < kPairs; ++q) {
              const float2 g = Mul2(dv[q], gm[q]);
              o2[q] = Mul2(inv2, Fma2(xv[j][q], nmgx, Add2(g, nmg)));
            }
            P o;
            NarrowPack<kVec>(o2, o);
            StoreStream(op + p, o);
            // Column sums: dgamma += dy * x_hat, dbeta += dy.
#pragma unroll
            for (int q = 0; q < kPairs; ++q) {
              ag[j][q] = Fma2(dv[q], xv[j][q], ag[j][q]);
              ab[j][q] = Add2(ab[j][q], dv[q]);
            }
          }
        }
      }
    } else if constexpr (kOp == kOpRmsFwd) {
      float2 s2 = make_float2(0.0f, 0.0f);
#pragma unroll
      for (int j = 0; j < kMaxPacks; ++j)
#pragma unroll
        for (int q = 0; q < kPairs; ++q) s2 = Fma2(xv[j][q], xv[j][q], s2);
      const float ms = GroupSum<kGroup, kThreads>(s2.x + s2.y, red, parity) * inv_n;
      const float inv = 1.0f / sqrtf(ms + a.epsilon);
      const float2 inv2 = Dup(inv);
      if (live && t == 0) static_cast<T*>(a.stat_t)[row] = FromF32<T>(inv);
      P* yp = reinterpret_cast<P*>(a.out) + row * packs;
      P* np = reinterpret_cast<P*>(a.out2) + row * packs;
#pragma unroll
      for (int j = 0; j < kMaxPacks; ++j) {
        const int p = t + j * kGroup;
        if (live && Has(j)) {
          float2 gm[kPairs], n2[kPairs], o2[kPairs];
          LoadRowVector(gsm, p, gm);
#pragma unroll
          for (int q = 0; q < kPairs; ++q) {
            n2[q] = Mul2(xv[j][q], inv2);
            o2[q] = Mul2(n2[q], gm[q]);
          }
          P o, nrm;
          NarrowPack<kVec>(n2, nrm);
          NarrowPack<kVec>(o2, o);
          StoreStream(np + p, nrm);
          StoreStream(yp + p, o);
        }
      }
    } else {  // kOpRmsGrad
      float2 s2 = make_float2(0.0f, 0.0f);
      float2 gv[kMaxPacks][kPairs];  // dy * gamma
#pragma unroll
      for (int j = 0; j < kMaxPacks; ++j) {
        const int p = t + j * kGroup;
        if (live && Has(j)) {
          float2 gm[kPairs], dv[kPairs];
          LoadRowVector(gsm, p, gm);
          WidenPack<kVec>(cd[j], dv);
#pragma unroll
          for (int q = 0; q < kPairs; ++q) {
            gv[j][q] = Mul2(dv[q], gm[q]);
            s2 = Fma2(xv[j][q], gv[j][q], s2);
          }
        }
      }
      const float dot = GroupSum<kGroup, kThreads>(s2.x + s2.y, red, parity);
      const float inv = live ? ToF32(static_cast<const T*>(a.inv_in)[row]) : 0.0f;
      const float2 inv2 = Dup(inv);
      const float2 ncoeff = Dup(-(dot * inv * inv * inv * inv_n));
      P* op = reinterpret_cast<P*>(a.out) + row * packs;
#pragma unroll
      for (int j = 0; j < kMaxPacks; ++j) {
        const int p = t + j * kGroup;
        if (live && Has(j)) {
          float2 o2[kPairs];
#pragma unroll
          for (int q = 0; q < kPairs; ++q) {
            o2[q] = Fma2(xv[j][q], ncoeff, Mul2(gv[j][q], inv2));
          }
          P o;
          NarrowPack<kVec>(o2, o);
          StoreStream(op + p, o);
        }
      }
    }
  }

  if constexpr (kOp == kOpLnGrad) {
    // One partial row (dgamma part, dbeta part) per CTA: the slabs of the row
    // lanes added in lane order.  Column c of half s sits at
    // ((s * kQuads + (c % kVec) / 4) * packs + c / kVec) * 4 + c % 4.
    // The ring is free once every thread has left the loop: the slabs of the
    // row lanes go there.
    AsyncWait<0>();
    __syncthreads();
#pragma unroll
    for (int j = 0; j < kMaxPacks; ++j) {
      const int p = t + j * kGroup;
      if (Has(j)) {
#pragma unroll
        for (int h = 0; h < kQuads; ++h) {
          *reinterpret_cast<float4*>(my_slab + (h * packs + p) * 4) = make_float4(
              ag[j][2 * h].x, ag[j][2 * h].y, ag[j][2 * h + 1].x, ag[j][2 * h + 1].y);
          *reinterpret_cast<float4*>(my_slab + ((kQuads + h) * packs + p) * 4) = make_float4(
              ab[j][2 * h].x, ab[j][2 * h].y, ab[j][2 * h + 1].x, ab[j][2 * h + 1].y);
        }
      }
    }
    __syncthreads();
    float* out = a.partial + static_cast<int64_t>(blockIdx.x) * 2 * a.row_size;
    for (int c = threadIdx.x; c < 2 * a.row_size; c += kThreads) {
      const int half = c / a.row_size;
      const int col = c - half * a.row_size;
      const int e = col % kVec;
      const int at = ((half * kQuads + e / 4) * packs + col / kVec) * 4 + (e & 3);
      float s = slab[at];
      for (int l = 1; l < kRows; ++l) s += slab[static_cast<size_t>(l) * 2 * a.row_size + at];
      out[c] = s;
    }
  }
}

// CTA-per-row form with element accesses: any row length, any alignment.  The
// row is walked two or three times (the later walks hit L1 / L2).
template <typename T, int kOp>
__global__ void __launch_bounds__(256) RowNormLoopKernel(RowArgs a) {
  constexpr int kThreads = 256;
  __shared__ float2 red[2 * (kThreads / 32)];
  int parity = 0;
  const T* gamma = static_cast<const T*>(a.gamma);
  const int n = a.row_size;
  const float inv_n = 1.0f / static_cast<float>(n);
  GridDepWait();
  GridDepLaunch();
  float* part = a.partial + static_cast<int64_t>(blockIdx.x) * 2 * n;
  if constexpr (kOp == kOpLnGrad) {
    for (int i = threadIdx.x; i < 2 * n; i += kThreads) part[i] = 0.0f;
    __syncthreads();
  }
  for (int64_t row = blockIdx.x; row < a.rows; row += gridDim.x) {
    const T* x = static_cast<const T*>(a.x) + row * n;
    const T* dy = static_cast<const T*>(a.dy) + row * n;
    if constexpr (kOp == kOpLnFwd || kOp == kOpLnGrad) {
      float s = 0.0f;
      for (int i = threadIdx.x; i < n; i += kThreads) s += ToF32(x[i]);
      const float mean0 = GroupSum<kThreads, kThreads>(s, red, parity) * inv_n;
      float r = 0.0f;
      for (int i = threadIdx.x; i < n; i += kThreads) r += ToF32(x[i]) - mean0;
      const float mean = mean0 + GroupSum<kThreads, kThreads>(r, red, parity) * inv_n;
      float q = 0.0f;
      for (int i = threadIdx.x; i < n; i += kThreads) {
        const float d = ToF32(x[i]) - mean;
        q += d * d;
      }
      const float var = GroupSum<kThreads, kThreads>(q, red, parity) * inv_n;
      const float inv_std = 1.0f / sqrtf(var + a.epsilon);
      if constexpr (kOp == kOpLnFwd) {
        const T* beta = static_cast<const T*>(a.beta);
        T* y = static_cast<T*>(a.out) + row * n;
        if (threadIdx.x == 0) {
          if (a.mean_out != nullptr) a.mean_out[row] = mean;
          if (a.inv_std_out != nullptr) a.inv_std_out[row] = inv_std;
        }
        for (int i = threadIdx.x; i < n; i += kThreads) {
          y[i] = FromF32<T>(fmaf((ToF32(x[i]) - mean) * inv_std, ToF32(gamma[i]),
                                 ToF32(beta[i])));
        }
      } else {
        float sg = 0.0f, sgx = 0.0f;
        for (int i = threadIdx.x; i < n; i += kThreads) {
          const float g = ToF32(dy[i]) * ToF32(gamma[i]);
          const float xh = (ToF32(x[i]) - mean) * inv_std;
          sg += g;
          sgx = fmaf(g, xh, sgx);
        }
        const float mg = GroupSum<kThreads, kThreads>(sg, red, parity) * inv_n;
        const float mgx = GroupSum<kThreads, kThreads>(sgx, red, parity) * inv_n;
        T* dx = static_cast<T*>(a.out) + row * n;
        for (int i = threadIdx.x; i < n; i += kThreads) {
          const float d = ToF32(dy[i]);
          const float g = d * ToF32(gamma[i]);
          const float xh = (ToF32(x[i]) - mean) * inv_std;
          dx[i] = FromF32<T>(inv_std * (g - mg - xh * mgx));
          // This thread is the only writer of column i of the CTA's row.
          part[i] = fmaf(d, xh, part[i]);
          part[n + i] += d;
        }
      }
    } else if constexpr (kOp == kOpRmsFwd) {
      float s = 0.0f;
      for (int i = threadIdx.x; i < n; i += kThreads) {
        const float v = ToF32(x[i]);
        s = fmaf(v, v, s);
      }
      const float ms = GroupSum<kThreads, kThreads>(s, red, parity) * inv_n;
      const float inv = 1.0f / sqrtf(ms + a.epsilon);
      if (threadIdx.x == 0) static_cast<T*>(a.stat_t)[row] = FromF32<T>(inv);
      T* y = static_cast<T*>(a.out) + row * n;
      T* nrm = static_cast<T*>(a.out2) + row * n;
      for (int i = threadIdx.x; i < n; i += kThreads) {
        const float v = ToF32(x[i]) * inv;
        nrm[i] = FromF32<T>(v);
        y[i] = FromF32<T>(v * ToF32(gamma[i]));
      }
    } else {
      float s = 0.0f;
      for (int i = threadIdx.x; i < n; i += kThreads) {
        s = fmaf(ToF32(x[i]), ToF32(dy[i]) * ToF32(gamma[i]), s);
      }
      const float dot = GroupSum<kThreads, kThreads>(s, red, parity);
      const float inv = ToF32(static_cast<const T*>(a.inv_in)[row]);
      const float coeff = dot * inv * inv * inv * inv_n;
      T* dx = static_cast<T*>(a.out) + row * n;
      for (int i = threadIdx.x; i < n; i += kThreads) {
        dx[i] = FromF32<T>(ToF32(dy[i]) * ToF32(gamma[i]) * inv - ToF32(x[i]) * coeff);
      }
    }
  }
}

// dgamma / dbeta = sum over the CTAs' partial rows, fixed order, fp64.
template <typename T>
__global__ void __launch_bounds__(256)
    LnGradFinalizeKernel(const float* __restrict__ partial, int n_partial,
                         int row_size, T* __restrict__ dgamma,
                         T* __restrict__ dbeta) {
  constexpr int kCh = 8, kLanes = 32;
  __shared__ double red[256];
  const int tc = threadIdx.x % kCh;
  const int tl = threadIdx.x / kCh;
  const int c = blockIdx.x * kCh + tc;  // column of the [2 * row_size] row
  GridDepWait();
  GridDepLaunch();
  double s0 = 0.0, s1 = 0.0;
  if (c < 2 * row_size) {
    int p = tl;
    for (; p + kLanes < n_partial; p += 2 * kLanes) {
      const float v0 = partial[static_cast<int64_t>(p) * 2 * row_size + c];
      const float v1 = partial[static_cast<int64_t>(p + kLanes) * 2 * row_size + c];
      s0 += v0;
      s1 += v1;
    }
    for (; p < n_partial; p += kLanes) {
      s0 += partial[static_cast<int64_t>(p) * 2 * row_size + c];
    }
  }
  double s = s0 + s1;
  red[threadIdx.x] = s;
  __syncthreads();
  if (tl == 0 && c < 2 * row_size) {
    for (int l = 1; l < kLanes; ++l) s += red[l * kCh + tc];
    if (c < row_size) {
      dgamma[c] = FromF32<T>(static_cast<float>(s));
    } else {
      dbeta[c - row_size] = FromF32<T>(static_cast<float>(s));
    }
  }
}

// ---------------------------------------------------------------------------

constexpr int kMaxCtasPerSm = 8;
constexpr int kMaxGradCtasPerSm = 4;  // bounds the partial rows of the gradient

inline int MaxGradCtas() { return SmCount() * kMaxGradCtasPerSm; }

// Dynamic shared memory of RowNormKernel: ring and widened gamma (and beta).
// The column-sum slabs of the LayerNorm gradient lie over the ring: the slabs
// of a CTA (2 * row_size floats per row lane) are never larger than two
// stages of the two-input ring.
template <int kOp>
size_t RowSmemBytes(int group, int elem_bytes, int threads, int max_packs, int row_size) {
  size_t bytes = static_cast<size_t>(RowStages(kOp, group, elem_bytes)) * RowPipe<kOp>::kInputs *
                 max_packs * threads * 16;
  bytes += static_cast<size_t>(kOp == kOpLnFwd ? 2 : 1) * row_size * sizeof(float);
  return bytes;
}

template <typename T, int kGroup, int kMaxPacks, int kOp, bool kFull>
int LaunchGroupAs(const RowArgs& a, int* ctas_out, cudaStream_t stream) {
  constexpr int kThreads = RowThreads(kGroup, kOp);
  constexpr int kRows = kThreads / kGroup;
  auto kernel = RowNormKernel<T, kGroup, kMaxPacks, kOp, kFull>;
  size_t smem = RowSmemBytes<kOp>(kGroup, sizeof(T), kThreads, kMaxPacks, a.row_size);
  // Function attributes and occupancy are per-device state; both are cached
  // per device for this instantiation.  The shared-memory size depends on the
  // row length, so the attribute is raised when a longer row arrives and the
  // occupancy is remembered for the latest size (a model repeats its shapes).
  static std::atomic<int> carveout_by_device[kMaxDevices];
  static std::atomic<int> smem_limit_by_device[kMaxDevices];
  static std::atomic<long long> occupancy_by_device[kMaxDevices];
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    cudaGetLastError();
    return static_cast<int>(cudaErrorInvalidDevice);
  }
  // Ask for the largest shared-memory carve-out: the ring, not L1, is what
  // these kernels live on, and the default carve-out fits fewer CTAs.
  PerDevice(carveout_by_device, [&] {
    cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout,
                         cudaSharedmemCarveoutMaxShared);
    cudaGetLastError();
    return 1;
  });
  if (smem > 40 * 1024 &&
      static_cast<int>(smem) > smem_limit_by_device[dev].load(std::memory_order_acquire)) {
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             static_cast<int>(smem)) != cudaSuccess) {
      return static_cast<int>(cudaGetLastError());
    }
    smem_limit_by_device[dev].store(static_cast<int>(smem), std::memory_order_release);
  }
  int per_sm = 0;
  const long long cached = occupancy_by_device[dev].load(std::memory_order_acquire);
  if (cached != 0 && (cached >> 8) == static_cast<long long>(smem)) {
    per_sm = static_cast<int>(cached & 0xff);
  } else {
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, kThreads, smem) !=
            cudaSuccess ||
        per_sm < 1) {
      cudaGetLastError();
      per_sm = 1;
    }
    if (per_sm > 255) per_sm = 255;
    occupancy_by_device[dev].store((static_cast<long long>(smem) << 8) | per_sm,
                                   std::memory_order_release);
  }
  constexpr int kCap = kOp == kOpLnGrad ? kMaxGradCtasPerSm : kMaxCtasPerSm;
  if (per_sm > kCap) per_sm = kCap;
  const int64_t need = CeilDiv(a.rows, kRows);
  int64_t grid = static_cast<int64_t>(SmCount()) * per_sm;
  if (grid > need) grid = need;
  *ctas_out = static_cast<int>(grid);
  return static_cast<int>(LaunchChained(true, kernel, dim3(static_cast<unsigned>(grid)),
                                        dim3(kThreads), smem, stream, a));
}

template <typename T, int kGroup, int kMaxPacks, int kOp>
int LaunchGroup(const RowArgs& a, int* ctas_out, cudaStream_t stream) {
  // Rows that fill the layout need no per-pack presence checks.  Only the
  // LayerNorm gradient gains from the specialised form (fp32 rows of 1024:
  // +8 %); the forward kernels measured the same or, where the compiler then
  // spills under their register cap, slower.
  if constexpr (kOp == kOpLnGrad) {
    if (a.row_size / VecWidth<T>::value == kGroup * kMaxPacks) {
      return LaunchGroupAs<T, kGroup, kMaxPacks, kOp, true>(a, ctas_out, stream);
    }
  }
  return LaunchGroupAs<T, kGroup, kMaxPacks, kOp, false>(a, ctas_out, stream);
}

template <typename T, int kOp>
int LaunchLoop(const RowArgs& a, int* ctas_out, cudaStream_t stream) {
  int64_t grid = static_cast<int64_t>(SmCount()) *
                 (kOp == kOpLnGrad ? kMaxGradCtasPerSm : kMaxCtasPerSm);
  if (grid > a.rows) grid = a.rows;
  *ctas_out = static_cast<int>(grid);
  return static_cast<int>(LaunchChained(true, RowNormLoopKernel<T, kOp>,
                                        dim3(static_cast<unsigned>(grid)), dim3(256), 0,
                                        stream, a));
}

template <typename T, int kOp, int kMaxPacks>
int DispatchPacks(const RowArgs& a, int* ctas_out, cudaStream_t stream) {
  constexpr int kVec = VecWidth<T>::value;
  const int packs = a.row_size / kVec;
  const auto fits = [&](int group) {
    if (packs > group * kMaxPacks) return false;
    const int threads = RowThreads(group, kOp);
    return RowSmemBytes<kOp>(group, sizeof(T), threads, kMaxPacks, a.row_size) <= 200 * 1024;
  };
  if (fits(8)) return LaunchGroup<T, 8, kMaxPacks, kOp>(a, ctas_out, stream);
  if (fits(32)) return LaunchGroup<T, 32, kMaxPacks, kOp>(a, ctas_out, stream);
  // Two-warp groups: measured better than a half-filled 128-thread group for
  // 16-bit rows (bf16 rows of 2048: LayerNorm 5.6 against 3.8 TB/s), worse for
  // fp32 rows of the same byte length.
  if constexpr (kMaxPacks == 2 || kMaxPacks == 3 || sizeof(T) == 2) {
    if (fits(64)) return LaunchGroup<T, 64, kMaxPacks, kOp>(a, ctas_out, stream);
  }
  if (fits(128)) return LaunchGroup<T, 128, kMaxPacks, kOp>(a, ctas_out, stream);
  if (fits(256)) return LaunchGroup<T, 256, kMaxPacks, kOp>(a, ctas_out, stream);
  if (fits(512)) return LaunchGroup<T, 512, kMaxPacks, kOp>(a, ctas_out, stream);
  return -1;  // no register layout holds this row
}

template <typename T, int kOp>
int Dispatch(const RowArgs& a, bool aligned, int* ctas_out, cudaStream_t stream) {
  constexpr int kVec = VecWidth<T>::value;
  if (aligned && a.row_size % kVec == 0) {
    // Packs per thread.  Four keep short rows inside one warp (shuffle-only
    // sums) and measured best for rows that fill the layout.  Rows of 3 * 2^k
    // packs (768, 1536, 3072 ... bf16 columns) take three: the layout is then
    // full again, with three quarters of the registers and of the ring (bf16
    // LayerNorm gradient of 768 columns: 5.6 against 4.5 TB/s).  Rows that
    // fill less than half of the four-pack layout of their group take two
    // (fp32 rows of 768: LayerNorm 5.5 against 4.6 TB/s); the LayerNorm
    // gradient, whose column sums live in registers, also at exactly half
    // (fp32 rows of 1024: 5.6 against 5.1 - the other ops measured the same
    // or slower there).  Tuning values 1 .. 4 force a layout.
    int want = GetTuning(kTuneRowNormPacks);
    if (want < 1 || want > 4) {
      want = 4;
      const int packs = a.row_size / kVec;
      int group = 512;
      for (int g : {8, 32, 64, 128, 256}) {
        if (g == 64 && sizeof(T) != 2) continue;  // as in DispatchPacks
        if (packs <= 4 * g) {
          group = g;
          break;
        }
      }
      if (packs < 2 * group || (packs == 2 * group && kOp == kOpLnGrad)) {
        want = 2;
      } else if (packs <= 3 * group && packs > 2 * group) {
        want = 3;
      }
    }
    int rc = -1;
    if (want == 1) rc = DispatchPacks<T, kOp, 1>(a, ctas_out, stream);
    if (want == 2) rc = DispatchPacks<T, kOp, 2>(a, ctas_out, stream);
    if (want == 3) rc = DispatchPacks<T, kOp, 3>(a, ctas_out, stream);
    if (rc == -1) rc = DispatchPacks<T, kOp, 4>(a, ctas_out, stream);
    if (rc != -1) return rc;
  }
  return LaunchLoop<T, kOp>(a, ctas_out, stream);
}

inline bool BadRows(int64_t rows, int64_t row_size) {
  return rows < 0 || row_size < 0 || row_size > (int64_t(1) << 24);
}

template <typename T>
int LayerNormFwd(const void* x, const void* gamma, const void* beta, void* y,
                 float* mean_out, float* inv_std_out, int64_t rows,
                 int64_t row_size, float epsilon, cudaStream_t stream) {
  if (BadRows(rows, row_size)) return MUSA_KERNELS_EINVAL;
  MUSA_TRACE("LaunchLayerNorm", 2 * sizeof(T) * rows * row_size);
  if (rows == 0 || row_size == 0) return MUSA_KERNELS_OK;
  if (x == nullptr || gamma == nullptr || beta == nullptr || y == nullptr) {
    return MUSA_KERNELS_EINVAL;
  }
  RowArgs a = {};
  a.x = x;
  a.gamma = gamma;
  a.beta = beta;
  a.out = y;
  a.mean_out = mean_out;
  a.inv_std_out = inv_std_out;
  a.rows = rows;
  a.row_size = static_cast<int>(row_size);
  a.epsilon = epsilon;
  int ctas = 0;
  const bool aligned = Aligned16(x) && Aligned16(gamma) && Aligned16(beta) && Aligned16(y);
  const int rc = Dispatch<T, kOpLnFwd>(a, aligned, &ctas, stream);
  return rc != 0 ? rc : static_cast<int>(cudaGetLastError());
}

template <typename T>
int LayerNormGrad(const void* dy, const void* x, const void* gamma, void* dx,
                  void* dgamma, void* dbeta, int64_t rows, int64_t row_size,
                  float epsilon, void* workspace, size_t workspace_bytes,
                  cudaStream_t stream) {
  if (BadRows(rows, row_size)) return MUSA_KERNELS_EINVAL;
  MUSA_TRACE("LaunchLayerNormGrad", 3 * sizeof(T) * rows * row_size);
  if (row_size == 0) return MUSA_KERNELS_OK;
  if (dgamma == nullptr || dbeta == nullptr) return MUSA_KERNELS_EINVAL;
  if (rows == 0) {
    cudaMemsetAsync(dgamma, 0, sizeof(T) * row_size, stream);
    cudaMemsetAsync(dbeta, 0, sizeof(T) * row_size, stream);
    return static_cast<int>(cudaGetLastError());
  }
  if (dy == nullptr || x == nullptr || gamma == nullptr || dx == nullptr) {
    return MUSA_KERNELS_EINVAL;
  }
  const size_t need = static_cast<size_t>(MaxGradCtas()) * 2 * row_size * sizeof(float);
  if (workspace == nullptr || workspace_bytes < need ||
      (reinterpret_cast<uintptr_t>(workspace) & 15u) != 0) {
    return MUSA_KERNELS_EWORKSPACE;
  }
  RowArgs a = {};
  a.x = x;
  a.dy = dy;
  a.gamma = gamma;
  a.out = dx;
  a.partial = static_cast<float*>(workspace);
  a.rows = rows;
  a.row_size = static_cast<int>(row_size);
  a.epsilon = epsilon;
  int ctas = 0;
  const bool aligned = Aligned16(x) && Aligned16(dy) && Aligned16(gamma) && Aligned16(dx);
  int rc = Dispatch<T, kOpLnGrad>(a, aligned, &ctas, stream);
  if (rc != 0) return rc;
  rc = static_cast<int>(LaunchChained(
      true, LnGradFinalizeKernel<T>,
      dim3(static_cast<unsigned>(CeilDiv(2 * row_size, 8))), dim3(256), 0, stream,
      static_cast<const float*>(a.partial), ctas, a.row_size, static_cast<T*>(dgamma),
      static_cast<T*>(dbeta)));
  return rc != 0 ? rc : static_cast<int>(cudaGetLastError());
}

template <typename T>
void RmsNormFwd(const void* x, const void* gamma, void* y, void* normalized,
                void* inv_rms, int64_t rows, int64_t row_size, float epsilon,
                cudaStream_t stream) {
  MUSA_TRACE("LaunchRmsNorm", rows > 0 && row_size > 0 ? 3 * sizeof(T) * rows * row_size : 0);
  if (rows <= 0 || row_size <= 0 || row_size > (int64_t(1) << 24)) return;
  RowArgs a = {};
  a.x = x;
  a.gamma = gamma;
  a.out = y;
  a.out2 = normalized;
  a.stat_t = inv_rms;
  a.rows = rows;
  a.row_size = static_cast<int>(row_size);
  a.epsilon = epsilon;
  int ctas = 0;
  const bool aligned =
      Aligned16(x) && Aligned16(gamma) && Aligned16(y) && Aligned16(normalized);
  Dispatch<T, kOpRmsFwd>(a, aligned, &ctas, stream);
}

template <typename T>
void RmsNormGradDx(const void* x, const void* inv_rms, const void* gamma,
                   const void* dy, void* dx, int64_t rows, int64_t row_size,
                   cudaStream_t stream) {
  MUSA_TRACE("LaunchRmsNormGradDx",
             rows > 0 && row_size > 0 ? 3 * sizeof(T) * rows * row_size : 0);
  if (rows <= 0 || row_size <= 0 || row_size > (int64_t(1) << 24)) return;
  RowArgs a = {};
  a.x = x;
  a.dy = dy;
  a.gamma = gamma;
  a.inv_in = inv_rms;
  a.out = dx;
  a.rows = rows;
  a.row_size = static_cast<int>(row_size);
  int ctas = 0;
  const bool aligned = Aligned16(x) && Aligned16(gamma) && Aligned16(dy) && Aligned16(dx);
  Dispatch<T, kOpRmsGrad>(a, aligned, &ctas, stream);
}

}  // namespace
}  // namespace musa_b200

using namespace musa_b200;

extern "C" {

size_t LayerNormGradWorkspaceBytes(int64_t rows, int64_t row_size) {
  if (BadRows(rows, row_size) || rows == 0 || row_size == 0) return 0;
  return static_cast<size_t>(MaxGradCtas()) * 2 * row_size * sizeof(float);
}

#define MUSA_DEFINE_LAYER_NORM(SUFFIX, TYPE)                                    \
  int LaunchLayerNorm_##SUFFIX(const void* x, const void* gamma,                \
                               const void* beta, void* y, float* mean,          \
                               float* inv_std, int64_t rows, int64_t row_size,  \
                               float epsilon, cudaStream_t stream) {            \
    return LayerNormFwd<TYPE>(x, gamma, beta, y, mean, inv_std, rows, row_size, \
                              epsilon, stream);                                 \
  }                                                                             \
  int LaunchLayerNormGrad_##SUFFIX(                                             \
      const void* dy, const void* x, const void* gamma, void* dx, void* dgamma, \
      void* dbeta, int64_t rows, int64_t row_size, float epsilon,               \
      void* workspace, size_t workspace_bytes, cudaStream_t stream) {           \
    return LayerNormGrad<TYPE>(dy, x, gamma, dx, dgamma, dbeta, rows, row_size, \
                               epsilon, workspace, workspace_bytes, stream);    \
  }
MUSA_DEFINE_LAYER_NORM(F32, float)
MUSA_DEFINE_LAYER_NORM(F16, __half)
MUSA_DEFINE_LAYER_NORM(BF16, __nv_bfloat16)
#undef MUSA_DEFINE_LAYER_NORM

void LaunchRmsNormFloat(const float* x, const float* gamma, float* y,
                        float* normalized, float* inv_rms, int64_t num_rows,
                        int64_t row_size, float epsilon, cudaStream_t stream) {
  RmsNormFwd<float>(x, gamma, y, normalized, inv_rms, num_rows, row_size, epsilon, stream);
}
void LaunchRmsNormBFloat16(const void* x, const void* gamma, void* y,
                           void* normalized, void* inv_rms, int64_t num_rows,
                           int64_t row_size, float epsilon, cudaStream_t stream) {
  RmsNormFwd<__nv_bfloat16>(x, gamma, y, normalized, inv_rms, num_rows, row_size, epsilon,
                            stream);
}
void LaunchRmsNormGradDxFloat(const float* x, const float* inv_rms,
                              const float* gamma, const float* dy, float* dx,
                              int64_t num_rows, int64_t row_size,
                              cudaStream_t stream) {
  RmsNormGradDx<float>(x, inv_rms, gamma, dy, dx, num_rows, row_size, stream);
}
void LaunchRmsNormGradDxBFloat16(const void* x, const void* inv_rms,
                                 const void* gamma, const void* dy, void* dx,
                                 int64_t num_rows, int64_t row_size,
                                 cudaStream_t stream) {
  RmsNormGradDx<__nv_bfloat16>(x, inv_rms, gamma, dy, dx, num_rows, row_size, stream);
}

}  // extern "C"
