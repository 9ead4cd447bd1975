// Cross-replica sum of small per-channel vectors, done by the GPUs themselves
// over NVLink peer memory: the exchange step of cross-replica BatchNorm
// (2*C + 1 floats per layer and pass) without a collective-library launch.
//
// Every replica owns one buffer in its OWN memory:
//     cell[2 slots][world][slot_floats]    8-byte cells (epoch << 32 | value bits)
// written by the peers (and by itself).  A cell is ONE 64-bit scalar, stored
// and loaded with single relaxed system-scope accesses, which the PTX memory
// model makes single-copy atomic: a reader sees either the old cell or the
// new one, never a mix, and the epoch inside the cell says whether the value
// is the one it waits for.  No separate flag and no memory fence are needed
// (the latency of one exchange is one NVLink store plus a poll).
// One exchange = one single-CTA kernel per replica:
//   1. epoch = local counter + 1 (a device-side counter, so a captured CUDA
//      graph replays correctly); slot = epoch & 1;
//   2. push: store {v[i], epoch} into cell[slot][rank][i] of EVERY replica
//      (plain stores to peer-mapped addresses);
//   3. gather, in its own memory: for each i, read cell[slot][q][i] for every
//      q and poll the ones whose epoch is still old.  The poll is bounded:
//      after kSpinLimit tries (about a second) the kernel records which
//      replica was missing in a status word and stops waiting for that replica
//      - for the rest of this exchange and, while the host has not read the
//      status word, in every later exchange - so a lost peer costs one wait,
//      not one per cell, and never hangs a GPU;
//   4. combine over q = 0..world-1, in rank order, so every replica gets
//      bit-identical results, written over the input vector: the plain sum,
//      or (moments mode, the forward of cross-replica BatchNorm) the merge of
//      per-replica [mean[C], M2[C], count] into the moments of the union.
// Two slots suffice: a replica can publish epoch e+2 only after it consumed
// e+1, which needs every replica to have published e+1, which each does only
// after consuming e.
//
// Remote data always lands in the consumer's local memory first and is read
// from there; no multicast object and no remote load is involved.
//
// The reference has no collective backend to take over from
// (musa_ext/mu/collective/musa_collective_runtime.cc:58-63 returns
// Unimplemented).
#include <cuda_runtime.h>

#include <cstring>
#include <new>

#include "common.cuh"
#include "exchange_dev.cuh"
#include "trace.h"
#include "../../include/musa_plugin_kernels.h"

namespace musa_b200 {
namespace {

struct ExchangeHost {
  ExchangeDev dev;
  ExchangeDev* dev_copy;  // device copy of `dev`
  void* base;             // the local allocation
  size_t bytes;
  void* opened[kMaxWorld];  // IPC mappings to close
  int device;
};

size_t Align256(size_t n) { return (n + 255) / 256 * 256; }

template <int kWorld>  // 0: run-time world size
__device__ __forceinline__ void ExchangeBody(const ExchangeDev& c, float* vec, int n,
                                             unsigned epoch, int mode, unsigned* dead) {
  constexpr int kW = kWorld > 0 ? kWorld : kMaxWorld;
  const int world = kWorld > 0 ? kWorld : c.world;
  const int slot = static_cast<int>(epoch & 1u);
  const long long slot_base = static_cast<long long>(slot) * world * c.slot_floats;
  const long long mine = slot_base + static_cast<long long>(c.rank) * c.slot_floats;

  // 2. push the local vector into every replica's memory.
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const unsigned long long cell = MakeCell(vec[i], epoch);
#pragma unroll
    for (int p = 0; p < kW; ++p) {
      if (p < world) StoreCell(c.cells[p] + mine + i, cell);
    }
  }

  // The combine step overwrites `vec`; in moments mode a thread's outputs are
  // not the elements it pushed, so every push has to be issued first.
  __syncthreads();

  // 3. + 4. gather from local memory and combine in rank order.
  const unsigned long long* local = c.cells[c.rank] + slot_base;
  if (mode == kExchangeSum) {
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
      unsigned long long got[kW];
#pragma unroll
      for (int q = 0; q < kW; ++q) {
        if (q < world) got[q] = LoadCell(local + static_cast<long long>(q) * c.slot_floats + i);
      }
      float total = 0.0f;
#pragma unroll
      for (int q = 0; q < kW; ++q) {
        if (q < world) {
          if (CellEpoch(got[q]) != epoch) {
            got[q] = AwaitCell(local + static_cast<long long>(q) * c.slot_floats + i, epoch, q,
                               dead, c.status);
          }
          total += CellValue(got[q]);
        }
      }
      vec[i] = total;
    }
    return;
  }
  // Moments: vec = [mean[C], M2[C], count], n = 2 * C + 1.  The union of the
  // replicas' rows has  N = sum n_q,  mean = sum n_q mean_q / N,
  // M2 = sum M2_q + sum n_q (mean_q - mean)^2  (fp64, rank order).
  const int channels = (n - 1) / 2;
  double counts[kW];
  double total_count = 0.0;
  {
    // All count cells at once; only the ones that have not arrived are polled.
    unsigned long long gn[kW];
#pragma unroll
    for (int q = 0; q < kW; ++q) {
      if (q < world) {
        gn[q] = LoadCell(local + static_cast<long long>(q) * c.slot_floats + 2 * channels);
      }
    }
#pragma unroll
    for (int q = 0; q < kW; ++q) {
      if (q < world) {
        if (CellEpoch(gn[q]) != epoch) {
          gn[q] = AwaitCell(local + static_cast<long long>(q) * c.slot_floats + 2 * channels,
                            epoch, q, dead, c.status);
        }
        counts[q] = static_cast<double>(CellValue(gn[q]));
        total_count += counts[q];
      }
    }
  }
  const double inv_total = total_count > 0.0 ? 1.0 / total_count : 0.0;
  for (int ch = threadIdx.x; ch < channels; ch += blockDim.x) {
    unsigned long long gm[kW], gs[kW];
#pragma unroll
    for (int q = 0; q < kW; ++q) {
      if (q < world) {
        const unsigned long long* base = local + static_cast<long long>(q) * c.slot_floats;
        gm[q] = LoadCell(base + ch);
        gs[q] = LoadCell(base + channels + ch);
      }
    }
    double mean = 0.0;
#pragma unroll
    for (int q = 0; q < kW; ++q) {
      if (q < world) {
        const unsigned long long* base = local + static_cast<long long>(q) * c.slot_floats;
        if (CellEpoch(gm[q]) != epoch) gm[q] = AwaitCell(base + ch, epoch, q, dead, c.status);
        if (CellEpoch(gs[q]) != epoch) {
          gs[q] = AwaitCell(base + channels + ch, epoch, q, dead, c.status);
        }
        mean += counts[q] * static_cast<double>(CellValue(gm[q]));
      }
    }
    mean *= inv_total;
    double m2 = 0.0;
#pragma unroll
    for (int q = 0; q < kW; ++q) {
      if (q < world) {
        const double d = static_cast<double>(CellValue(gm[q])) - mean;
        m2 += static_cast<double>(CellValue(gs[q])) + counts[q] * d * d;
      }
    }
    vec[ch] = static_cast<float>(mean);
    vec[channels + ch] = static_cast<float>(m2);
  }
  __syncthreads();  // every thread has read its own count input by now
  if (threadIdx.x == 0) vec[2 * channels] = static_cast<float>(total_count);
}

__global__ void __launch_bounds__(kExchangeThreads)
    ExchangeSumsKernel(const ExchangeDev* ctxs, float* const* vectors,
                       float* single_vector, int n, int mode) {
  GridDepWait();
  GridDepLaunch();
  const ExchangeDev& c = ctxs[blockIdx.x];
  float* vec = vectors != nullptr ? vectors[blockIdx.x] : single_vector;
  const unsigned epoch = *c.epoch + 1u;  // nobody writes it before the barrier below
  // A replica that an earlier exchange gave up on (the host has not read the
  // status word yet) is not waited for again.
  __shared__ unsigned dead;
  if (threadIdx.x == 0) {
    const int st = *reinterpret_cast<volatile int*>(c.status);
    dead = st > 0 && st <= kMaxWorld ? 1u << (st - 1) : 0u;
  }
  __syncthreads();
  switch (c.world) {
    case 1: ExchangeBody<1>(c, vec, n, epoch, mode, &dead); break;
    case 2: ExchangeBody<2>(c, vec, n, epoch, mode, &dead); break;
    case 4: ExchangeBody<4>(c, vec, n, epoch, mode, &dead); break;
    case 8: ExchangeBody<8>(c, vec, n, epoch, mode, &dead); break;
    default: ExchangeBody<0>(c, vec, n, epoch, mode, &dead); break;
  }
  __syncthreads();
  if (threadIdx.x == 0) *c.epoch = epoch;
}

}  // namespace

const ExchangeDev* ExchangeDeviceContext(void* handle, long long* slot_floats,
                                         unsigned** epoch) {
  auto* h = static_cast<ExchangeHost*>(handle);
  if (h == nullptr) return nullptr;
  if (slot_floats != nullptr) *slot_floats = h->dev.slot_floats;
  if (epoch != nullptr) *epoch = h->dev.epoch;
  return h->dev_copy;
}

}  // namespace musa_b200

using namespace musa_b200;

extern "C" {

void* MusaExchangeCreate(int rank, int world, int64_t max_floats) {
  if (rank < 0 || world < 1 || world > kMaxWorld || rank >= world || max_floats < 1) {
    return nullptr;
  }
  auto* h = new (std::nothrow) ExchangeHost();
  if (h == nullptr) return nullptr;
  std::memset(h, 0, sizeof(*h));
  if (cudaGetDevice(&h->device) != cudaSuccess) {
    delete h;
    return nullptr;
  }
  const long long slot_floats = static_cast<long long>(Align256(max_floats * 4) / 4);
  const size_t cell_bytes = Align256(sizeof(unsigned long long) * 2 * world * slot_floats);
  h->bytes = cell_bytes + 256 /*epoch*/ + 256 /*status*/ + Align256(sizeof(ExchangeDev));
  if (cudaMalloc(&h->base, h->bytes) != cudaSuccess ||
      cudaMemset(h->base, 0, h->bytes) != cudaSuccess) {
    cudaGetLastError();
    if (h->base) cudaFree(h->base);
    delete h;
    return nullptr;
  }
  char* p = static_cast<char*>(h->base);
  h->dev.rank = rank;
  h->dev.world = world;
  h->dev.slot_floats = slot_floats;
  h->dev.cells[rank] = reinterpret_cast<unsigned long long*>(p);
  h->dev.epoch = reinterpret_cast<unsigned*>(p + cell_bytes);
  h->dev.status = reinterpret_cast<int*>(p + cell_bytes + 256);
  h->dev_copy = reinterpret_cast<ExchangeDev*>(p + cell_bytes + 512);
  return h;
}

// 64-byte CUDA IPC handle of the local buffer, for the other processes.
int MusaExchangeIpcHandle(void* handle, void* out64) {
  auto* h = static_cast<ExchangeHost*>(handle);
  if (h == nullptr || out64 == nullptr) return MUSA_KERNELS_EINVAL;
  cudaIpcMemHandle_t ipc;
  const cudaError_t err = cudaIpcGetMemHandle(&ipc, h->base);
  if (err != cudaSuccess) return static_cast<int>(err);
  static_assert(sizeof(ipc) == 64, "CUDA IPC handles are 64 bytes");
  std::memcpy(out64, &ipc, 64);
  return 0;
}

// `handles`: world x 64 bytes, the IPC handles of all replicas in rank order
// (the local entry is ignored).  Maps every peer buffer and uploads the table.
int MusaExchangeOpenPeers(void* handle, const void* handles) {
  auto* h = static_cast<ExchangeHost*>(handle);
  if (h == nullptr || (handles == nullptr && h->dev.world > 1)) return MUSA_KERNELS_EINVAL;
  for (int q = 0; q < h->dev.world; ++q) {
    if (q == h->dev.rank) continue;
    cudaIpcMemHandle_t ipc;
    std::memcpy(&ipc, static_cast<const char*>(handles) + 64 * q, 64);
    void* mapped = nullptr;
    const cudaError_t err =
        cudaIpcOpenMemHandle(&mapped, ipc, cudaIpcMemLazyEnablePeerAccess);
    if (err != cudaSuccess) return static_cast<int>(err);
    h->opened[q] = mapped;
    h->dev.cells[q] = static_cast<unsigned long long*>(mapped);
  }
  return static_cast<int>(
      cudaMemcpy(h->dev_copy, &h->dev, sizeof(ExchangeDev), cudaMemcpyHostToDevice));
}

// In place: `vector` (n floats, local device memory) becomes the sum over all
// replicas.  One single-CTA kernel on `stream`; no host synchronisation.
namespace {
int LaunchExchange(void* handle, float* vector, int64_t n, int mode, cudaStream_t stream) {
  auto* h = static_cast<ExchangeHost*>(handle);
  if (h == nullptr || vector == nullptr || n < 0) return MUSA_KERNELS_EINVAL;
  if (n > h->dev.slot_floats) return MUSA_KERNELS_ETOOLARGE;
  MUSA_TRACE("LaunchExchange", 4 * n);
  if (n == 0) return MUSA_KERNELS_OK;
  const cudaError_t err = LaunchChained(
      true, ExchangeSumsKernel, dim3(1), dim3(kExchangeThreads), 0, stream,
      static_cast<const ExchangeDev*>(h->dev_copy), static_cast<float* const*>(nullptr),
      vector, static_cast<int>(n), mode);
  if (err != cudaSuccess) {
    cudaGetLastError();
    return static_cast<int>(err);
  }
  return MUSA_KERNELS_OK;
}
}  // namespace

int LaunchExchangeSums(void* handle, float* vector, int64_t n, cudaStream_t stream) {
  return LaunchExchange(handle, vector, n, kExchangeSum, stream);
}

// In place: `moments` = [mean[C], M2[C], count] of the local rows (fp32,
// 2 * C + 1 floats) becomes the same three quantities of the rows of all
// replicas together (M2 = sum of squared deviations from the mean).
int LaunchExchangeMoments(void* handle, float* moments, int64_t channels,
                          cudaStream_t stream) {
  if (channels < 0) return MUSA_KERNELS_EINVAL;
  if (channels == 0) return MUSA_KERNELS_OK;
  return LaunchExchange(handle, moments, 2 * channels + 1, kExchangeMoments, stream);
}

// 0, or 1 + q if a wait for replica q ran out; clears the word.  Synchronises
// the device: call it between steps, not inside one.
int MusaExchangeStatus(void* handle) {
  auto* h = static_cast<ExchangeHost*>(handle);
  if (h == nullptr) return MUSA_KERNELS_EINVAL;
  int status = 0;
  if (cudaMemcpy(&status, h->dev.status, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) {
    return -100;
  }
  if (status != 0) cudaMemset(h->dev.status, 0, sizeof(int));
  return status;
}

void MusaExchangeDestroy(void* handle) {
  auto* h = static_cast<ExchangeHost*>(handle);
  if (h == nullptr) return;
  for (int q = 0; q < kMaxWorld; ++q) {
    if (h->opened[q] != nullptr) cudaIpcCloseMemHandle(h->opened[q]);
  }
  if (h->base != nullptr) cudaFree(h->base);
  delete h;
}

// ---- Peer-visible device memory: plain cudaMalloc blocks whose CUDA IPC
// handle other processes of the node can open (set-up time only).
void* MusaPeerAlloc(int64_t bytes) {
  if (bytes <= 0) return nullptr;
  void* p = nullptr;
  if (cudaMalloc(&p, static_cast<size_t>(bytes)) != cudaSuccess) {
    cudaGetLastError();
    return nullptr;
  }
  return p;
}

int MusaPeerFree(void* ptr) {
  return ptr == nullptr ? 0 : static_cast<int>(cudaFree(ptr));
}

int MusaPeerIpcHandle(void* ptr, void* out64) {
  if (ptr == nullptr || out64 == nullptr) return MUSA_KERNELS_EINVAL;
  cudaIpcMemHandle_t ipc;
  const cudaError_t err = cudaIpcGetMemHandle(&ipc, ptr);
  if (err != cudaSuccess) {
    cudaGetLastError();
    return static_cast<int>(err);
  }
  std::memcpy(out64, &ipc, 64);
  return 0;
}

void* MusaPeerOpen(const void* handle64) {
  if (handle64 == nullptr) return nullptr;
  cudaIpcMemHandle_t ipc;
  std::memcpy(&ipc, handle64, 64);
  void* mapped = nullptr;
  if (cudaIpcOpenMemHandle(&mapped, ipc, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
    cudaGetLastError();
    return nullptr;
  }
  return mapped;
}

// One asynchronous device-to-device copy (local or peer-mapped addresses) on
// `stream`: a copy engine moves it.
int MusaPeerCopyAsync(void* dst, const void* src, int64_t bytes, cudaStream_t stream) {
  if (bytes < 0 || (bytes > 0 && (dst == nullptr || src == nullptr))) return MUSA_KERNELS_EINVAL;
  if (bytes == 0) return MUSA_KERNELS_OK;
  const cudaError_t err = cudaMemcpyAsync(dst, src, static_cast<size_t>(bytes),
                                          cudaMemcpyDeviceToDevice, stream);
  if (err != cudaSuccess) cudaGetLastError();
  return static_cast<int>(err);
}

int MusaPeerClose(void* mapped) {
  return mapped == nullptr ? 0 : static_cast<int>(cudaIpcCloseMemHandle(mapped));
}

// Test hook: `world` replicas emulated on ONE GPU by one launch of `world`
// CTAs (one per replica, each with its own buffer in this GPU's memory), so the
// protocol can be checked where only one GPU is at hand.  `vectors`: device
// array of `world` pointers to n-float vectors; each becomes the total.
// `rounds` exchanges are run back to back to exercise the slot reuse.
// `missing_rank`: -1, or world - 1 to leave the last replica out (one round):
// the others' waits must then run out and report it (return 1000 + world).
int MusaExchangeSelfTest(int world, int64_t n, float* const* vectors, int rounds,
                         int missing_rank, int mode, cudaStream_t stream) {
  if (world < 1 || world > 8 || n < 1 || vectors == nullptr) return MUSA_KERNELS_EINVAL;
  ExchangeHost* hs[8] = {};
  int rc = 0;
  for (int r = 0; r < world; ++r) {
    hs[r] = static_cast<ExchangeHost*>(MusaExchangeCreate(r, world, n));
    if (hs[r] == nullptr) rc = MUSA_KERNELS_EINVAL;
  }
  ExchangeDev* table = nullptr;
  if (rc == 0 && cudaMalloc(&table, sizeof(ExchangeDev) * world) != cudaSuccess) rc = -100;
  if (rc == 0) {
    for (int r = 0; r < world; ++r) {
      for (int q = 0; q < world; ++q) {
        hs[r]->dev.cells[q] = hs[q]->dev.cells[q];
      }
      cudaMemcpy(table + r, &hs[r]->dev, sizeof(ExchangeDev), cudaMemcpyHostToDevice);
    }
    // With a "missing" replica, only the others run: their waits must run out
    // and report it instead of hanging.
    const int ctas = missing_rank >= 0 ? world - 1 : world;
    for (int round = 0; round < rounds && rc == 0; ++round) {
      float* none = nullptr;
      int n32 = static_cast<int>(n);
      void* args[] = {&table, const_cast<float* const**>(&vectors), &none, &n32, &mode};
      CountKernelLaunch();
      rc = static_cast<int>(cudaLaunchCooperativeKernel(
          reinterpret_cast<void*>(ExchangeSumsKernel), dim3(ctas), dim3(kExchangeThreads),
          args, 0, stream));
    }
    if (rc == 0) rc = static_cast<int>(cudaStreamSynchronize(stream));
    if (rc == 0) {
      for (int r = 0; r < (missing_rank >= 0 ? world - 1 : world); ++r) {
        const int st = MusaExchangeStatus(hs[r]);
        if (st != 0) rc = 1000 + st;  // 1000 + 1 + q: replica q never arrived
      }
    }
  }
  if (table != nullptr) cudaFree(table);
  for (int r = 0; r < world; ++r) MusaExchangeDestroy(hs[r]);
  return rc;
}

}  // extern "C"
