// Cross-replica sum of small per-channel vectors, done by the GPUs themselves
// over NVLink peer memory: the exchange step of cross-replica BatchNorm
// (2*C + 1 floats per layer and pass) without a collective-library launch.
//
// Every replica owns one buffer in its OWN memory:
//     cell[2 slots][world][slot_floats]    8-byte cells {value bits, epoch}
// written by the peers (and by itself).  A cell is stored with one aligned
// 8-byte store, so a reader sees either the old cell or the new one, never a
// mix: the epoch inside the cell says whether the value is the one it waits
// for.  No separate flag and no memory fence are needed (the latency of one
// exchange is one NVLink store plus a poll).
// One exchange = one single-CTA kernel per replica:
//   1. epoch = local counter + 1 (a device-side counter, so a captured CUDA
//      graph replays correctly); slot = epoch & 1;
//   2. push: store {v[i], epoch} into cell[slot][rank][i] of EVERY replica
//      (plain stores to peer-mapped addresses);
//   3. gather, in its own memory: for each i, read cell[slot][q][i] for every
//      q and poll the ones whose epoch is still old.  The poll is bounded:
//      after kSpinLimit tries the kernel records which replica was missing in
//      a status word and goes on, so a lost peer never hangs a GPU;
//   4. total[i] = sum over q = 0..world-1, in rank order, so every replica
//      gets bit-identical totals; written over the input vector.
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
#include "../../include/musa_plugin_kernels.h"

namespace musa_b200 {
namespace {

constexpr int kMaxWorld = 16;
constexpr int kExchangeThreads = 512;
// Polls of one cell before a wait gives up (each poll is a volatile load plus
// a short sleep: of the order of a second in total).
constexpr long long kSpinLimit = 4LL << 20;

struct ExchangeDev {
  int rank;
  int world;
  long long slot_floats;
  uint2* cells[kMaxWorld];  // cell buffer of every replica (peer-mapped)
  unsigned* epoch;          // local
  int* status;              // local: 0 ok, 1 + q when replica q never arrived
};

struct ExchangeHost {
  ExchangeDev dev;
  ExchangeDev* dev_copy;  // device copy of `dev`
  void* base;             // the local allocation
  size_t bytes;
  void* opened[kMaxWorld];  // IPC mappings to close
  int device;
};

size_t Align256(size_t n) { return (n + 255) / 256 * 256; }

__device__ __forceinline__ uint2 LoadCell(const uint2* p) {
  uint2 v;
  asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];"
               : "=r"(v.x), "=r"(v.y)
               : "l"(p));
  return v;
}

__device__ __forceinline__ void StoreCell(uint2* p, uint2 v) {
  asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(p), "r"(v.x), "r"(v.y)
               : "memory");
}

template <int kWorld>  // 0: run-time world size
__device__ __forceinline__ void ExchangeBody(const ExchangeDev& c, float* vec, int n,
                                             unsigned epoch) {
  const int world = kWorld > 0 ? kWorld : c.world;
  const int slot = static_cast<int>(epoch & 1u);
  const long long slot_base = static_cast<long long>(slot) * world * c.slot_floats;
  const long long mine = slot_base + static_cast<long long>(c.rank) * c.slot_floats;

  // 2. push the local vector into every replica's memory.
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const uint2 cell = make_uint2(__float_as_uint(vec[i]), epoch);
#pragma unroll
    for (int p = 0; p < (kWorld > 0 ? kWorld : kMaxWorld); ++p) {
      if (p < world) StoreCell(c.cells[p] + mine + i, cell);
    }
  }

  // 3. + 4. gather from local memory and sum in rank order.
  const uint2* local = c.cells[c.rank] + slot_base;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    uint2 got[kWorld > 0 ? kWorld : kMaxWorld];
#pragma unroll
    for (int q = 0; q < (kWorld > 0 ? kWorld : kMaxWorld); ++q) {
      if (q < world) got[q] = LoadCell(local + static_cast<long long>(q) * c.slot_floats + i);
    }
    float total = 0.0f;
#pragma unroll
    for (int q = 0; q < (kWorld > 0 ? kWorld : kMaxWorld); ++q) {
      if (q < world) {
        long long polls = 0;
        while (got[q].y != epoch) {
          if (++polls > kSpinLimit) {
            atomicCAS(c.status, 0, 1 + q);
            break;
          }
          __nanosleep(40);
          got[q] = LoadCell(local + static_cast<long long>(q) * c.slot_floats + i);
        }
        total += __uint_as_float(got[q].x);
      }
    }
    vec[i] = total;
  }
}

__global__ void __launch_bounds__(kExchangeThreads)
    ExchangeSumsKernel(const ExchangeDev* ctxs, float* const* vectors,
                       float* single_vector, int n) {
  GridDepWait();
  GridDepLaunch();
  const ExchangeDev& c = ctxs[blockIdx.x];
  float* vec = vectors != nullptr ? vectors[blockIdx.x] : single_vector;
  const unsigned epoch = *c.epoch + 1u;  // nobody writes it before the barrier below
  switch (c.world) {
    case 1: ExchangeBody<1>(c, vec, n, epoch); break;
    case 2: ExchangeBody<2>(c, vec, n, epoch); break;
    case 4: ExchangeBody<4>(c, vec, n, epoch); break;
    case 8: ExchangeBody<8>(c, vec, n, epoch); break;
    default: ExchangeBody<0>(c, vec, n, epoch); break;
  }
  __syncthreads();
  if (threadIdx.x == 0) *c.epoch = epoch;
}

}  // namespace
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
  const size_t cell_bytes = Align256(sizeof(uint2) * 2 * world * slot_floats);
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
  h->dev.cells[rank] = reinterpret_cast<uint2*>(p);
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
    h->dev.cells[q] = static_cast<uint2*>(mapped);
  }
  return static_cast<int>(
      cudaMemcpy(h->dev_copy, &h->dev, sizeof(ExchangeDev), cudaMemcpyHostToDevice));
}

// In place: `vector` (n floats, local device memory) becomes the sum over all
// replicas.  One single-CTA kernel on `stream`; no host synchronisation.
int LaunchExchangeSums(void* handle, float* vector, int64_t n, cudaStream_t stream) {
  auto* h = static_cast<ExchangeHost*>(handle);
  if (h == nullptr || vector == nullptr || n < 0) return MUSA_KERNELS_EINVAL;
  if (n > h->dev.slot_floats) return MUSA_KERNELS_ETOOLARGE;
  if (n == 0) return MUSA_KERNELS_OK;
  LaunchChained(true, ExchangeSumsKernel, dim3(1), dim3(kExchangeThreads), 0, stream,
                static_cast<const ExchangeDev*>(h->dev_copy),
                static_cast<float* const*>(nullptr), vector, static_cast<int>(n));
  return static_cast<int>(cudaGetLastError());
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
                         int missing_rank, cudaStream_t stream) {
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
      void* args[] = {&table, const_cast<float* const**>(&vectors), &none, &n32};
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
