// DeviceDriver over the CUDA runtime.
#include <cuda_runtime.h>

#include <atomic>
#include <cstdlib>
#include <cstring>

#include "device_driver.h"

namespace musa_rt {
namespace {

__global__ void Fill32Kernel(uint32_t* dst, uint32_t pattern, size_t count) {
  const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
       i < count; i += stride) {
    dst[i] = pattern;
  }
}

cudaMemcpyKind ToCuda(CopyKind k) {
  switch (k) {
    case CopyKind::kHostToDevice: return cudaMemcpyHostToDevice;
    case CopyKind::kDeviceToHost: return cudaMemcpyDeviceToHost;
    default: return cudaMemcpyDeviceToDevice;
  }
}

// Clears the sticky "last error" after a failed query-style call.
int Code(cudaError_t e) {
  if (e != cudaSuccess) cudaGetLastError();
  return static_cast<int>(e);
}

class CudaDriverImpl : public DeviceDriver {
 public:
  const char* Name() const override { return "cuda"; }
  int DeviceCount(int* count) override { return Code(cudaGetDeviceCount(count)); }
  int SetDevice(int ordinal) override { return Code(cudaSetDevice(ordinal)); }
  int Malloc(void** ptr, size_t bytes) override { return Code(cudaMalloc(ptr, bytes)); }
  int Free(void* ptr) override { return Code(cudaFree(ptr)); }
  int HostAlloc(void** ptr, size_t bytes) override {
    return Code(cudaHostAlloc(ptr, bytes, cudaHostAllocDefault));
  }
  int HostFree(void* ptr) override { return Code(cudaFreeHost(ptr)); }
  int MemGetInfo(size_t* f, size_t* t) override { return Code(cudaMemGetInfo(f, t)); }
  int StreamCreate(StreamHandle* s) override {
    return Code(cudaStreamCreateWithFlags(reinterpret_cast<cudaStream_t*>(s),
                                          cudaStreamNonBlocking));
  }
  int StreamDestroy(StreamHandle s) override {
    return Code(cudaStreamDestroy(static_cast<cudaStream_t>(s)));
  }
  int StreamSynchronize(StreamHandle s) override {
    return Code(cudaStreamSynchronize(static_cast<cudaStream_t>(s)));
  }
  int StreamQuery(StreamHandle s) override {
    return Code(cudaStreamQuery(static_cast<cudaStream_t>(s)));
  }
  int EventCreate(EventHandle* e, bool with_timing) override {
    return Code(cudaEventCreateWithFlags(
        reinterpret_cast<cudaEvent_t*>(e),
        with_timing ? cudaEventDefault : cudaEventDisableTiming));
  }
  int EventDestroy(EventHandle e) override {
    return Code(cudaEventDestroy(static_cast<cudaEvent_t>(e)));
  }
  int EventRecord(EventHandle e, StreamHandle s) override {
    return Code(cudaEventRecord(static_cast<cudaEvent_t>(e), static_cast<cudaStream_t>(s)));
  }
  int EventQuery(EventHandle e) override {
    return Code(cudaEventQuery(static_cast<cudaEvent_t>(e)));
  }
  int EventSynchronize(EventHandle e) override {
    return Code(cudaEventSynchronize(static_cast<cudaEvent_t>(e)));
  }
  int EventElapsedMs(EventHandle a, EventHandle b, float* ms) override {
    return Code(cudaEventElapsedTime(ms, static_cast<cudaEvent_t>(a),
                                     static_cast<cudaEvent_t>(b)));
  }
  int StreamWaitEvent(StreamHandle s, EventHandle e) override {
    return Code(cudaStreamWaitEvent(static_cast<cudaStream_t>(s),
                                    static_cast<cudaEvent_t>(e), 0));
  }
  int MemcpyAsync(void* dst, const void* src, size_t n, CopyKind k,
                  StreamHandle s) override {
    return Code(cudaMemcpyAsync(dst, src, n, ToCuda(k), static_cast<cudaStream_t>(s)));
  }
  int Memcpy(void* dst, const void* src, size_t n, CopyKind k) override {
    return Code(cudaMemcpy(dst, src, n, ToCuda(k)));
  }
  int MemsetAsync(void* dst, int byte, size_t n, StreamHandle s) override {
    return Code(cudaMemsetAsync(dst, byte, n, static_cast<cudaStream_t>(s)));
  }
  int Memset32Async(void* dst, uint32_t pattern, size_t count, StreamHandle s) override {
    if (count == 0) return 0;
    size_t blocks = (count + 255) / 256;
    if (blocks > 148 * 8) blocks = 148 * 8;
    Fill32Kernel<<<static_cast<unsigned>(blocks), 256, 0, static_cast<cudaStream_t>(s)>>>(
        static_cast<uint32_t*>(dst), pattern, count);
    return Code(cudaGetLastError());
  }
  int LaunchHostFunc(StreamHandle s, void (*fn)(void*), void* arg) override {
    return Code(cudaLaunchHostFunc(static_cast<cudaStream_t>(s), fn, arg));
  }
  int DeviceSynchronize() override { return Code(cudaDeviceSynchronize()); }
  PointerKind Classify(const void* ptr) override {
    cudaPointerAttributes attr;
    if (cudaPointerGetAttributes(&attr, ptr) != cudaSuccess) {
      cudaGetLastError();
      return PointerKind::kPageableHost;
    }
    if (attr.type == cudaMemoryTypeDevice || attr.type == cudaMemoryTypeManaged) {
      return PointerKind::kDevice;
    }
    return attr.type == cudaMemoryTypeHost ? PointerKind::kPinnedHost
                                           : PointerKind::kPageableHost;
  }
  std::string ErrorString(int code) override {
    return cudaGetErrorString(static_cast<cudaError_t>(code));
  }
};

std::atomic<int> g_use_fake{-1};

}  // namespace

DeviceDriver* CudaDriver() {
  static CudaDriverImpl* impl = new CudaDriverImpl();
  return impl;
}

void SelectDriver(bool fake) { g_use_fake.store(fake ? 1 : 0); }

DeviceDriver* ActiveDriver() {
  int v = g_use_fake.load();
  if (v < 0) {
    const char* env = std::getenv("MUSA_RT_FAKE_DRIVER");
    v = (env != nullptr && std::strcmp(env, "1") == 0) ? 1 : 0;
    g_use_fake.store(v);
  }
  return v == 1 ? FakeDriver() : CudaDriver();
}

}  // namespace musa_rt
