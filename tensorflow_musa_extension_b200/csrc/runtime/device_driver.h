// The device-runtime calls the plugin's stream-executor layer is built on,
// behind one interface with two implementations:
//   * CudaDriver  - the CUDA runtime (streams, events, cudaMalloc, pinned host
//     memory, async copies): the re-target of the reference's musa* calls in
//     musa_ext/mu/musa_se_plugin.cc and musa_ext/mu/device/*;
//   * FakeDriver  - a host-only emulation (a worker thread per stream, events
//     that complete when their stream reaches them) so that the event manager,
//     the pinned pool, stream dependencies and the copy paths can be tested
//     with real concurrency on a machine without a GPU, the way the reference
//     tests its registry with a fake ordinal and a fake stream pointer
//     (musa_ext/mu/musa_se_plugin.cc:1008-1045).
// All calls return 0 on success or an error code (a cudaError_t value for the
// CUDA driver); nothing throws.
#pragma once

#include <cstddef>
#include <cstdint>
#include <string>

namespace musa_rt {

using StreamHandle = void*;  // cudaStream_t
using EventHandle = void*;   // cudaEvent_t

enum class CopyKind { kHostToDevice, kDeviceToHost, kDeviceToDevice };
enum class PointerKind { kPageableHost, kPinnedHost, kDevice };

constexpr int kNotReady = 600;  // value of cudaErrorNotReady

class DeviceDriver {
 public:
  virtual ~DeviceDriver() = default;
  virtual const char* Name() const = 0;
  virtual int DeviceCount(int* count) = 0;
  virtual int SetDevice(int ordinal) = 0;
  virtual int Malloc(void** ptr, size_t bytes) = 0;
  virtual int Free(void* ptr) = 0;
  virtual int HostAlloc(void** ptr, size_t bytes) = 0;
  virtual int HostFree(void* ptr) = 0;
  virtual int MemGetInfo(size_t* free_bytes, size_t* total_bytes) = 0;
  virtual int StreamCreate(StreamHandle* stream) = 0;
  virtual int StreamDestroy(StreamHandle stream) = 0;
  virtual int StreamSynchronize(StreamHandle stream) = 0;
  virtual int StreamQuery(StreamHandle stream) = 0;  // 0 | kNotReady | error
  virtual int EventCreate(EventHandle* event, bool with_timing) = 0;
  virtual int EventDestroy(EventHandle event) = 0;
  virtual int EventRecord(EventHandle event, StreamHandle stream) = 0;
  virtual int EventQuery(EventHandle event) = 0;  // 0 | kNotReady | error
  virtual int EventSynchronize(EventHandle event) = 0;
  virtual int EventElapsedMs(EventHandle start, EventHandle stop, float* ms) = 0;
  virtual int StreamWaitEvent(StreamHandle stream, EventHandle event) = 0;
  virtual int MemcpyAsync(void* dst, const void* src, size_t bytes, CopyKind kind,
                          StreamHandle stream) = 0;
  virtual int Memcpy(void* dst, const void* src, size_t bytes, CopyKind kind) = 0;
  virtual int MemsetAsync(void* dst, int byte, size_t bytes, StreamHandle stream) = 0;
  virtual int Memset32Async(void* dst, uint32_t pattern, size_t count,
                            StreamHandle stream) = 0;
  virtual int LaunchHostFunc(StreamHandle stream, void (*fn)(void*), void* arg) = 0;
  virtual int DeviceSynchronize() = 0;
  virtual PointerKind Classify(const void* ptr) = 0;
  virtual std::string ErrorString(int code) = 0;
};

DeviceDriver* CudaDriver();
DeviceDriver* FakeDriver();

// The driver the runtime uses: CUDA unless the process selected the fake one
// (MusaRtUseFakeDriver, or MUSA_RT_FAKE_DRIVER=1 in the environment).
DeviceDriver* ActiveDriver();
void SelectDriver(bool fake);

// Fake-driver controls for tests: number of devices it reports, and a gate that
// stalls a stream until released (returns a gate id; 0 on failure).
void FakeDriverSetDeviceCount(int count);
uint64_t FakeDriverBlockStream(StreamHandle stream);
void FakeDriverReleaseGate(uint64_t gate);
int64_t FakeDriverLiveAllocations();  // device + pinned blocks not yet freed
int64_t FakeDriverLiveEvents();

}  // namespace musa_rt
