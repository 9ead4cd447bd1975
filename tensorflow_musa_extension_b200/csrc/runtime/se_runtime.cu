// The StreamExecutor-callback layer of the plugin on the CUDA runtime (see
// include/musa_plugin_runtime.h for the mapping to the reference's
// plugin_se_* functions).  Every entry point selects the device first and
// reports failures as a tensorflow::error code plus a thread-local message,
// the way the reference routes every runtime error into TF_Status
// (musa_ext/mu/musa_runtime_adapter.cc:10-32).
#include <cuda_runtime.h>

#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

#include "../../../include/musa_plugin_runtime.h"
#include "device_driver.h"
#include "runtime_registry.h"

using namespace musa_rt;

namespace {

constexpr int kOk = 0, kInvalidArgument = 3, kFailedPrecondition = 9,
              kUnimplemented = 12, kInternal = 13;

thread_local std::string g_last_error;

int Fail(int code, const std::string& msg) {
  g_last_error = msg;
  return code;
}

int Ok() {
  g_last_error.clear();
  return kOk;
}

// "<context>: <driver error string>" -> INTERNAL.
int FromDriver(int rc, const char* context) {
  if (rc == 0) return Ok();
  return Fail(kInternal, std::string(context) + ": " + ActiveDriver()->ErrorString(rc));
}

bool EnvIsOne(const char* name) {
  const char* p = std::getenv(name);
  return p != nullptr && std::strcmp(p, "1") == 0;
}

int SelectDevice(int ordinal) {
  if (ordinal < 0) return Fail(kInvalidArgument, "negative device ordinal");
  return FromDriver(ActiveDriver()->SetDevice(ordinal), "cudaSetDevice");
}

StreamHandle Raw(MusaRtStream s) {
  return (s != nullptr && s->magic == MUSA_RT_STREAM_MAGIC) ? s->stream : nullptr;
}

bool ValidStream(MusaRtStream s) { return s != nullptr && s->magic == MUSA_RT_STREAM_MAGIC; }

int DeviceCountImpl(int* count, bool strict) {
  if (count == nullptr) return Fail(kInvalidArgument, "null count");
  int n = 0;
  const int rc = ActiveDriver()->DeviceCount(&n);
  if (rc != 0) {
    *count = 0;
    if (strict) {
      return Fail(kFailedPrecondition,
                  "device enumeration failed: " + ActiveDriver()->ErrorString(rc));
    }
    return Ok();  // CPU-only machine: no devices, not an error
  }
  *count = n;
  return Ok();
}

// Host -> device with the pinned bounce for pageable sources (synchronous form
// only; the asynchronous form cannot know when a pageable source may change).
int HtoD(int ordinal, StreamHandle stream, void* dst, const void* src, uint64_t size,
         bool sync) {
  DeviceDriver* d = ActiveDriver();
  if (size == 0) return Ok();
  if (dst == nullptr) return Fail(kInvalidArgument, "null device pointer in memcpy H2D");
  if (src == nullptr) return Fail(kInvalidArgument, "null host pointer for src in memcpy H2D");
  const PointerKind kind = d->Classify(src);
  if (kind == PointerKind::kDevice) {
    return FromDriver(sync ? d->Memcpy(dst, src, size, CopyKind::kDeviceToDevice)
                           : d->MemcpyAsync(dst, src, size, CopyKind::kDeviceToDevice, stream),
                      "cudaMemcpy H2D(D2D)");
  }
  if (EnvIsOne("MUSA_SE_SYNC_H2D")) {
    return FromDriver(d->Memcpy(dst, src, size, CopyKind::kHostToDevice), "cudaMemcpy H2D");
  }
  if (kind == PointerKind::kPinnedHost) {
    return FromDriver(sync ? d->Memcpy(dst, src, size, CopyKind::kHostToDevice)
                           : d->MemcpyAsync(dst, src, size, CopyKind::kHostToDevice, stream),
                      sync ? "cudaMemcpy H2D" : "cudaMemcpyAsync H2D");
  }
  if (!sync && !EnvIsOne("MUSA_SE_DISABLE_PAGEABLE_H2D_BOUNCE") &&
      !EnvIsOne("MUSA_SE_DISABLE_ASYNC_H2D_BOUNCE")) {
    // Pageable source on an asynchronous copy: stage it through pinned chunks.
    // The host copy of chunk k+1 runs while the DMA of chunk k is in flight,
    // every chunk goes back to the pool once the stream has passed it, and the
    // source is fully read by the time this returns, so the caller may reuse
    // it at once.  (The reference falls back to a blocking cudaMemcpy here.)
    PinnedMemoryPool* chunk_pool = RegistryPinnedPool(ordinal);
    if (chunk_pool != nullptr) {
      constexpr uint64_t kChunk = 8ull << 20;
      uint64_t done = 0;
      while (done < size) {
        const uint64_t len = size - done < kChunk ? size - done : kChunk;
        void* staging = chunk_pool->Allocate(len);
        if (staging == nullptr) break;
        std::memcpy(staging, static_cast<const char*>(src) + done, len);
        const int rc = d->MemcpyAsync(static_cast<char*>(dst) + done, staging, len,
                                      CopyKind::kHostToDevice, stream);
        if (rc != 0) {
          chunk_pool->FreeCompleted(staging, len);
          return Fail(kInternal, "cudaMemcpyAsync H2D via pinned bounce buffer failed");
        }
        chunk_pool->FreeAsync(staging, len, stream);
        done += len;
      }
      if (done == size) return Ok();
      // Out of pinned memory part-way: the rest goes the blocking way, after
      // the chunks already queued on the stream.
      int rc = d->StreamSynchronize(stream);
      if (rc == 0) {
        rc = d->Memcpy(static_cast<char*>(dst) + done,
                       static_cast<const char*>(src) + done, size - done,
                       CopyKind::kHostToDevice);
      }
      return FromDriver(rc, "cudaMemcpy H2D");
    }
  }
  const bool bounce = sync && !EnvIsOne("MUSA_SE_DISABLE_PAGEABLE_H2D_BOUNCE") &&
                      !EnvIsOne("MUSA_SE_DISABLE_SYNC_H2D_BOUNCE");
  PinnedMemoryPool* pool = bounce ? RegistryPinnedPool(ordinal) : nullptr;
  void* staging = pool != nullptr ? pool->Allocate(size) : nullptr;
  if (staging == nullptr) {
    // Pageable source: a synchronous copy is the only safe form.
    return FromDriver(d->Memcpy(dst, src, size, CopyKind::kHostToDevice), "cudaMemcpy H2D");
  }
  std::memcpy(staging, src, size);
  int rc = d->MemcpyAsync(dst, staging, size, CopyKind::kHostToDevice, nullptr);
  if (rc != 0) {
    pool->FreeCompleted(staging, size);
    return Fail(kInternal, "cudaMemcpyAsync H2D via pinned bounce buffer failed");
  }
  rc = d->StreamSynchronize(nullptr);
  if (rc == 0) {
    pool->FreeCompleted(staging, size);
  } else {
    pool->FreeAsync(staging, size, nullptr);
  }
  return FromDriver(rc, "cudaStreamSynchronize H2D");
}

struct HostFn {
  void (*fn)(void*);
  void* arg;
};

}  // namespace

extern "C" {

const char* MusaRtLastError(void) { return g_last_error.c_str(); }
const char* MusaRtPlatformName(void) { return "MUSA_PLUGGABLE"; }
const char* MusaRtDeviceType(void) { return "MUSA"; }

int MusaRtInitPluginCheck(size_t params_struct_size, size_t min_struct_size) {
  if (EnvIsOne("TENSORFLOW_MUSA_USE_LEGACY_DEVICE")) {
    return Fail(kUnimplemented,
                "PluggableDevice path disabled by TENSORFLOW_MUSA_USE_LEGACY_DEVICE=1");
  }
  if (params_struct_size != 0 && params_struct_size < min_struct_size) {
    return Fail(kInvalidArgument, "SE_PlatformRegistrationParams is too small");
  }
  return Ok();
}

int MusaRtGetDeviceCount(int* count) {
  return DeviceCountImpl(count, EnvIsOne("MUSA_STRICT_DEVICE_ENUM"));
}

int MusaRtCreateDevice(int ordinal) {
  if (ordinal < 0) return Fail(kInvalidArgument, "negative device ordinal");
  RegistryOnDeviceCreated(ordinal);
  return Ok();
}

int MusaRtDestroyDevice(int ordinal) {
  if (ordinal < 0) return Fail(kInvalidArgument, "negative device ordinal");
  RegistryOnDeviceDestroyed(ordinal);
  return Ok();
}

int MusaRtAllocate(int ordinal, uint64_t size, void** ptr) {
  if (ptr == nullptr) return Fail(kInvalidArgument, "null result pointer");
  *ptr = nullptr;
  if (int rc = SelectDevice(ordinal)) return rc;
  if (size == 0) return Ok();
  void* p = nullptr;
  if (ActiveDriver()->Malloc(&p, size) != 0) p = nullptr;  // NULL signals out-of-memory
  *ptr = p;
  return Ok();
}

int MusaRtDeallocate(int ordinal, void* ptr) {
  if (ptr == nullptr) return Ok();
  if (int rc = SelectDevice(ordinal)) return rc;
  return FromDriver(ActiveDriver()->Free(ptr), "cudaFree");
}

int MusaRtHostAllocate(int ordinal, uint64_t size, void** ptr) {
  if (ptr == nullptr) return Fail(kInvalidArgument, "null result pointer");
  *ptr = nullptr;
  if (int rc = SelectDevice(ordinal)) return rc;
  if (size == 0) return Ok();
  void* p = nullptr;
  if (ActiveDriver()->HostAlloc(&p, size) != 0) p = nullptr;
  *ptr = p;
  return Ok();
}

int MusaRtHostDeallocate(int ordinal, void* ptr) {
  if (ptr == nullptr) return Ok();
  if (int rc = SelectDevice(ordinal)) return rc;
  return FromDriver(ActiveDriver()->HostFree(ptr), "cudaFreeHost");
}

int MusaRtDeviceMemoryUsage(int ordinal, int64_t* free_bytes, int64_t* total_bytes) {
  if (free_bytes == nullptr || total_bytes == nullptr) {
    return Fail(kInvalidArgument, "null result pointer");
  }
  if (int rc = SelectDevice(ordinal)) return rc;
  size_t f = 0, t = 0;
  if (int rc = FromDriver(ActiveDriver()->MemGetInfo(&f, &t), "cudaMemGetInfo")) return rc;
  *free_bytes = static_cast<int64_t>(f);
  *total_bytes = static_cast<int64_t>(t);
  return Ok();
}

int MusaRtCreateStream(int ordinal, MusaRtStream* stream) {
  if (stream == nullptr) return Fail(kInvalidArgument, "null result pointer");
  *stream = nullptr;
  if (int rc = SelectDevice(ordinal)) return rc;
  StreamHandle raw = nullptr;
  if (int rc = FromDriver(ActiveDriver()->StreamCreate(&raw), "cudaStreamCreate")) return rc;
  auto* s = new MusaRtStream_st();
  s->magic = MUSA_RT_STREAM_MAGIC;
  s->stream = raw;
  *stream = s;
  return Ok();
}

int MusaRtDestroyStream(int ordinal, MusaRtStream stream) {
  if (stream == nullptr) return Ok();
  if (!ValidStream(stream)) return Fail(kInvalidArgument, "not a plugin stream");
  int rc = SelectDevice(ordinal);
  RegistryOnStreamDestroyed(ordinal, stream->stream);
  if (rc == kOk && stream->stream != nullptr) {
    rc = FromDriver(ActiveDriver()->StreamDestroy(stream->stream), "cudaStreamDestroy");
  }
  stream->magic = 0;
  delete stream;
  return rc;
}

int MusaRtGetStreamStatus(int ordinal, MusaRtStream stream) {
  if (!ValidStream(stream)) return Fail(kInvalidArgument, "null stream in get_stream_status");
  if (int rc = SelectDevice(ordinal)) return rc;
  const int q = ActiveDriver()->StreamQuery(stream->stream);
  if (q == 0 || q == kNotReady) return Ok();
  return FromDriver(q, "cudaStreamQuery");
}

void* MusaRtRawStream(MusaRtStream stream) { return Raw(stream); }

int MusaRtCreateStreamDependency(int ordinal, MusaRtStream dependent, MusaRtStream other) {
  if (!ValidStream(dependent) || !ValidStream(other)) {
    return Fail(kInvalidArgument, "null stream in create_stream_dependency");
  }
  if (int rc = SelectDevice(ordinal)) return rc;
  DeviceDriver* d = ActiveDriver();
  EventHandle ev = nullptr;
  if (int rc = FromDriver(d->EventCreate(&ev, false), "cudaEventCreate")) return rc;
  int rc = d->EventRecord(ev, other->stream);
  if (rc != 0) {
    d->EventDestroy(ev);
    return FromDriver(rc, "cudaEventRecord");
  }
  rc = d->StreamWaitEvent(dependent->stream, ev);
  if (rc != 0) {
    d->EventDestroy(ev);
    return FromDriver(rc, "cudaStreamWaitEvent");
  }
  // The wait is only queued: the event must outlive it.
  EventMgr* mgr = EnvIsOne("MUSA_SE_SYNC_STREAM_DEPENDENCY") ? nullptr : RegistryEventMgr(ordinal);
  if (mgr == nullptr) {
    rc = d->StreamSynchronize(dependent->stream);
    const int drc = d->EventDestroy(ev);
    if (rc != 0) return FromDriver(rc, "cudaStreamSynchronize");
    return FromDriver(drc, "cudaEventDestroy");
  }
  mgr->ThenExecute(dependent->stream, [ev, ordinal] {
    ActiveDriver()->SetDevice(ordinal);
    ActiveDriver()->EventDestroy(ev);
  });
  return Ok();
}

int MusaRtCreateEvent(int ordinal, MusaRtEvent* event) {
  if (event == nullptr) return Fail(kInvalidArgument, "null result pointer");
  *event = nullptr;
  if (int rc = SelectDevice(ordinal)) return rc;
  EventHandle raw = nullptr;
  if (int rc = FromDriver(ActiveDriver()->EventCreate(&raw, false), "cudaEventCreate")) return rc;
  auto* e = new MusaRtEvent_st();
  e->event = raw;
  *event = e;
  return Ok();
}

int MusaRtDestroyEvent(int ordinal, MusaRtEvent event) {
  if (event == nullptr) return Ok();
  int rc = SelectDevice(ordinal);
  if (rc == kOk && event->event != nullptr) {
    rc = FromDriver(ActiveDriver()->EventDestroy(event->event), "cudaEventDestroy");
  }
  delete event;
  return rc;
}

int MusaRtRecordEvent(int ordinal, MusaRtStream stream, MusaRtEvent event) {
  if (!ValidStream(stream) || event == nullptr) {
    return Fail(kInvalidArgument, "null stream or event in record_event");
  }
  if (int rc = SelectDevice(ordinal)) return rc;
  return FromDriver(ActiveDriver()->EventRecord(event->event, stream->stream), "cudaEventRecord");
}

int MusaRtGetEventStatus(int ordinal, MusaRtEvent event) {
  if (event == nullptr || SelectDevice(ordinal) != kOk) return 2;
  const int q = ActiveDriver()->EventQuery(event->event);
  return q == 0 ? 0 : (q == kNotReady ? 1 : 2);
}

int MusaRtWaitForEvent(int ordinal, MusaRtStream stream, MusaRtEvent event) {
  if (!ValidStream(stream) || event == nullptr) {
    return Fail(kInvalidArgument, "null stream or event in wait_for_event");
  }
  if (int rc = SelectDevice(ordinal)) return rc;
  return FromDriver(ActiveDriver()->StreamWaitEvent(stream->stream, event->event),
                    "cudaStreamWaitEvent");
}

int MusaRtBlockHostForEvent(int ordinal, MusaRtEvent event) {
  if (event == nullptr) return Fail(kInvalidArgument, "null event in block_host_for_event");
  if (int rc = SelectDevice(ordinal)) return rc;
  return FromDriver(ActiveDriver()->EventSynchronize(event->event), "cudaEventSynchronize");
}

int MusaRtCreateTimer(int ordinal, MusaRtTimer* timer) {
  if (timer == nullptr) return Fail(kInvalidArgument, "null result pointer");
  *timer = nullptr;
  if (int rc = SelectDevice(ordinal)) return rc;
  DeviceDriver* d = ActiveDriver();
  EventHandle a = nullptr, b = nullptr;
  if (int rc = FromDriver(d->EventCreate(&a, true), "cudaEventCreate")) return rc;
  if (int rc = d->EventCreate(&b, true)) {
    d->EventDestroy(a);
    return FromDriver(rc, "cudaEventCreate");
  }
  auto* t = new MusaRtTimer_st();
  t->start = a;
  t->stop = b;
  *timer = t;
  return Ok();
}

int MusaRtDestroyTimer(int ordinal, MusaRtTimer timer) {
  if (timer == nullptr) return Ok();
  const int rc = SelectDevice(ordinal);
  if (rc == kOk) {
    ActiveDriver()->EventDestroy(timer->start);
    ActiveDriver()->EventDestroy(timer->stop);
  }
  delete timer;
  return rc;
}

int MusaRtStartTimer(int ordinal, MusaRtStream stream, MusaRtTimer timer) {
  if (!ValidStream(stream) || timer == nullptr) {
    return Fail(kInvalidArgument, "null stream or timer in start_timer");
  }
  if (int rc = SelectDevice(ordinal)) return rc;
  return FromDriver(ActiveDriver()->EventRecord(timer->start, stream->stream), "cudaEventRecord");
}

int MusaRtStopTimer(int ordinal, MusaRtStream stream, MusaRtTimer timer) {
  if (!ValidStream(stream) || timer == nullptr) {
    return Fail(kInvalidArgument, "null stream or timer in stop_timer");
  }
  if (int rc = SelectDevice(ordinal)) return rc;
  return FromDriver(ActiveDriver()->EventRecord(timer->stop, stream->stream), "cudaEventRecord");
}

uint64_t MusaRtTimerNanoseconds(MusaRtTimer timer) {
  if (timer == nullptr) return 0;
  DeviceDriver* d = ActiveDriver();
  if (d->EventSynchronize(timer->stop) != 0) return 0;
  float ms = 0.0f;
  if (d->EventElapsedMs(timer->start, timer->stop, &ms) != 0 || ms < 0.0f) return 0;
  return static_cast<uint64_t>(static_cast<double>(ms) * 1e6);
}

int MusaRtMemcpyDtoH(int ordinal, MusaRtStream stream, void* host_dst, const void* device_src,
                     uint64_t size) {
  if (!ValidStream(stream)) return Fail(kInvalidArgument, "null stream in memcpy_dtoh");
  if (size == 0) return Ok();
  if (host_dst == nullptr) return Fail(kInvalidArgument, "null host pointer for dst in memcpy D2H");
  if (device_src == nullptr) return Fail(kInvalidArgument, "null device pointer in memcpy D2H");
  if (int rc = SelectDevice(ordinal)) return rc;
  return FromDriver(ActiveDriver()->MemcpyAsync(host_dst, device_src, size,
                                                CopyKind::kDeviceToHost, stream->stream),
                    "cudaMemcpyAsync D2H");
}

int MusaRtMemcpyHtoD(int ordinal, MusaRtStream stream, void* device_dst, const void* host_src,
                     uint64_t size) {
  if (!ValidStream(stream)) return Fail(kInvalidArgument, "null stream in memcpy_htod");
  if (int rc = SelectDevice(ordinal)) return rc;
  return HtoD(ordinal, stream->stream, device_dst, host_src, size, /*sync=*/false);
}

int MusaRtMemcpyDtoD(int ordinal, MusaRtStream stream, void* device_dst, const void* device_src,
                     uint64_t size) {
  if (!ValidStream(stream)) return Fail(kInvalidArgument, "null stream in memcpy_dtod");
  if (size == 0) return Ok();
  if (device_dst == nullptr || device_src == nullptr) {
    return Fail(kInvalidArgument, "null device pointer in memcpy D2D");
  }
  if (int rc = SelectDevice(ordinal)) return rc;
  return FromDriver(ActiveDriver()->MemcpyAsync(device_dst, device_src, size,
                                                CopyKind::kDeviceToDevice, stream->stream),
                    "cudaMemcpyAsync D2D");
}

int MusaRtSyncMemcpyDtoH(int ordinal, void* host_dst, const void* device_src, uint64_t size) {
  if (size == 0) return Ok();
  if (host_dst == nullptr) return Fail(kInvalidArgument, "null host pointer for dst in memcpy D2H");
  if (device_src == nullptr) return Fail(kInvalidArgument, "null device pointer in memcpy D2H");
  if (int rc = SelectDevice(ordinal)) return rc;
  return FromDriver(ActiveDriver()->Memcpy(host_dst, device_src, size, CopyKind::kDeviceToHost),
                    "cudaMemcpy D2H");
}

int MusaRtSyncMemcpyHtoD(int ordinal, void* device_dst, const void* host_src, uint64_t size) {
  if (int rc = SelectDevice(ordinal)) return rc;
  return HtoD(ordinal, nullptr, device_dst, host_src, size, /*sync=*/true);
}

int MusaRtSyncMemcpyDtoD(int ordinal, void* device_dst, const void* device_src, uint64_t size) {
  if (size == 0) return Ok();
  if (device_dst == nullptr || device_src == nullptr) {
    return Fail(kInvalidArgument, "null device pointer in memcpy D2D");
  }
  if (int rc = SelectDevice(ordinal)) return rc;
  return FromDriver(ActiveDriver()->Memcpy(device_dst, device_src, size, CopyKind::kDeviceToDevice),
                    "cudaMemcpy D2D");
}

int MusaRtMemZero(int ordinal, MusaRtStream stream, void* ptr, uint64_t size) {
  return MusaRtMemset(ordinal, stream, ptr, 0, size);
}

int MusaRtMemset(int ordinal, MusaRtStream stream, void* ptr, uint8_t value, uint64_t size) {
  if (!ValidStream(stream)) return Fail(kInvalidArgument, "null stream in memset");
  if (size == 0) return Ok();
  if (ptr == nullptr) return Fail(kInvalidArgument, "null device pointer in memset");
  if (int rc = SelectDevice(ordinal)) return rc;
  return FromDriver(ActiveDriver()->MemsetAsync(ptr, value, size, stream->stream),
                    "cudaMemsetAsync");
}

int MusaRtMemset32(int ordinal, MusaRtStream stream, void* ptr, uint32_t pattern, uint64_t size) {
  if (!ValidStream(stream)) return Fail(kInvalidArgument, "null stream in memset32");
  if (size == 0) return Ok();
  if (ptr == nullptr) return Fail(kInvalidArgument, "null device pointer in memset32");
  if (size % 4 != 0 || (reinterpret_cast<uintptr_t>(ptr) & 3u) != 0) {
    return Fail(kInvalidArgument, "memset32 needs a 4-byte aligned pointer and size");
  }
  if (int rc = SelectDevice(ordinal)) return rc;
  return FromDriver(ActiveDriver()->Memset32Async(ptr, pattern, size / 4, stream->stream),
                    "memset32");
}

int MusaRtHostCallback(int ordinal, MusaRtStream stream, void (*fn)(void*), void* arg) {
  if (!ValidStream(stream) || fn == nullptr) {
    return Fail(kInvalidArgument, "null stream or callback in host_callback");
  }
  if (int rc = SelectDevice(ordinal)) return rc;
  return FromDriver(ActiveDriver()->LaunchHostFunc(stream->stream, fn, arg), "cudaLaunchHostFunc");
}

int MusaRtBlockHostUntilDone(int ordinal, MusaRtStream stream) {
  if (!ValidStream(stream)) return Fail(kInvalidArgument, "null stream in block_host_until_done");
  if (int rc = SelectDevice(ordinal)) return rc;
  return FromDriver(ActiveDriver()->StreamSynchronize(stream->stream), "cudaStreamSynchronize");
}

int MusaRtSynchronizeAllActivity(int ordinal) {
  if (int rc = SelectDevice(ordinal)) return rc;
  return FromDriver(ActiveDriver()->DeviceSynchronize(), "cudaDeviceSynchronize");
}

// ------------------------------------------------------------ test hooks --

int MUSA_TestPluginGetDeviceCount(int* count) { return MusaRtGetDeviceCount(count); }

static int SmokeImpl(bool relaxed) {
  int n = 0;
  const int rc = DeviceCountImpl(&n, !relaxed);
  if (rc != kOk) return rc;
  if (n == 0) {
    if (relaxed) return Ok();  // smoke skipped: nothing to run on
    return Fail(kFailedPrecondition, "MUSA_TestSeRuntimeSmokeStrict: zero MUSA devices");
  }
  // Host -> device -> device -> host round trip through the callbacks.
  if (int r = MusaRtCreateDevice(0)) return r;
  int result = kOk;
  MusaRtStream s = nullptr;
  void *a = nullptr, *b = nullptr;
  std::vector<uint32_t> src(4096), back(4096, 0);
  for (size_t i = 0; i < src.size(); ++i) src[i] = static_cast<uint32_t>(i * 2654435761u);
  const uint64_t bytes = src.size() * sizeof(uint32_t);
  do {
    if ((result = MusaRtCreateStream(0, &s)) != kOk) break;
    if ((result = MusaRtAllocate(0, bytes, &a)) != kOk) break;
    if ((result = MusaRtAllocate(0, bytes, &b)) != kOk) break;
    if (a == nullptr || b == nullptr) {
      result = Fail(kInternal, "MUSA_TestSeRuntimeSmoke: allocation failed");
      break;
    }
    if ((result = MusaRtSyncMemcpyHtoD(0, a, src.data(), bytes)) != kOk) break;
    if ((result = MusaRtMemcpyDtoD(0, s, b, a, bytes)) != kOk) break;
    if ((result = MusaRtBlockHostUntilDone(0, s)) != kOk) break;
    if ((result = MusaRtSyncMemcpyDtoH(0, back.data(), b, bytes)) != kOk) break;
    if (std::memcmp(src.data(), back.data(), bytes) != 0) {
      result = Fail(kInternal, "MUSA_TestSeRuntimeSmoke: memcpy check failed");
    }
  } while (false);
  const std::string keep = g_last_error;
  MusaRtDeallocate(0, a);
  MusaRtDeallocate(0, b);
  MusaRtDestroyStream(0, s);
  MusaRtDestroyDevice(0);
  if (result != kOk) g_last_error = keep;
  return result;
}

int MUSA_TestSeRuntimeSmoke(void) { return SmokeImpl(true); }
int MUSA_TestSeRuntimeSmokeStrict(void) { return SmokeImpl(false); }

size_t MUSA_TestSeRegistryLiveOrdinalsForTest(void) { return RegistryLiveOrdinals().size(); }

int MUSA_TestRegistryDeviceLifecycle(void) {
  constexpr int kFakeOrdinal = 42;
  if (RegistryHasLiveDevice(kFakeOrdinal)) {
    return Fail(kInternal, "MUSA_TestRegistryDeviceLifecycle: ordinal 42 already live");
  }
  const size_t before = RegistryLiveOrdinals().size();
  RegistryOnDeviceCreated(kFakeOrdinal);
  RegistryOnDeviceCreated(kFakeOrdinal);  // second reference
  if (RegistryLiveOrdinals().size() != before + 1 || RegistryRefCount(kFakeOrdinal) != 2) {
    return Fail(kInternal, "MUSA_TestRegistryDeviceLifecycle: expected one live ordinal");
  }
  RegistryOnStreamDestroyed(kFakeOrdinal, reinterpret_cast<StreamHandle>(0x1234));
  RegistryOnDeviceDestroyed(kFakeOrdinal);
  if (!RegistryHasLiveDevice(kFakeOrdinal)) {
    return Fail(kInternal, "MUSA_TestRegistryDeviceLifecycle: released too early");
  }
  RegistryOnDeviceDestroyed(kFakeOrdinal);
  if (RegistryHasLiveDevice(kFakeOrdinal) || RegistryLiveOrdinals().size() != before) {
    return Fail(kInternal, "MUSA_TestRegistryDeviceLifecycle: expected empty registry");
  }
  if (RegistryEventMgr(kFakeOrdinal) != nullptr || RegistryPinnedPool(kFakeOrdinal) != nullptr) {
    return Fail(kInternal, "MUSA_TestRegistryDeviceLifecycle: helpers for a dead ordinal");
  }
  return Ok();
}

int MUSA_TestDeviceMetadata(int ordinal, char* name, size_t name_cap, int* sm_count,
                            int64_t* total_memory) {
  if (std::strcmp(ActiveDriver()->Name(), "cuda") != 0) {
    if (name != nullptr && name_cap > 0) {
      std::strncpy(name, "fake device", name_cap - 1);
      name[name_cap - 1] = '\0';
    }
    if (sm_count != nullptr) *sm_count = 1;
    if (total_memory != nullptr) *total_memory = int64_t(1) << 34;
    return Ok();
  }
  cudaDeviceProp prop;
  const cudaError_t err = cudaGetDeviceProperties(&prop, ordinal);
  if (err != cudaSuccess) {
    cudaGetLastError();
    return Fail(kInternal, std::string("cudaGetDeviceProperties: ") + cudaGetErrorString(err));
  }
  if (name != nullptr && name_cap > 0) {
    std::strncpy(name, prop.name, name_cap - 1);
    name[name_cap - 1] = '\0';
  }
  if (sm_count != nullptr) *sm_count = prop.multiProcessorCount;
  if (total_memory != nullptr) *total_memory = static_cast<int64_t>(prop.totalGlobalMem);
  return Ok();
}

// ------------------------------------------------- fake driver and helpers --

void MusaRtUseFakeDriver(int enable) { SelectDriver(enable != 0); }
const char* MusaRtDriverName(void) { return ActiveDriver()->Name(); }
void MusaRtFakeSetDeviceCount(int count) { FakeDriverSetDeviceCount(count); }
uint64_t MusaRtFakeBlockStream(MusaRtStream stream) {
  return ValidStream(stream) ? FakeDriverBlockStream(stream->stream) : 0;
}
void MusaRtFakeReleaseGate(uint64_t gate) { FakeDriverReleaseGate(gate); }
int64_t MusaRtFakeLiveAllocations(void) { return FakeDriverLiveAllocations(); }
int64_t MusaRtFakeLiveEvents(void) { return FakeDriverLiveEvents(); }

void* MusaRtPinnedAllocate(int ordinal, uint64_t size) {
  PinnedMemoryPool* pool = RegistryPinnedPool(ordinal);
  return pool != nullptr ? pool->Allocate(size) : nullptr;
}

int MusaRtPinnedFreeAsync(int ordinal, void* ptr, uint64_t size, MusaRtStream stream) {
  PinnedMemoryPool* pool = RegistryPinnedPool(ordinal);
  if (pool == nullptr) return Fail(kFailedPrecondition, "no live device for this ordinal");
  pool->FreeAsync(ptr, size, Raw(stream));
  return Ok();
}

int MusaRtPinnedStats(int ordinal, uint64_t out[7]) {
  PinnedMemoryPool* pool = RegistryPinnedPool(ordinal);
  if (pool == nullptr || out == nullptr) {
    return Fail(kFailedPrecondition, "no live device for this ordinal");
  }
  const PinnedPoolStats s = pool->stats();
  out[0] = s.host_allocs;
  out[1] = s.reuse_hits;
  out[2] = s.event_allocs;
  out[3] = s.event_reuse_hits;
  out[4] = s.free_blocks;
  out[5] = s.pending_blocks;
  out[6] = s.bytes_held;
  return Ok();
}

int MusaRtThenExecute(int ordinal, MusaRtStream stream, void (*fn)(void*), void* arg) {
  if (!ValidStream(stream) || fn == nullptr) {
    return Fail(kInvalidArgument, "null stream or callback in then_execute");
  }
  EventMgr* mgr = RegistryEventMgr(ordinal);
  if (mgr == nullptr) return Fail(kFailedPrecondition, "no live device for this ordinal");
  const HostFn call{fn, arg};
  mgr->ThenExecute(stream->stream, [call] { call.fn(call.arg); });
  return Ok();
}

uint64_t MusaRtEventMgrCallbacksRun(int ordinal) {
  EventMgr* mgr = RegistryEventMgr(ordinal);
  return mgr != nullptr ? mgr->callbacks_run() : 0;
}

}  // extern "C"
