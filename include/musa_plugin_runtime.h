/* C ABI of the device runtime inside libmusa_plugin_kernels.so: what the
 * plugin's StreamExecutor C-API callbacks do, re-targeted to CUDA streams,
 * events and allocators.
 *
 * In the reference these are the `plugin_se_*` functions that
 * plugin_create_stream_executor installs in the SP_StreamExecutor table
 * (musa_ext/mu/musa_se_plugin.cc:216-846, table :1166-1213).  TensorFlow's
 * stream_executor.h is not available to this build, so each callback is
 * exported here as a plain function with the SP_Device replaced by its ordinal
 * and TF_Status replaced by a returned code plus MusaRtLastError(); filling
 * the SP_StreamExecutor table is then one forwarding line per entry.
 *
 * Return codes are tensorflow::error codes: 0 OK, 3 INVALID_ARGUMENT,
 * 9 FAILED_PRECONDITION, 12 UNIMPLEMENTED, 13 INTERNAL (a runtime call
 * failed; the message carries "<what>: <driver error string>", as
 * musa_ext/mu/musa_runtime_adapter.cc:10-20 formats it).
 */
#ifndef MUSA_PLUGIN_RUNTIME_H_
#define MUSA_PLUGIN_RUNTIME_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Stream wrapper with the layout and tag of the reference's SP_Stream_st
 * (musa_ext/mu/musa_plugin_sp_stream.h:23-32): kernels recognise a plugin
 * stream by the 64-bit magic and read the raw stream next to it. */
#define MUSA_RT_STREAM_MAGIC UINT64_C(0x4D55534153455053)
typedef struct MusaRtStream_st {
  uint64_t magic;
  void* stream; /* cudaStream_t */
} * MusaRtStream;
typedef struct MusaRtEvent_st {
  void* event; /* cudaEvent_t */
} * MusaRtEvent;
typedef struct MusaRtTimer_st {
  void* start;
  void* stop;
} * MusaRtTimer;

/* Message of the last failed call on this thread ("" if none). */
const char* MusaRtLastError(void);

/* Platform identity reported to TensorFlow by SE_InitPlugin
 * (musa_ext/mu/musa_se_plugin.cc:59-61, 1276-1281). */
const char* MusaRtPlatformName(void); /* "MUSA_PLUGGABLE" */
const char* MusaRtDeviceType(void);   /* "MUSA" */

/* SE_InitPlugin's gate: 12 UNIMPLEMENTED when TENSORFLOW_MUSA_USE_LEGACY_DEVICE=1
 * asks for the legacy path, 3 when the registration struct is too small
 * (struct_size == 0 is accepted), else 0 (:1241-1258). */
int MusaRtInitPluginCheck(size_t params_struct_size, size_t min_struct_size);

/* plugin_get_device_count (:855-873).  Without a usable driver the relaxed
 * mode (default) reports 0 devices and OK; MUSA_STRICT_DEVICE_ENUM=1 makes it
 * 9 FAILED_PRECONDITION. */
int MusaRtGetDeviceCount(int* count);

/* plugin_create_device / plugin_destroy_device (:1047-1096): reference-counted
 * registration of the ordinal in the runtime registry. */
int MusaRtCreateDevice(int ordinal);
int MusaRtDestroyDevice(int ordinal);

/* allocate / deallocate / host_memory_allocate / host_memory_deallocate
 * (:216-291).  Allocation failure leaves *ptr NULL and returns 0, as the
 * reference signals it (opaque = nullptr, :232-238). */
int MusaRtAllocate(int ordinal, uint64_t size, void** ptr);
int MusaRtDeallocate(int ordinal, void* ptr);
int MusaRtHostAllocate(int ordinal, uint64_t size, void** ptr);
int MusaRtHostDeallocate(int ordinal, void* ptr);
int MusaRtDeviceMemoryUsage(int ordinal, int64_t* free_bytes, int64_t* total_bytes);

/* create_stream / destroy_stream / get_stream_status (:303-360, :434-446). */
int MusaRtCreateStream(int ordinal, MusaRtStream* stream);
int MusaRtDestroyStream(int ordinal, MusaRtStream stream);
int MusaRtGetStreamStatus(int ordinal, MusaRtStream stream);
/* The raw stream behind a wrapper, NULL unless the magic matches: what
 * tf_compat::GpuStreamFromTfStream does with a plugin CStream
 * (musa_ext/mu/tf_compat/pluggable_tf_compat.cc:36-58). */
void* MusaRtRawStream(MusaRtStream stream);

/* create_stream_dependency (:362-432): `dependent` waits for the work queued
 * on `other` so far.  The temporary event lives until `dependent` has passed
 * the wait (destroyed from the event manager's callback), or the call blocks
 * and destroys it when MUSA_SE_SYNC_STREAM_DEPENDENCY=1 or no event manager
 * exists for the ordinal. */
int MusaRtCreateStreamDependency(int ordinal, MusaRtStream dependent, MusaRtStream other);

/* create_event / destroy_event / record_event / get_event_status /
 * wait_for_event / block_host_for_event (:448-527, :752-800). */
int MusaRtCreateEvent(int ordinal, MusaRtEvent* event);
int MusaRtDestroyEvent(int ordinal, MusaRtEvent event);
int MusaRtRecordEvent(int ordinal, MusaRtStream stream, MusaRtEvent event);
/* 0 complete, 1 pending, 2 error (SE_EVENT_COMPLETE / PENDING / ERROR). */
int MusaRtGetEventStatus(int ordinal, MusaRtEvent event);
int MusaRtWaitForEvent(int ordinal, MusaRtStream stream, MusaRtEvent event);
int MusaRtBlockHostForEvent(int ordinal, MusaRtEvent event);

/* create_timer / destroy_timer / start_timer / stop_timer / timer_nanoseconds:
 * a timer is two events (:529-597, :837-844). */
int MusaRtCreateTimer(int ordinal, MusaRtTimer* timer);
int MusaRtDestroyTimer(int ordinal, MusaRtTimer timer);
int MusaRtStartTimer(int ordinal, MusaRtStream stream, MusaRtTimer timer);
int MusaRtStopTimer(int ordinal, MusaRtStream stream, MusaRtTimer timer);
uint64_t MusaRtTimerNanoseconds(MusaRtTimer timer);

/* memcpy_dtoh / memcpy_htod / memcpy_dtod and their sync_ forms (:599-700).
 * A pageable host source of a synchronous H2D copy goes through the pinned
 * bounce pool (copy to pinned, async copy on the null stream, synchronise);
 * MUSA_SE_SYNC_H2D=1 forces plain synchronous copies,
 * MUSA_SE_DISABLE_PAGEABLE_H2D_BOUNCE=1 / MUSA_SE_DISABLE_SYNC_H2D_BOUNCE=1
 * switch the bounce off (:127-212). */
int MusaRtMemcpyDtoH(int ordinal, MusaRtStream stream, void* host_dst, const void* device_src, uint64_t size);
int MusaRtMemcpyHtoD(int ordinal, MusaRtStream stream, void* device_dst, const void* host_src, uint64_t size);
int MusaRtMemcpyDtoD(int ordinal, MusaRtStream stream, void* device_dst, const void* device_src, uint64_t size);
int MusaRtSyncMemcpyDtoH(int ordinal, void* host_dst, const void* device_src, uint64_t size);
int MusaRtSyncMemcpyHtoD(int ordinal, void* device_dst, const void* host_src, uint64_t size);
int MusaRtSyncMemcpyDtoD(int ordinal, void* device_dst, const void* device_src, uint64_t size);

/* mem_zero / memset / memset32 (:702-750). */
int MusaRtMemZero(int ordinal, MusaRtStream stream, void* ptr, uint64_t size);
int MusaRtMemset(int ordinal, MusaRtStream stream, void* ptr, uint8_t value, uint64_t size);
int MusaRtMemset32(int ordinal, MusaRtStream stream, void* ptr, uint32_t pattern, uint64_t size);

/* host_callback (:802-835): `fn(arg)` runs after the work queued on `stream`. */
int MusaRtHostCallback(int ordinal, MusaRtStream stream, void (*fn)(void*), void* arg);

/* block_host_until_done / synchronize_all_activity (:752-800). */
int MusaRtBlockHostUntilDone(int ordinal, MusaRtStream stream);
int MusaRtSynchronizeAllActivity(int ordinal);

/* ---- test hooks, with the names of the reference's
 * (musa_ext/mu/musa_se_plugin.cc:887-1146). */
int MUSA_TestPluginGetDeviceCount(int* count);
int MUSA_TestSeRuntimeSmoke(void);       /* relaxed: OK when there is no device */
int MUSA_TestSeRuntimeSmokeStrict(void); /* 9 FAILED_PRECONDITION without a device */
int MUSA_TestRegistryDeviceLifecycle(void); /* fake ordinal 42 through create/destroy */
size_t MUSA_TestSeRegistryLiveOrdinalsForTest(void);
int MUSA_TestDeviceMetadata(int ordinal, char* name, size_t name_cap, int* sm_count, int64_t* total_memory);

/* ---- host-only driver for tests without a GPU (no reference counterpart):
 * select it before the first runtime call of the process. */
void MusaRtUseFakeDriver(int enable);
const char* MusaRtDriverName(void);
void MusaRtFakeSetDeviceCount(int count);
uint64_t MusaRtFakeBlockStream(MusaRtStream stream);
void MusaRtFakeReleaseGate(uint64_t gate);
int64_t MusaRtFakeLiveAllocations(void);
int64_t MusaRtFakeLiveEvents(void);
/* Pinned pool of an ordinal: allocate / free-after-stream / counters
 * (GPUPinnedMemoryPool, musa_ext/mu/device/pinned_memory_pool.h:46-108). */
void* MusaRtPinnedAllocate(int ordinal, uint64_t size);
int MusaRtPinnedFreeAsync(int ordinal, void* ptr, uint64_t size, MusaRtStream stream);
int MusaRtPinnedStats(int ordinal, uint64_t out[7]);
/* Event manager of an ordinal: run fn(arg) on a worker thread once `stream`
 * has completed its queued work (MusaEventMgr::ThenExecute,
 * musa_ext/mu/device/musa_event_mgr.h:58-60). */
int MusaRtThenExecute(int ordinal, MusaRtStream stream, void (*fn)(void*), void* arg);
uint64_t MusaRtEventMgrCallbacksRun(int ordinal);

#ifdef __cplusplus
}
#endif

#endif /* MUSA_PLUGIN_RUNTIME_H_ */
