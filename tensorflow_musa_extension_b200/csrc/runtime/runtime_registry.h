// Per-device runtime state of the PluggableDevice path: reference-counted per
// ordinal from device create / destroy, with the event manager and the pinned
// pool created on first use.  Streams are never looked up by ordinal: a kernel
// takes the stream of its own device context.
//
// Re-target of musa_ext/mu/musa_runtime_registry.{h,cc} (:34-73, :41-134); the
// per-stream muDNN handle of the reference has no counterpart because the
// kernels here need no library handle.
#pragma once

#include <cstdint>
#include <memory>
#include <vector>

#include "event_mgr.h"
#include "pinned_pool.h"

namespace musa_rt {

void RegistryOnDeviceCreated(int32_t ordinal);
void RegistryOnDeviceDestroyed(int32_t ordinal);
void RegistryOnStreamDestroyed(int32_t ordinal, StreamHandle stream);

// nullptr when the ordinal has no live device.
EventMgr* RegistryEventMgr(int32_t ordinal);
PinnedMemoryPool* RegistryPinnedPool(int32_t ordinal);

bool RegistryHasLiveDevice(int32_t ordinal);
int RegistryRefCount(int32_t ordinal);
std::vector<int32_t> RegistryLiveOrdinals();

}  // namespace musa_rt
