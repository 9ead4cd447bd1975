#include "runtime_registry.h"

#include <algorithm>
#include <map>
#include <mutex>

namespace musa_rt {
namespace {

struct DeviceState {
  int ref_count = 0;
  std::unique_ptr<EventMgr> event_mgr;
  std::unique_ptr<PinnedMemoryPool> pinned_pool;
};

std::mutex g_mu;
std::map<int32_t, DeviceState>& States() {
  static auto* m = new std::map<int32_t, DeviceState>();
  return *m;
}

}  // namespace

void RegistryOnDeviceCreated(int32_t ordinal) {
  std::lock_guard<std::mutex> l(g_mu);
  ++States()[ordinal].ref_count;
}

void RegistryOnDeviceDestroyed(int32_t ordinal) {
  DeviceState dead;
  {
    std::lock_guard<std::mutex> l(g_mu);
    auto it = States().find(ordinal);
    if (it == States().end()) return;
    if (--it->second.ref_count > 0) return;
    dead = std::move(it->second);
    States().erase(it);
  }
  // Joins the helper threads outside the registry lock.
  dead.event_mgr.reset();
  dead.pinned_pool.reset();
}

void RegistryOnStreamDestroyed(int32_t, StreamHandle) {
  // Nothing is keyed by stream in this build (the reference drops the
  // stream's library handle here).
}

EventMgr* RegistryEventMgr(int32_t ordinal) {
  std::lock_guard<std::mutex> l(g_mu);
  auto it = States().find(ordinal);
  if (it == States().end() || it->second.ref_count <= 0) return nullptr;
  if (!it->second.event_mgr) {
    it->second.event_mgr.reset(new EventMgr(ActiveDriver(), ordinal));
  }
  return it->second.event_mgr.get();
}

PinnedMemoryPool* RegistryPinnedPool(int32_t ordinal) {
  std::lock_guard<std::mutex> l(g_mu);
  auto it = States().find(ordinal);
  if (it == States().end() || it->second.ref_count <= 0) return nullptr;
  if (!it->second.pinned_pool) {
    it->second.pinned_pool.reset(new PinnedMemoryPool(ActiveDriver(), ordinal));
  }
  return it->second.pinned_pool.get();
}

bool RegistryHasLiveDevice(int32_t ordinal) { return RegistryRefCount(ordinal) > 0; }

int RegistryRefCount(int32_t ordinal) {
  std::lock_guard<std::mutex> l(g_mu);
  auto it = States().find(ordinal);
  return it == States().end() ? 0 : it->second.ref_count;
}

std::vector<int32_t> RegistryLiveOrdinals() {
  std::lock_guard<std::mutex> l(g_mu);
  std::vector<int32_t> out;
  for (const auto& kv : States()) {
    if (kv.second.ref_count > 0) out.push_back(kv.first);
  }
  return out;
}

}  // namespace musa_rt
