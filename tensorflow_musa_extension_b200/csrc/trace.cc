// Launcher tracing: NVTX ranges and per-launcher counters (see trace.h).
#include "trace.h"

#include <nvtx3/nvToolsExt.h>

#include <chrono>
#include <cstdlib>
#include <cstring>
#include <mutex>

#include "../../include/musa_plugin_kernels.h"

namespace musa_b200 {

std::atomic<int> g_trace_state{-1};
std::atomic<long long> g_kernel_launches{0};

namespace {
constexpr int kMaxSlots = 128;
struct Slot {
  const char* name;  // string literal of the call site
  std::atomic<long long> calls, bytes, host_ns, kernels;
};
Slot g_slots[kMaxSlots];
std::atomic<int> g_used{0};
std::mutex g_slot_mutex;

int64_t NowNs() {
  return std::chrono::duration_cast<std::chrono::nanoseconds>(
             std::chrono::steady_clock::now().time_since_epoch())
      .count();
}

int FindSlot(const char* name) {
  const int used = g_used.load(std::memory_order_acquire);
  for (int i = 0; i < used; ++i) {
    if (g_slots[i].name == name || std::strcmp(g_slots[i].name, name) == 0) return i;
  }
  std::lock_guard<std::mutex> lock(g_slot_mutex);
  const int now = g_used.load(std::memory_order_acquire);
  for (int i = used; i < now; ++i) {
    if (std::strcmp(g_slots[i].name, name) == 0) return i;
  }
  if (now >= kMaxSlots) return -1;
  g_slots[now].name = name;
  g_used.store(now + 1, std::memory_order_release);
  return now;
}
}  // namespace

bool TraceInit() {
  const char* env = std::getenv("MUSA_B200_TRACE");
  const int on = env != nullptr && env[0] != '\0' && env[0] != '0' ? 1 : 0;
  int expected = -1;
  g_trace_state.compare_exchange_strong(expected, on);
  return g_trace_state.load(std::memory_order_relaxed) > 0;
}

void LaunchScope::Begin(const char* name, int64_t bytes) {
  slot_ = FindSlot(name);
  nvtxRangePushA(name);
  if (slot_ < 0) {
    slot_ = kMaxSlots;  // range only: the table is full
    return;
  }
  g_slots[slot_].calls.fetch_add(1, std::memory_order_relaxed);
  g_slots[slot_].bytes.fetch_add(bytes, std::memory_order_relaxed);
  launches0_ = g_kernel_launches.load(std::memory_order_relaxed);
  t0_ = NowNs();
}

void LaunchScope::End() {
  if (slot_ < kMaxSlots) {
    g_slots[slot_].host_ns.fetch_add(NowNs() - t0_, std::memory_order_relaxed);
    g_slots[slot_].kernels.fetch_add(
        g_kernel_launches.load(std::memory_order_relaxed) - launches0_,
        std::memory_order_relaxed);
  }
  nvtxRangePop();
}

}  // namespace musa_b200

using namespace musa_b200;

extern "C" {

int MusaKernelsTraceEnable(int on) {
  TraceOn();  // settle the environment default first
  return g_trace_state.exchange(on ? 1 : 0) > 0 ? 1 : 0;
}

int MusaKernelsTraceSnapshot(MusaLaunchCounter* out, int max_entries) {
  const int used = g_used.load(std::memory_order_acquire);
  if (out == nullptr) return used;
  int n = 0;
  for (int i = 0; i < used && n < max_entries; ++i, ++n) {
    out[n].name = g_slots[i].name;
    out[n].calls = g_slots[i].calls.load(std::memory_order_relaxed);
    out[n].bytes = g_slots[i].bytes.load(std::memory_order_relaxed);
    out[n].host_ns = g_slots[i].host_ns.load(std::memory_order_relaxed);
    out[n].kernels = g_slots[i].kernels.load(std::memory_order_relaxed);
  }
  return n;
}

long long MusaKernelsLaunchCount(void) {
  return g_kernel_launches.load(std::memory_order_relaxed);
}

void MusaKernelsTraceReset(void) {
  const int used = g_used.load(std::memory_order_acquire);
  for (int i = 0; i < used; ++i) {
    g_slots[i].calls.store(0, std::memory_order_relaxed);
    g_slots[i].bytes.store(0, std::memory_order_relaxed);
    g_slots[i].host_ns.store(0, std::memory_order_relaxed);
    g_slots[i].kernels.store(0, std::memory_order_relaxed);
  }
}

}  // extern "C"
