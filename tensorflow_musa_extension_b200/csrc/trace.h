// Optional tracing of the launcher layer: an NVTX range around every launcher
// call and per-launcher counters (calls, kernel launches, algorithmic bytes,
// host time spent in the call).  Off by default; MUSA_B200_TRACE=1 in the environment or
// MusaKernelsTraceEnable(1) turns it on.  When it is off a launcher pays one
// relaxed atomic load.
//
// The reference traces its allocator and copy paths only and leaves kernels
// untraced (mu/device/musa_telemetry.h:47-199; its kernel timing macros were
// removed, docs/DEBUG_GUIDE.md:3,192); this is the kernel-side counterpart.
#pragma once

#include <stdint.h>

#include <atomic>

namespace musa_b200 {

extern std::atomic<int> g_trace_state;  // -1 unknown, 0 off, 1 on
bool TraceInit();
inline bool TraceOn() {
  const int s = g_trace_state.load(std::memory_order_relaxed);
  return s > 0 || (s < 0 && TraceInit());
}

// Kernel launches made by the library since it was loaded (every launch site
// counts; one relaxed add).  A LaunchScope attributes the launches made while
// it is open to its launcher (exact as long as one thread launches at a time).
extern std::atomic<long long> g_kernel_launches;
inline void CountKernelLaunch() { g_kernel_launches.fetch_add(1, std::memory_order_relaxed); }

class LaunchScope {
 public:
  LaunchScope(const char* name, int64_t bytes) : slot_(-1) {
    if (TraceOn()) Begin(name, bytes);
  }
  ~LaunchScope() {
    if (slot_ >= 0) End();
  }
  LaunchScope(const LaunchScope&) = delete;
  LaunchScope& operator=(const LaunchScope&) = delete;

 private:
  void Begin(const char* name, int64_t bytes);
  void End();
  int slot_;
  int64_t t0_;
  long long launches0_;
};

}  // namespace musa_b200

// `bytes`: the algorithmic bytes of the call (what the op has to move), as in
// the roofline figures; 0 where a launcher has no such figure.
#define MUSA_TRACE(name, bytes) \
  ::musa_b200::LaunchScope musa_trace_scope_(name, static_cast<int64_t>(bytes))
