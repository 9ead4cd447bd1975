// Library identity, per-device SM count cache and the tuning table.
#include <atomic>
#include <mutex>

#include "common.cuh"
#include "tuning.h"
#include "../../include/musa_plugin_kernels.h"

namespace musa_b200 {

namespace {
std::atomic<int> g_sm_count[kMaxDevices];
std::atomic<int> g_tuning[kTuneCount];
std::once_flag g_tuning_once;

void InitTuningOnce() {
  std::call_once(g_tuning_once, [] {
    static const int defaults[kTuneCount] = {
        /*AdamCtasPerSm*/ 0, /*AdamUnroll*/ 2, /*BiasActCtasPerSm*/ 0,
        /*BiasActUnroll*/ 4, /*BnCtasPerSm*/ 0, /*BnClusterFold*/ 0,
        /*BnApplyReverse*/ 1, /*BnStatsKeep*/ 1, /*BnStatsPipe*/ 4,
        /*BnApplyDeep*/ 1, /*BnPdl*/ 1, /*BnL2KeepMb*/ 64, /*RowNormPacks*/ 0,
        /*BnApplyAddsRows*/ 64, /*BnStatsMaxTx*/ 16, /*BnL2KeepPartial*/ 1,
        /*BnStatsDropRest*/ 1, /*BnApplyDropAll*/ 0, /*BnApplyEarlyLoads*/ 1,
        /*BnFinalizeLanes*/ 128, /*BnApplyCtasPerSm*/ 0, /*BnInterleave*/ 1,
        /*BnApplyMaxTx*/ 16, /*BnFullWave*/ 1};
    for (int i = 0; i < kTuneCount; ++i) g_tuning[i].store(defaults[i]);
  });
}
}  // namespace

int SmCount() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    return 148;
  }
  int n = g_sm_count[dev].load(std::memory_order_relaxed);
  if (n > 0) return n;
  if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) !=
          cudaSuccess ||
      n <= 0) {
    n = 148;
  }
  g_sm_count[dev].store(n, std::memory_order_relaxed);
  return n;
}

int GetTuning(int key) {
  InitTuningOnce();
  if (key < 0 || key >= kTuneCount) return 0;
  return g_tuning[key].load(std::memory_order_relaxed);
}

}  // namespace musa_b200

extern "C" {

const char* MusaKernelsVersion(void) {
  return "musa_plugin_kernels-b200 0.1 (sm_100a)";
}

int MusaKernelsTargetArch(void) { return 100; }

// Sweep/test hook, not part of the reference boundary: sets one launch-shape
// knob for the whole process and returns the previous value (-1: bad key).
int MusaKernelsSetTuning(int key, int value) {
  musa_b200::InitTuningOnce();
  if (key < 0 || key >= musa_b200::kTuneCount) return -1;
  return musa_b200::g_tuning[key].exchange(value);
}

int MusaKernelsGetTuning(int key) { return musa_b200::GetTuning(key); }

}  // extern "C"
