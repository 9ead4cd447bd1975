// Process-wide launch-shape knobs.  The defaults are the shipped
// configuration; MusaKernelsSetTuning() exists so that a sweep can compare
// launch shapes without rebuilding.  Launchers only read these values.
#pragma once

namespace musa_b200 {

enum TuningKey {
  kTuneAdamCtasPerSm = 0,   // 0: one tile per CTA; k: persistent, k CTAs per SM
  kTuneAdamUnroll = 1,      // packs in flight per thread and stream: 1, 2, 4
  kTuneBiasActCtasPerSm = 2,
  kTuneBiasActUnroll = 3,
  kTuneBnCtasPerSm = 4,     // CTAs per SM of the BatchNorm statistics grids; 0: what fits
  kTuneBnClusterFold = 5,   // CTAs per cluster of the stats kernel that fold their partial rows on chip
                            // (the element-wise kernel adds the rest: no finalize kernel); 0, 1: off
  kTuneBnApplyReverse = 6,  // 1: apply pass walks rows in reverse (L2 reuse)
  kTuneBnStatsKeep = 7,     // 1: stats pass loads with the default L2 policy
  kTuneBnStatsPipe = 8,     // cp.async stages of the stats kernel (3 or 4); 0: register loads
  kTuneBnApplyDeep = 9,     // 1: forward element-wise pass keeps 8 rows in flight
  kTuneBnPdl = 10,          // 1: BatchNorm kernels use programmatic dependent launch
  kTuneBnL2KeepMb = 11,     // MB of its reads that the stats pass asks L2 to hold back (0: off)
  kTuneRowNormPacks = 12,   // packs per thread of the row kernels: 1 .. 4; 0: chosen per op and row
  kTuneBnApplyAddsRows = 13,  // the element-wise kernel adds up to this many partial rows itself (no
                              // finalize kernel); 0: never
  kTuneBnStatsMaxTx = 14,   // channel packs per column block of the stats kernel; 0: by rule
  kTuneBnL2KeepPartial = 15,  // 1: tensors beyond the budget keep the budget's share
  kTuneBnStatsDropRest = 16,  // 1: rows outside the kept share are read evict-first
  kTuneBnApplyDropAll = 17,   // 1: the element-wise pass reads evict-first at every size
  kTuneBnApplyEarlyLoads = 18,  // 1: first rows of the element-wise pass are loaded before its wait
  kTuneBnFinalizeLanes = 19,  // partial lanes per CTA of the finalize kernel: 32 or 128
  kTuneBnApplyCtasPerSm = 20,  // CTAs per SM of the element-wise grids; 0: what fits
  kTuneBnInterleave = 21,   // 1: CTAs take row tiles round-robin instead of one contiguous range
  kTuneBnApplyMaxTx = 22,   // channel packs per column block of the element-wise kernel; 0: the row
  kTuneBnFullWave = 23,     // 1: with interleaved row tiles the grid keeps the full wave (no shrink to whole row ranges)
  kTuneCount = 24
};

int GetTuning(int key);

}  // namespace musa_b200
