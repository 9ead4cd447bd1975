// Driver of the fusion patterns: "musa_graph_optimizer".
//
// Mirrors MusaGraphOptimizer::{Init, Optimize, OptimizeFusion} of the reference
// (musa_ext/mu/optimizer/musa_graph_optimizer.cc:5414-5478, 5480-5833,
// 5843-5995): patterns are grouped by priority (descending); each group is
// swept forward and then in reverse, first match applied and the sweep
// restarted, until a fixed point or 50 iterations; the parameter
// `disabled_fusion_patterns` ("all" or a comma list, trimmed, case-insensitive,
// :5998-6036) switches patterns off.  The layout and mixed-precision passes and
// the model-specific rewrites of the reference are not part of this build.
#pragma once

#include <map>
#include <string>
#include <unordered_set>

#include "fusion_pattern_manager.h"

namespace musa_graph {

constexpr char kOptimizerName[] = "musa_graph_optimizer";
constexpr char kDisabledFusionPatternsParam[] = "disabled_fusion_patterns";
constexpr int kMaxFusionIterations = 50;

struct OptimizeReport {
  int applied = 0;
  int fallbacks = 0;
  int iterations = 0;
  bool hit_iteration_limit = false;
  std::map<std::string, int> applied_by_pattern;
  std::string ToJson() const;
};

class MusaGraphOptimizer {
 public:
  // Parameters as key -> value strings (the Grappler custom-optimizer
  // parameter_map).  Unknown keys are rejected; known ones that configure
  // passes outside this build are accepted and ignored.
  Status Init(const std::map<std::string, std::string>& params);
  Status Optimize(GraphDef* graph, OptimizeReport* report) const;

  void SetDisabledFusionPatterns(const std::string& disabled_patterns);
  bool IsFusionPatternDisabled(const std::string& pattern_name) const;
  static std::string NormalizeFusionPatternName(const std::string& value);

 private:
  bool disable_all_ = false;
  std::unordered_set<std::string> disabled_;
};

}  // namespace musa_graph
