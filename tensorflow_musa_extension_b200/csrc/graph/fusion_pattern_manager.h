// Fusion-pattern framework of the MUSA graph optimizer: the pattern interface,
// the pattern and kernel registries and the graph-editing helpers, with the
// interface of the reference (musa_ext/graph/fusion/fusion_pattern_manager.h:
// 35-202) over the TF-free GraphDef of graph_def.h.
//
// Contract kept from the reference:
//   * a pattern matches from the LAST node of a chain (the activation, the Mul,
//     the optimizer op) and never starts from a node named "<x>_original";
//   * Apply renames the matched output to "<name>_original", adds the fused
//     node under the original name and device, and removes the old nodes only
//     if nothing else consumes them (protected inputs are never removed);
//   * Apply is idempotent across sweeps and looks nodes up by name again,
//     because earlier rewrites of the same sweep invalidate indices;
//   * higher priority is applied first.
#pragma once

#include <functional>
#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <unordered_map>
#include <unordered_set>
#include <vector>

#include "graph_def.h"

namespace musa_graph {

// tensorflow::Status, reduced to what the optimizer needs.
struct Status {
  enum Code { kOk = 0, kInvalidArgument = 3, kNotFound = 5, kInternal = 13 };
  Code code = kOk;
  std::string message;
  bool ok() const { return code == kOk; }
  static Status OK() { return Status(); }
  static Status InvalidArgument(std::string m) {
    return Status{kInvalidArgument, std::move(m)};
  }
  static Status NotFound(std::string m) { return Status{kNotFound, std::move(m)}; }
};

struct FusionMatchResult {
  bool matched = false;
  // Names, not pointers: the graph's node vector moves when a sweep edits it.
  std::vector<std::string> matched_nodes;
  std::map<std::string, std::string> captured_nodes;  // role -> node name
  std::map<std::string, std::string> captured_attrs;

  bool IsValid() const { return matched && !matched_nodes.empty(); }
  void Reset() {
    matched = false;
    matched_nodes.clear();
    captured_nodes.clear();
    captured_attrs.clear();
  }
};

class FusionPattern {
 public:
  virtual ~FusionPattern() = default;
  virtual FusionMatchResult Match(const GraphDef& graph,
                                  int start_node_idx) const = 0;
  virtual Status Apply(GraphDef* graph,
                       const FusionMatchResult& match_result) const = 0;
  virtual int GetPriority() const = 0;  // higher = applied first
  virtual bool IsKernelAvailable() const = 0;
  virtual std::string GetName() const = 0;
  virtual std::string GetFallbackReason() const { return ""; }

  void SetEnabled(bool enabled) { enabled_ = enabled; }
  bool IsEnabled() const { return enabled_; }

 protected:
  bool enabled_ = true;
};

class FusionKernelRegistry {
 public:
  static FusionKernelRegistry& GetInstance();
  void RegisterKernel(const std::string& pattern_name,
                      std::function<bool()> is_available_func);
  bool IsKernelAvailable(const std::string& pattern_name) const;
  std::vector<std::string> GetAvailableKernels() const;
  void MarkKernelAsImplemented(const std::string& pattern_name);

 private:
  FusionKernelRegistry() = default;
  mutable std::mutex mu_;
  std::unordered_map<std::string, std::function<bool()>> kernel_availability_;
  std::unordered_set<std::string> implemented_kernels_;
};

class FusionPatternManager {
 public:
  static FusionPatternManager& GetInstance();
  void RegisterPattern(std::unique_ptr<FusionPattern> pattern);
  std::vector<const FusionPattern*> GetSortedPatterns() const;
  bool HasAvailableKernel(const std::string& pattern_name) const;
  void SetPatternEnabled(const std::string& pattern_name, bool enabled);
  const FusionPattern* GetPattern(const std::string& pattern_name) const;
  std::vector<std::string> GetRegisteredPatternNames() const;
  void ClearPatterns();

 private:
  FusionPatternManager() = default;
  mutable std::mutex mu_;
  std::vector<std::unique_ptr<FusionPattern>> patterns_;
};

#define REGISTER_FUSION_PATTERN(PatternClass)                        \
  static struct PatternClass##Registrar {                            \
    PatternClass##Registrar() {                                      \
      ::musa_graph::FusionPatternManager::GetInstance().RegisterPattern( \
          std::make_unique<PatternClass>());                         \
    }                                                                \
  } g_##PatternClass##_registrar;

#define REGISTER_FUSION_KERNEL(PatternName, IsAvailableFunc)          \
  static struct PatternName##KernelRegistrar {                        \
    PatternName##KernelRegistrar() {                                  \
      ::musa_graph::FusionKernelRegistry::GetInstance().RegisterKernel( \
          #PatternName, IsAvailableFunc);                             \
    }                                                                 \
  } g_##PatternName##_kernel_registrar;

class FusionGraphUtils {
 public:
  static int FindNodeIndex(const GraphDef& graph, const std::string& node_name);
  static const NodeDef* GetNodeByName(const GraphDef& graph,
                                      const std::string& node_name);
  static bool HasInput(const NodeDef& node, const std::string& input_name);
  // "^name" and "name:port" both give "name".
  static std::string GetProducerNodeName(const std::string& input);
  static const NodeDef* FindProducer(const GraphDef& graph,
                                     const std::string& input);
  static void RemoveNode(GraphDef* graph, int node_idx);
  static bool HasAnyConsumer(const GraphDef& graph, const std::string& node_name);
  // Data and control consumers of `node_name`, not counting `node_name` itself
  // nor the nodes in `except`.
  static int CountConsumers(const GraphDef& graph, const std::string& node_name,
                            const std::unordered_set<std::string>& except = {});
  static int RemoveNodesIfUnused(
      GraphDef* graph, const std::vector<std::string>& node_names,
      const std::unordered_set<std::string>& protected_node_names = {});
  static void RedirectInputs(GraphDef* graph, const std::string& old_node_name,
                             const std::string& new_node_name);
  static bool IsMusaNode(const NodeDef& node);
  static bool IsOpType(const NodeDef& node, const std::string& op_type);
  static bool EndsWith(const std::string& s, const std::string& suffix);
  // "1", "true", "TRUE", "yes", "YES", "on", "ON"
  static bool IsTruthyEnvVar(const char* env_name);
};

}  // namespace musa_graph
