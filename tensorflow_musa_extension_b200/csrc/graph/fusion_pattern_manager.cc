#include "fusion_pattern_manager.h"

#include <algorithm>
#include <cstdlib>

namespace musa_graph {

// ---------------------------------------------------- FusionKernelRegistry --

FusionKernelRegistry& FusionKernelRegistry::GetInstance() {
  static FusionKernelRegistry* instance = new FusionKernelRegistry();
  return *instance;
}

void FusionKernelRegistry::RegisterKernel(
    const std::string& pattern_name, std::function<bool()> is_available_func) {
  if (pattern_name.empty()) return;
  std::lock_guard<std::mutex> lock(mu_);
  kernel_availability_[pattern_name] = std::move(is_available_func);
}

bool FusionKernelRegistry::IsKernelAvailable(
    const std::string& pattern_name) const {
  std::function<bool()> probe;
  {
    std::lock_guard<std::mutex> lock(mu_);
    if (implemented_kernels_.count(pattern_name) > 0) return true;
    const auto it = kernel_availability_.find(pattern_name);
    if (it == kernel_availability_.end() || !it->second) return false;
    probe = it->second;
  }
  return probe();
}

std::vector<std::string> FusionKernelRegistry::GetAvailableKernels() const {
  std::vector<std::string> names;
  std::vector<std::pair<std::string, std::function<bool()>>> probes;
  {
    std::lock_guard<std::mutex> lock(mu_);
    names.assign(implemented_kernels_.begin(), implemented_kernels_.end());
    for (const auto& kv : kernel_availability_) {
      if (kv.second && implemented_kernels_.count(kv.first) == 0) {
        probes.emplace_back(kv.first, kv.second);
      }
    }
  }
  for (const auto& p : probes) {
    if (p.second()) names.push_back(p.first);
  }
  std::sort(names.begin(), names.end());
  return names;
}

void FusionKernelRegistry::MarkKernelAsImplemented(
    const std::string& pattern_name) {
  std::lock_guard<std::mutex> lock(mu_);
  implemented_kernels_.insert(pattern_name);
}

// ---------------------------------------------------- FusionPatternManager --

FusionPatternManager& FusionPatternManager::GetInstance() {
  static FusionPatternManager* instance = new FusionPatternManager();
  return *instance;
}

void FusionPatternManager::RegisterPattern(
    std::unique_ptr<FusionPattern> pattern) {
  if (!pattern) return;
  const std::string name = pattern->GetName();
  if (name.empty()) return;
  std::lock_guard<std::mutex> lock(mu_);
  for (const auto& existing : patterns_) {
    if (existing->GetName() == name) return;  // first registration wins
  }
  patterns_.push_back(std::move(pattern));
}

std::vector<const FusionPattern*> FusionPatternManager::GetSortedPatterns()
    const {
  std::vector<const FusionPattern*> out;
  {
    std::lock_guard<std::mutex> lock(mu_);
    for (const auto& p : patterns_) out.push_back(p.get());
  }
  // Priority descending; registration order breaks ties.
  std::stable_sort(out.begin(), out.end(),
                   [](const FusionPattern* a, const FusionPattern* b) {
                     return a->GetPriority() > b->GetPriority();
                   });
  return out;
}

bool FusionPatternManager::HasAvailableKernel(
    const std::string& pattern_name) const {
  const FusionPattern* p = GetPattern(pattern_name);
  return p != nullptr && p->IsKernelAvailable();
}

void FusionPatternManager::SetPatternEnabled(const std::string& pattern_name,
                                             bool enabled) {
  std::lock_guard<std::mutex> lock(mu_);
  for (auto& p : patterns_) {
    if (p->GetName() == pattern_name) p->SetEnabled(enabled);
  }
}

const FusionPattern* FusionPatternManager::GetPattern(
    const std::string& pattern_name) const {
  std::lock_guard<std::mutex> lock(mu_);
  for (const auto& p : patterns_) {
    if (p->GetName() == pattern_name) return p.get();
  }
  return nullptr;
}

std::vector<std::string> FusionPatternManager::GetRegisteredPatternNames()
    const {
  std::vector<std::string> names;
  std::lock_guard<std::mutex> lock(mu_);
  for (const auto& p : patterns_) names.push_back(p->GetName());
  return names;
}

void FusionPatternManager::ClearPatterns() {
  std::lock_guard<std::mutex> lock(mu_);
  patterns_.clear();
}

// -------------------------------------------------------- FusionGraphUtils --

int FusionGraphUtils::FindNodeIndex(const GraphDef& graph,
                                    const std::string& node_name) {
  for (int i = 0; i < graph.node_size(); ++i) {
    if (graph.node[i].name == node_name) return i;
  }
  return -1;
}

const NodeDef* FusionGraphUtils::GetNodeByName(const GraphDef& graph,
                                               const std::string& node_name) {
  const int idx = FindNodeIndex(graph, node_name);
  return idx >= 0 ? &graph.node[idx] : nullptr;
}

bool FusionGraphUtils::HasInput(const NodeDef& node,
                                const std::string& input_name) {
  return std::find(node.input.begin(), node.input.end(), input_name) !=
         node.input.end();
}

std::string FusionGraphUtils::GetProducerNodeName(const std::string& input) {
  if (input.empty()) return "";
  if (input[0] == '^') return input.substr(1);
  const size_t colon = input.find(':');
  return colon == std::string::npos ? input : input.substr(0, colon);
}

const NodeDef* FusionGraphUtils::FindProducer(const GraphDef& graph,
                                              const std::string& input) {
  const std::string name = GetProducerNodeName(input);
  return name.empty() ? nullptr : GetNodeByName(graph, name);
}

void FusionGraphUtils::RemoveNode(GraphDef* graph, int node_idx) {
  if (node_idx < 0 || node_idx >= graph->node_size()) return;
  const int last = graph->node_size() - 1;
  if (node_idx != last) std::swap(graph->node[node_idx], graph->node[last]);
  graph->node.pop_back();
}

int FusionGraphUtils::CountConsumers(
    const GraphDef& graph, const std::string& node_name,
    const std::unordered_set<std::string>& except) {
  int count = 0;
  for (const auto& node : graph.node) {
    if (node.name == node_name || except.count(node.name) > 0) continue;
    for (const auto& in : node.input) {
      if (GetProducerNodeName(in) == node_name) {
        ++count;
        break;
      }
    }
  }
  return count;
}

bool FusionGraphUtils::HasAnyConsumer(const GraphDef& graph,
                                      const std::string& node_name) {
  return CountConsumers(graph, node_name) > 0;
}

int FusionGraphUtils::RemoveNodesIfUnused(
    GraphDef* graph, const std::vector<std::string>& node_names,
    const std::unordered_set<std::string>& protected_node_names) {
  std::vector<std::string> candidates;
  for (const auto& name : node_names) {
    if (name.empty() || protected_node_names.count(name) > 0) continue;
    if (std::find(candidates.begin(), candidates.end(), name) ==
        candidates.end()) {
      candidates.push_back(name);
    }
  }
  // Removing a consumer can free its producer: repeat until nothing changes.
  int removed = 0;
  bool changed = true;
  while (changed) {
    changed = false;
    for (auto it = candidates.begin(); it != candidates.end();) {
      const int idx = FindNodeIndex(*graph, *it);
      if (idx < 0) {
        it = candidates.erase(it);
        continue;
      }
      if (HasAnyConsumer(*graph, *it)) {
        ++it;
        continue;
      }
      RemoveNode(graph, idx);
      it = candidates.erase(it);
      ++removed;
      changed = true;
    }
  }
  return removed;
}

void FusionGraphUtils::RedirectInputs(GraphDef* graph,
                                      const std::string& old_node_name,
                                      const std::string& new_node_name) {
  for (auto& node : graph->node) {
    if (node.name == new_node_name) continue;
    for (auto& in : node.input) {
      if (GetProducerNodeName(in) != old_node_name) continue;
      if (in[0] == '^') {
        in = "^" + new_node_name;
      } else {
        const size_t colon = in.find(':');
        in = colon == std::string::npos ? new_node_name
                                        : new_node_name + in.substr(colon);
      }
    }
  }
}

bool FusionGraphUtils::IsMusaNode(const NodeDef& node) {
  return node.device.find("MUSA") != std::string::npos;
}

bool FusionGraphUtils::IsOpType(const NodeDef& node,
                                const std::string& op_type) {
  return node.op == op_type;
}

bool FusionGraphUtils::EndsWith(const std::string& s,
                                const std::string& suffix) {
  return s.size() >= suffix.size() &&
         s.compare(s.size() - suffix.size(), suffix.size(), suffix) == 0;
}

bool FusionGraphUtils::IsTruthyEnvVar(const char* env_name) {
  const char* v = std::getenv(env_name);
  if (v == nullptr) return false;
  const std::string s(v);
  return s == "1" || s == "true" || s == "TRUE" || s == "yes" || s == "YES" ||
         s == "on" || s == "ON";
}

}  // namespace musa_graph
