#include "musa_graph_optimizer.h"
#include "graph_dump.h"

#include <algorithm>
#include <cctype>
#include <cstring>
#include <functional>
#include <sstream>

#include "../../../include/musa_plugin_graph.h"

namespace musa_graph {

void LinkBiasAddActivationFusion();
void LinkAdamMixedFusion();
void LinkBiasAddReluGradFusion();

std::string OptimizeReport::ToJson() const {
  std::ostringstream os;
  os << "{\"applied\": " << applied << ", \"fallbacks\": " << fallbacks
     << ", \"iterations\": " << iterations << ", \"hit_iteration_limit\": "
     << (hit_iteration_limit ? "true" : "false") << ", \"patterns\": {";
  bool first = true;
  for (const auto& kv : applied_by_pattern) {
    os << (first ? "" : ", ") << "\"" << kv.first << "\": " << kv.second;
    first = false;
  }
  os << "}}";
  return os.str();
}

std::string MusaGraphOptimizer::NormalizeFusionPatternName(
    const std::string& value) {
  size_t b = 0, e = value.size();
  while (b < e && std::isspace(static_cast<unsigned char>(value[b]))) ++b;
  while (e > b && std::isspace(static_cast<unsigned char>(value[e - 1]))) --e;
  std::string out = value.substr(b, e - b);
  std::transform(out.begin(), out.end(), out.begin(), [](unsigned char c) {
    return static_cast<char>(std::tolower(c));
  });
  return out;
}

void MusaGraphOptimizer::SetDisabledFusionPatterns(
    const std::string& disabled_patterns) {
  disabled_.clear();
  disable_all_ = false;
  std::stringstream ss(disabled_patterns);
  std::string token;
  while (std::getline(ss, token, ',')) {
    const std::string name = NormalizeFusionPatternName(token);
    if (name.empty()) continue;
    if (name == "all") {
      disable_all_ = true;
      disabled_.clear();
      return;
    }
    disabled_.insert(name);
  }
}

bool MusaGraphOptimizer::IsFusionPatternDisabled(
    const std::string& pattern_name) const {
  return disable_all_ ||
         disabled_.count(NormalizeFusionPatternName(pattern_name)) > 0;
}

Status MusaGraphOptimizer::Init(
    const std::map<std::string, std::string>& params) {
  for (const auto& kv : params) {
    if (kv.first == kDisabledFusionPatternsParam) {
      SetDisabledFusionPatterns(kv.second);
    } else if (kv.first == "aggressive_mode" || kv.first == "precision_mode" ||
               kv.first == "disable_layout_optimizer" ||
               kv.first == "disable_amp") {
      // Parameters of the layout / mixed-precision passes: accepted so that an
      // existing ConfigProto keeps working; those passes do not exist here.
    } else {
      return Status::InvalidArgument("unknown " + std::string(kOptimizerName) +
                                     " parameter: " + kv.first);
    }
  }
  return Status::OK();
}

Status MusaGraphOptimizer::Optimize(GraphDef* graph,
                                    OptimizeReport* report) const {
  LinkBiasAddActivationFusion();
  LinkAdamMixedFusion();
  LinkBiasAddReluGradFusion();
  OptimizeReport local;
  OptimizeReport& rep = report != nullptr ? *report : local;
  rep = OptimizeReport();
  if (graph == nullptr) return Status::InvalidArgument("null graph");
  if (graph->node.empty()) return Status::OK();
  // Dumps at the stages of the reference's Optimize()
  // (musa_ext/mu/optimizer/musa_graph_optimizer.cc:5486-5517); the layout and
  // AMP passes are not part of this build, so only the fusion pass appears.
  GraphDefDumper dumper("musa_graph_optimizer");
  dumper.DumpInitial(*graph);
  dumper.DumpBeforePass(*graph, "fusion");
  struct FinalDump {
    GraphDefDumper* d;
    GraphDef* g;
    ~FinalDump() {
      d->DumpAfterPass(*g, "fusion");
      d->DumpFinal(*g);
    }
  } final_dump{&dumper, graph};

  const auto patterns = FusionPatternManager::GetInstance().GetSortedPatterns();
  std::map<int, std::vector<const FusionPattern*>, std::greater<int>> groups;
  for (const FusionPattern* p : patterns) {
    if (!p->IsEnabled() || IsFusionPatternDisabled(p->GetName())) continue;
    groups[p->GetPriority()].push_back(p);
  }
  if (groups.empty()) return Status::OK();

  // One scan direction: apply the first match, restart, stop when a whole
  // sweep applies nothing.  Returns whether the graph changed.
  auto run_scan = [&](const std::vector<const FusionPattern*>& active,
                      bool reverse) {
    bool modified = false;
    // Guard against a pattern whose Apply reports success without removing
    // its own match: a sweep may restart at most once per node and pattern.
    int restarts = 0;
    const int restart_cap =
        kMaxFusionIterations * std::max(1, graph->node_size());
    while (restarts++ <= restart_cap) {
      bool applied = false;
      const int count = graph->node_size();
      for (int off = 0; off < count && !applied; ++off) {
        const int idx = reverse ? count - 1 - off : off;
        for (const FusionPattern* p : active) {
          const FusionMatchResult m = p->Match(*graph, idx);
          if (!m.matched) continue;
          if (!p->IsKernelAvailable()) {
            p->Apply(graph, m);  // the pattern's own fallback (a no-op here)
            ++rep.fallbacks;
            continue;
          }
          if (p->Apply(graph, m).ok()) {
            modified = applied = true;
            ++rep.applied;
            ++rep.applied_by_pattern[p->GetName()];
            break;
          }
        }
      }
      if (!applied) break;
    }
    return modified;
  };

  bool graph_modified = true;
  while (graph_modified && rep.iterations < kMaxFusionIterations) {
    graph_modified = false;
    ++rep.iterations;
    for (const auto& group : groups) {
      bool group_modified = true;
      int group_iterations = 0;
      while (group_modified && group_iterations < kMaxFusionIterations) {
        group_modified = false;
        ++group_iterations;
        if (run_scan(group.second, false)) group_modified = graph_modified = true;
        if (run_scan(group.second, true)) group_modified = graph_modified = true;
      }
      if (group_modified) rep.hit_iteration_limit = true;
    }
  }
  if (graph_modified) rep.hit_iteration_limit = true;
  return Status::OK();
}

namespace {

// "key=value;key=value" -> map.  Values may contain commas and '='.
std::map<std::string, std::string> ParseParams(const char* text) {
  std::map<std::string, std::string> out;
  if (text == nullptr) return out;
  std::stringstream ss(text);
  std::string item;
  while (std::getline(ss, item, ';')) {
    const size_t eq = item.find('=');
    const std::string key = MusaGraphOptimizer::NormalizeFusionPatternName(
        eq == std::string::npos ? item : item.substr(0, eq));
    if (key.empty()) continue;
    out[key] = eq == std::string::npos ? "" : item.substr(eq + 1);
  }
  return out;
}

void CopyText(const std::string& s, char* buf, size_t cap) {
  if (buf == nullptr || cap == 0) return;
  const size_t n = std::min(cap - 1, s.size());
  std::memcpy(buf, s.data(), n);
  buf[n] = '\0';
}

}  // namespace
}  // namespace musa_graph

using namespace musa_graph;

extern "C" {

const char* MusaGraphOptimizerName(void) { return kOptimizerName; }

int MusaGraphOptimizerRun(const void* graph_def, size_t graph_def_size,
                          const char* params, void** out_graph_def,
                          size_t* out_size, char* report, size_t report_cap) {
  if (out_graph_def == nullptr || out_size == nullptr) return Status::kInvalidArgument;
  *out_graph_def = nullptr;
  *out_size = 0;
  if (graph_def == nullptr && graph_def_size != 0) return Status::kInvalidArgument;
  MusaGraphOptimizer opt;
  const Status init = opt.Init(ParseParams(params));
  if (!init.ok()) {
    CopyText(init.message, report, report_cap);
    return init.code;
  }
  GraphDef graph;
  if (!graph.ParseFromArray(graph_def, graph_def_size)) {
    CopyText("malformed GraphDef", report, report_cap);
    return Status::kInvalidArgument;
  }
  OptimizeReport rep;
  const Status st = opt.Optimize(&graph, &rep);
  if (!st.ok()) {
    CopyText(st.message, report, report_cap);
    return st.code;
  }
  const std::string bytes = graph.SerializeAsString();
  void* mem = std::malloc(bytes.size() > 0 ? bytes.size() : 1);
  if (mem == nullptr) return Status::kInternal;
  std::memcpy(mem, bytes.data(), bytes.size());
  *out_graph_def = mem;
  *out_size = bytes.size();
  CopyText(rep.ToJson(), report, report_cap);
  return Status::kOk;
}

void MusaGraphOptimizerFree(void* graph_def) { std::free(graph_def); }

int MusaGraphOptimizerListPatterns(char* buf, size_t cap) {
  LinkBiasAddActivationFusion();
  LinkAdamMixedFusion();
  LinkBiasAddReluGradFusion();
  std::ostringstream os;
  const auto patterns = FusionPatternManager::GetInstance().GetSortedPatterns();
  for (const FusionPattern* p : patterns) {
    os << p->GetName() << ":" << p->GetPriority() << ":"
       << (p->IsKernelAvailable() ? 1 : 0) << "\n";
  }
  CopyText(os.str(), buf, cap);
  return static_cast<int>(patterns.size());
}

int MusaGraphSetPatternEnabled(const char* pattern_name, int enabled) {
  if (pattern_name == nullptr) return Status::kInvalidArgument;
  if (FusionPatternManager::GetInstance().GetPattern(pattern_name) == nullptr) {
    return Status::kNotFound;
  }
  FusionPatternManager::GetInstance().SetPatternEnabled(pattern_name, enabled != 0);
  return Status::kOk;
}

}  // extern "C"
