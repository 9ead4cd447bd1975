// GraphDef dumps around the optimizer's passes (the reference's
// GraphDefDumper, musa_ext/mu/optimizer/graph_utils.h:29-58) and the
// allow-growth switch of the device registration
// (musa_ext/mu/device_register.cc:34-72).
#pragma once

#include <string>

#include "graph_def.h"

namespace musa_graph {

bool IsGraphDefDumpingEnabled();
std::string GetDumpDirectory();
bool IsGraphDefTextDumpEnabled();
bool IsSlimGraphDefDumpEnabled();

// Human-readable listing of the decoded part of a graph (text-format subset).
std::string GraphDefToText(const GraphDef& graph);
// Copy without tensor payloads, shapes, lists and undecoded fields.
GraphDef SlimGraphDef(const GraphDef& graph);

class GraphDefDumper {
 public:
  explicit GraphDefDumper(const std::string& optimizer_name);
  // Writes <dir>/<optimizer>_<id:04>_<stage>.pb (+ .slim.pb, .pbtxt when
  // enabled); a no-op returning true when dumping is off.
  bool DumpAtStage(const GraphDef& graph, const std::string& stage);
  bool DumpInitial(const GraphDef& g) { return DumpAtStage(g, "initial"); }
  bool DumpFinal(const GraphDef& g) { return DumpAtStage(g, "final"); }
  bool DumpBeforePass(const GraphDef& g, const std::string& pass) {
    return DumpAtStage(g, "before_" + pass);
  }
  bool DumpAfterPass(const GraphDef& g, const std::string& pass) {
    return DumpAtStage(g, "after_" + pass);
  }
  int dump_id() const { return dump_id_; }

 private:
  std::string optimizer_name_;
  int dump_id_;
};

bool GetAllowGrowth();
void SetAllowGrowth(bool enabled);

}  // namespace musa_graph
