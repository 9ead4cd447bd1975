// Cast(bf16/f16 -> f32) -> ResourceApplyAdam(T = float)
//   =>  MusaResourceApplyAdamMixed(T = bf16/f16), the Cast dropped when the
//       optimizer op was its only reader.
// Same rewrite, priority (40), name and kill switch as the reference pattern
// (musa_ext/graph/fusion/adam_mixed_fusion.cc:93-216, adam_mixed_fusion.h:43-63).
#include "fusion_pattern_manager.h"

namespace musa_graph {
namespace {

using U = FusionGraphUtils;

class MusaAdamMixedFusion : public FusionPattern {
 public:
  FusionMatchResult Match(const GraphDef& graph, int idx) const override {
    FusionMatchResult r;
    if (idx < 0 || idx >= graph.node_size()) return r;
    const NodeDef& adam = graph.node[idx];
    // Only the stock op that Keras' Adam emits; an optimizer op whose state is
    // itself 16-bit is left alone.
    if (adam.op != "ResourceApplyAdam" || !U::IsMusaNode(adam)) return r;
    if (adam.AttrType("T") != DT_FLOAT) return r;
    // var, m, v, beta1_power, beta2_power, lr, beta1, beta2, epsilon, grad
    if (adam.input.size() < 10) return r;
    const NodeDef* cast = U::FindProducer(graph, adam.input[9]);
    if (cast == nullptr || cast->op != "Cast") return r;
    if (cast->AttrType("DstT") != DT_FLOAT) return r;
    const int src = cast->AttrType("SrcT");
    if (src != DT_BFLOAT16 && src != DT_HALF) return r;
    if (cast->input.empty()) return r;
    r.matched = true;
    r.matched_nodes = {adam.name, cast->name};
    r.captured_nodes["adam"] = adam.name;
    r.captured_nodes["cast"] = cast->name;
    r.captured_attrs["grad_dtype"] = src == DT_BFLOAT16 ? "BFLOAT16" : "HALF";
    return r;
  }

  Status Apply(GraphDef* graph, const FusionMatchResult& m) const override {
    if (!m.IsValid()) return Status::InvalidArgument("Invalid Adam-mixed match");
    if (!IsKernelAvailable()) return Status::OK();
    const auto adam_it = m.captured_nodes.find("adam");
    const auto cast_it = m.captured_nodes.find("cast");
    if (adam_it == m.captured_nodes.end() || cast_it == m.captured_nodes.end()) {
      return Status::InvalidArgument("Missing captured nodes in Adam-mixed pattern");
    }
    const std::string adam_name = adam_it->second, cast_name = cast_it->second;
    const int adam_idx = U::FindNodeIndex(*graph, adam_name);
    if (adam_idx < 0) return Status::NotFound("Adam node disappeared before rewrite");
    NodeDef& adam = graph->node[adam_idx];
    if (adam.op == "MusaResourceApplyAdamMixed") return Status::OK();  // idempotent
    if (adam.op != "ResourceApplyAdam" || adam.input.size() < 10) {
      return Status::NotFound("Adam node changed before rewrite");
    }
    const NodeDef* cast = U::GetNodeByName(*graph, cast_name);
    if (cast == nullptr || cast->op != "Cast" || cast->input.empty()) {
      return Status::NotFound("Cast node changed before rewrite");
    }
    if (cast->AttrType("DstT") != DT_FLOAT) return Status::NotFound("Cast DstT changed");
    const int src = cast->AttrType("SrcT");
    if (src != DT_BFLOAT16 && src != DT_HALF) return Status::NotFound("Cast SrcT changed");
    const std::string grad_input = cast->input[0];
    if (grad_input.empty()) return Status::NotFound("Cast has no data input");
    const int other_readers = U::CountConsumers(*graph, cast_name, {adam_name});

    adam.op = "MusaResourceApplyAdamMixed";
    adam.attr["T"] = AttrValue::Type(src);
    adam.input[9] = grad_input;
    if (other_readers == 0) {
      U::RemoveNodesIfUnused(graph, {cast_name},
                             {adam_name, U::GetProducerNodeName(grad_input)});
    }
    return Status::OK();
  }

  int GetPriority() const override { return 40; }
  bool IsKernelAvailable() const override {
    return !U::IsTruthyEnvVar("MUSA_DISABLE_ADAM_MIXED_FUSION");
  }
  std::string GetName() const override { return "MusaAdamMixedFusion"; }
  std::string GetFallbackReason() const override {
    return "disabled by MUSA_DISABLE_ADAM_MIXED_FUSION";
  }
};

}  // namespace

REGISTER_FUSION_PATTERN(MusaAdamMixedFusion);
REGISTER_FUSION_KERNEL(MusaAdamMixedFusion, []() { return true; });

void LinkAdamMixedFusion() {}

}  // namespace musa_graph
