// Graph pattern for the backward of a BiasAdd -> Relu chain:
//   dz = ReluGrad(dy, y);  db = BiasAddGrad(dz)
//     -> (dz, db) = MusaBiasAddReluGrad(dy, y)
// The reference runs the two ops one after the other
// (musa_ext/kernels/nn/musa_relu_grad_op.cc,
// musa_ext/kernels/nn/musa_biasadd_grad_op.cc): five passes over the tensor
// where three are needed.  New pattern in the reference's registry, written to
// the protocol of musa_ext/graph/fusion/linear_activation_fusion.cc:42-47,
// :164-251: match from the last node of the chain, never from a "*_original"
// node, carry T and the device over, remove the old nodes only when nothing
// reads them.
//
// ReluGrad usually has other readers (the gradients of the layer's MatMul), so
// the fused node takes the ReluGrad's name with backprops as output 0: those
// readers stay as they are.  The readers of the BiasAddGrad are pointed at
// output 1 of the fused node.
#include <unordered_set>

#include "fusion_pattern_manager.h"

namespace musa_graph {
namespace {

using U = FusionGraphUtils;

constexpr char kKillSwitch[] = "MUSA_DISABLE_BIASADD_RELU_GRAD_FUSION";
constexpr char kFusedOp[] = "MusaBiasAddReluGrad";

bool IsFloatLike(int dt) {
  return dt == DT_FLOAT || dt == DT_HALF || dt == DT_BFLOAT16;
}

bool IsPortZeroData(const std::string& input) {
  if (input.empty() || input[0] == '^') return false;
  const size_t colon = input.find(':');
  return colon == std::string::npos || input.substr(colon) == ":0";
}

int DataInputCount(const NodeDef& n) {
  int c = 0;
  for (const auto& in : n.input) c += (!in.empty() && in[0] != '^') ? 1 : 0;
  return c;
}

void AppendControlInputs(const NodeDef& from, NodeDef* to) {
  for (const auto& in : from.input) {
    if (!in.empty() && in[0] == '^' && !U::HasInput(*to, in)) to->input.push_back(in);
  }
}

// data_format of a BiasAddGrad node; the op's default when absent or empty.
std::string DataFormat(const NodeDef& n) {
  const auto it = n.attr.find("data_format");
  std::string f;
  if (it == n.attr.end() || !it->second.GetString(&f) || f.empty()) return "NHWC";
  return f;
}

// Every reader of output 0 of `old_name` reads `new_tensor` instead; control
// edges on `old_name` move to the producer of `new_tensor`.
void RedirectOutputZero(GraphDef* graph, const std::string& old_name,
                        const std::string& new_tensor) {
  const std::string new_node = U::GetProducerNodeName(new_tensor);
  for (auto& node : graph->node) {
    if (node.name == old_name) continue;
    for (auto& in : node.input) {
      if (in.empty() || U::GetProducerNodeName(in) != old_name) continue;
      if (in[0] == '^') {
        in = "^" + new_node;
      } else if (IsPortZeroData(in)) {
        in = new_tensor;
      }
    }
  }
}

class MusaBiasAddReluGradFusion : public FusionPattern {
 public:
  FusionMatchResult Match(const GraphDef& graph, int idx) const override {
    FusionMatchResult r;
    if (idx < 0 || idx >= graph.node_size()) return r;
    const NodeDef& bias_grad = graph.node[idx];
    if (bias_grad.op != "BiasAddGrad" || !U::IsMusaNode(bias_grad)) return r;
    if (U::EndsWith(bias_grad.name, "_original")) return r;
    const int dt = bias_grad.AttrType("T");
    if (!IsFloatLike(dt) || DataInputCount(bias_grad) != 1) return r;
    if (bias_grad.input.empty() || !IsPortZeroData(bias_grad.input[0])) return r;
    const std::string f = DataFormat(bias_grad);
    if (f != "NHWC" && f != "NCHW") return r;
    // A BiasAddGrad that nothing reads may be fetched by name: leave it.
    if (!U::HasAnyConsumer(graph, bias_grad.name)) return r;
    const NodeDef* relu_grad = U::FindProducer(graph, bias_grad.input[0]);
    if (relu_grad == nullptr || relu_grad->op != "ReluGrad") return r;
    if (!U::IsMusaNode(*relu_grad) || relu_grad->AttrType("T") != dt) return r;
    if (U::EndsWith(relu_grad->name, "_original")) return r;
    if (DataInputCount(*relu_grad) != 2 || relu_grad->input.size() < 2) return r;
    if (relu_grad->input[0][0] == '^' || relu_grad->input[1][0] == '^') return r;
    // Two devices would need a copy of dz in between.
    if (relu_grad->device != bias_grad.device) return r;
    r.matched = true;
    r.matched_nodes = {bias_grad.name, relu_grad->name};
    r.captured_nodes["bias_add_grad"] = bias_grad.name;
    r.captured_nodes["relu_grad"] = relu_grad->name;
    r.captured_attrs["T"] = DataTypeString(dt);
    return r;
  }

  Status Apply(GraphDef* graph, const FusionMatchResult& m) const override {
    if (!m.IsValid()) return Status::InvalidArgument("invalid " + GetName() + " match");
    if (!IsKernelAvailable()) return Status::OK();  // fallback: leave the pair
    const auto bg = m.captured_nodes.find("bias_add_grad");
    const auto rg = m.captured_nodes.find("relu_grad");
    if (bg == m.captured_nodes.end() || rg == m.captured_nodes.end()) {
      return Status::InvalidArgument("missing captured nodes in " + GetName());
    }
    const int bg_idx = U::FindNodeIndex(*graph, bg->second);
    const int rg_idx = U::FindNodeIndex(*graph, rg->second);
    if (bg_idx < 0) return Status::NotFound("BiasAddGrad vanished: " + bg->second);
    if (rg_idx < 0) return Status::NotFound("ReluGrad vanished: " + rg->second);
    if (graph->node[rg_idx].op == kFusedOp) return Status::OK();  // already done

    const NodeDef& bias_grad = graph->node[bg_idx];
    const NodeDef& relu_grad = graph->node[rg_idx];
    NodeDef fused;
    fused.name = relu_grad.name;
    fused.op = kFusedOp;
    fused.device = relu_grad.device;
    fused.input.push_back(relu_grad.input[0]);
    fused.input.push_back(relu_grad.input[1]);
    AppendControlInputs(relu_grad, &fused);
    AppendControlInputs(bias_grad, &fused);
    const auto t_it = relu_grad.attr.find("T");
    fused.attr["T"] = t_it != relu_grad.attr.end()
                          ? t_it->second
                          : AttrValue::Type(relu_grad.AttrType("T"));
    fused.attr["data_format"] = AttrValue::String(DataFormat(bias_grad));

    const std::string fused_name = fused.name;
    const std::string bias_grad_name = bias_grad.name;
    const std::string renamed = fused_name + "_original";
    std::unordered_set<std::string> keep = {
        fused_name, U::GetProducerNodeName(fused.input[0]),
        U::GetProducerNodeName(fused.input[1])};
    // The old ReluGrad steps aside; its readers now see the fused node, which
    // carries its name and the same value on output 0.
    graph->node[rg_idx].name = renamed;
    graph->node.push_back(std::move(fused));
    RedirectOutputZero(graph, bias_grad_name, fused_name + ":1");
    U::RemoveNodesIfUnused(graph, {bias_grad_name, renamed}, keep);
    return Status::OK();
  }

  int GetPriority() const override { return 53; }
  bool IsKernelAvailable() const override {
    return !U::IsTruthyEnvVar(kKillSwitch) &&
           FusionKernelRegistry::GetInstance().IsKernelAvailable(GetName());
  }
  std::string GetName() const override { return "MusaBiasAddReluGradFusion"; }
  std::string GetFallbackReason() const override {
    return std::string("disabled by ") + kKillSwitch + " or kernel not registered";
  }
};

}  // namespace

REGISTER_FUSION_PATTERN(MusaBiasAddReluGradFusion);
REGISTER_FUSION_KERNEL(MusaBiasAddReluGradFusion, []() { return true; });

// Keeps this translation unit (and its static registrar) in the link.
void LinkBiasAddReluGradFusion() {}

}  // namespace musa_graph
