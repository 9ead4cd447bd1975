// Graph patterns that fold a BiasAdd and the activation after it into one op:
//   Relu(BiasAdd(x, b))               -> MusaBiasAddRelu(x, b)
//   Mul(x, Sigmoid(BiasAdd(x, b)))    -> MusaBiasAddSwish(x, b)
//   Sigmoid(BiasAdd(x, b))            -> MusaBiasAddSigmoid(x, b)
// New patterns plugged into the reference's registry: the reference fuses
// BiasAdd + activation only behind a MatMul
// (musa_ext/graph/fusion/linear_activation_fusion.cc:100-117) and runs a
// stand-alone BiasAdd -> Relu as two full passes over the tensor.  They follow
// that file's protocol (:42-47, :164-251): match from the last node, never from
// a "*_original" node, rename the matched output to "<name>_original", add the
// fused node under the original name and device, copy T, and remove the old
// nodes only when nothing else reads them.
//
// A chain is fused only if its intermediate results have no other reader:
// otherwise the BiasAdd would have to stay and the tensor would be read twice.
#include <unordered_set>

#include "fusion_pattern_manager.h"

namespace musa_graph {
namespace {

using U = FusionGraphUtils;

constexpr char kKillSwitch[] = "MUSA_DISABLE_BIASADD_ACT_FUSION";

bool IsFloatLike(int dt) {
  return dt == DT_FLOAT || dt == DT_HALF || dt == DT_BFLOAT16;
}

bool IsBiasAdd(const NodeDef& n) { return n.op == "BiasAdd" || n.op == "BiasAddV1"; }

// A data input that names output 0 of its producer ("name" or "name:0").
bool IsPortZeroData(const std::string& input) {
  if (input.empty() || input[0] == '^') return false;
  const size_t colon = input.find(':');
  return colon == std::string::npos || input.substr(colon) == ":0";
}

// "name:0" and "name" denote the same tensor.
std::string CanonicalTensor(const std::string& input) {
  const size_t colon = input.find(':');
  if (colon != std::string::npos && input.substr(colon) == ":0") {
    return input.substr(0, colon);
  }
  return input;
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

// The BiasAdd feeding `consumer` through `input`, if it is fusable: on the
// MUSA device, of the same float-like T, with two data inputs, and read by
// nobody but `consumer`.
const NodeDef* FusableBiasAdd(const GraphDef& graph, const NodeDef& consumer,
                              const std::string& input, int dt) {
  if (!IsPortZeroData(input)) return nullptr;
  const NodeDef* bias_add = U::FindProducer(graph, input);
  if (bias_add == nullptr || !IsBiasAdd(*bias_add)) return nullptr;
  if (!U::IsMusaNode(*bias_add) || bias_add->AttrType("T") != dt) return nullptr;
  if (DataInputCount(*bias_add) != 2 || bias_add->input.size() < 2) return nullptr;
  if (bias_add->input[0][0] == '^' || bias_add->input[1][0] == '^') return nullptr;
  if (U::CountConsumers(graph, bias_add->name, {consumer.name}) != 0) return nullptr;
  return bias_add;
}

// Replaces the node `out_name` by a fused node with the given op and inputs.
Status ReplaceChain(GraphDef* graph, const std::string& out_name,
                    const std::string& fused_op,
                    const std::vector<std::string>& chain,  // last .. first
                    const std::string& bias_add_name) {
  const int out_idx = U::FindNodeIndex(*graph, out_name);
  if (out_idx < 0) return Status::NotFound("output node vanished: " + out_name);
  if (graph->node[out_idx].op == fused_op) return Status::OK();  // already done
  const int bias_idx = U::FindNodeIndex(*graph, bias_add_name);
  if (bias_idx < 0) return Status::NotFound("BiasAdd vanished: " + bias_add_name);

  NodeDef fused;
  fused.name = out_name;
  fused.op = fused_op;
  fused.device = graph->node[out_idx].device;
  const NodeDef& bias_add = graph->node[bias_idx];
  fused.input.push_back(bias_add.input[0]);
  fused.input.push_back(bias_add.input[1]);
  for (const auto& name : chain) {
    const NodeDef* n = U::GetNodeByName(*graph, name);
    if (n != nullptr) AppendControlInputs(*n, &fused);
  }
  const auto t_it = graph->node[out_idx].attr.find("T");
  fused.attr["T"] = t_it != graph->node[out_idx].attr.end()
                        ? t_it->second
                        : AttrValue::Type(bias_add.AttrType("T"));
  const auto fmt = bias_add.attr.find("data_format");
  fused.attr["data_format"] =
      fmt != bias_add.attr.end() ? fmt->second : AttrValue::String("NHWC");

  std::unordered_set<std::string> keep = {
      out_name, U::GetProducerNodeName(bias_add.input[0]),
      U::GetProducerNodeName(bias_add.input[1])};
  const std::string renamed = out_name + "_original";
  graph->node[out_idx].name = renamed;
  graph->node.push_back(std::move(fused));

  std::vector<std::string> removable = {renamed};
  for (size_t i = 1; i < chain.size(); ++i) removable.push_back(chain[i]);
  U::RemoveNodesIfUnused(graph, removable, keep);
  return Status::OK();
}

class BiasAddUnaryFusion : public FusionPattern {
 public:
  BiasAddUnaryFusion(std::string unary_op, std::string fused_op,
                     std::string name, int priority)
      : unary_op_(std::move(unary_op)), fused_op_(std::move(fused_op)),
        name_(std::move(name)), priority_(priority) {}

  FusionMatchResult Match(const GraphDef& graph, int idx) const override {
    FusionMatchResult r;
    if (idx < 0 || idx >= graph.node_size()) return r;
    const NodeDef& act = graph.node[idx];
    if (act.op != unary_op_ || !U::IsMusaNode(act)) return r;
    if (U::EndsWith(act.name, "_original")) return r;
    const int dt = act.AttrType("T");
    if (!IsFloatLike(dt) || DataInputCount(act) != 1 || act.input.empty()) return r;
    const NodeDef* bias_add = FusableBiasAdd(graph, act, act.input[0], dt);
    if (bias_add == nullptr) return r;
    r.matched = true;
    r.matched_nodes = {act.name, bias_add->name};
    r.captured_nodes["activation"] = act.name;
    r.captured_nodes["bias_add"] = bias_add->name;
    r.captured_attrs["T"] = DataTypeString(dt);
    return r;
  }

  Status Apply(GraphDef* graph, const FusionMatchResult& m) const override {
    if (!m.IsValid()) return Status::InvalidArgument("invalid " + name_ + " match");
    if (!IsKernelAvailable()) return Status::OK();  // fallback: leave the chain
    const auto act = m.captured_nodes.find("activation");
    const auto bias = m.captured_nodes.find("bias_add");
    if (act == m.captured_nodes.end() || bias == m.captured_nodes.end()) {
      return Status::InvalidArgument("missing captured nodes in " + name_);
    }
    return ReplaceChain(graph, act->second, fused_op_, {act->second, bias->second},
                        bias->second);
  }

  int GetPriority() const override { return priority_; }
  bool IsKernelAvailable() const override {
    return !U::IsTruthyEnvVar(kKillSwitch) &&
           FusionKernelRegistry::GetInstance().IsKernelAvailable(name_);
  }
  std::string GetName() const override { return name_; }
  std::string GetFallbackReason() const override {
    return std::string("disabled by ") + kKillSwitch + " or kernel not registered";
  }

 private:
  std::string unary_op_, fused_op_, name_;
  int priority_;
};

class MusaBiasAddReluFusion : public BiasAddUnaryFusion {
 public:
  MusaBiasAddReluFusion()
      : BiasAddUnaryFusion("Relu", "MusaBiasAddRelu", "MusaBiasAddReluFusion", 55) {}
};

class MusaBiasAddSigmoidFusion : public BiasAddUnaryFusion {
 public:
  MusaBiasAddSigmoidFusion()
      : BiasAddUnaryFusion("Sigmoid", "MusaBiasAddSigmoid",
                           "MusaBiasAddSigmoidFusion", 54) {}
};

// Mul(x, Sigmoid(BiasAdd(x, b))), operands of the Mul in either order.
class MusaBiasAddSwishFusion : public FusionPattern {
 public:
  FusionMatchResult Match(const GraphDef& graph, int idx) const override {
    FusionMatchResult r;
    if (idx < 0 || idx >= graph.node_size()) return r;
    const NodeDef& mul = graph.node[idx];
    if (mul.op != "Mul" || !U::IsMusaNode(mul)) return r;
    if (U::EndsWith(mul.name, "_original")) return r;
    const int dt = mul.AttrType("T");
    if (!IsFloatLike(dt) || DataInputCount(mul) != 2 || mul.input.size() < 2) return r;
    for (int side = 0; side < 2; ++side) {
      const std::string& gate = mul.input[side];
      const std::string& x = mul.input[1 - side];
      if (!IsPortZeroData(gate) || x.empty() || x[0] == '^') continue;
      const NodeDef* sig = U::FindProducer(graph, gate);
      if (sig == nullptr || sig->op != "Sigmoid" || !U::IsMusaNode(*sig)) continue;
      if (sig->AttrType("T") != dt || DataInputCount(*sig) != 1) continue;
      if (U::CountConsumers(graph, sig->name, {mul.name}) != 0) continue;
      const NodeDef* bias_add = FusableBiasAdd(graph, *sig, sig->input[0], dt);
      if (bias_add == nullptr) continue;
      // The gate must be computed from the very tensor it multiplies.
      if (CanonicalTensor(bias_add->input[0]) != CanonicalTensor(x)) continue;
      r.matched = true;
      r.matched_nodes = {mul.name, sig->name, bias_add->name};
      r.captured_nodes["mul"] = mul.name;
      r.captured_nodes["sigmoid"] = sig->name;
      r.captured_nodes["bias_add"] = bias_add->name;
      r.captured_attrs["T"] = DataTypeString(dt);
      return r;
    }
    return r;
  }

  Status Apply(GraphDef* graph, const FusionMatchResult& m) const override {
    if (!m.IsValid()) return Status::InvalidArgument("invalid swish match");
    if (!IsKernelAvailable()) return Status::OK();
    const auto mul = m.captured_nodes.find("mul");
    const auto sig = m.captured_nodes.find("sigmoid");
    const auto bias = m.captured_nodes.find("bias_add");
    if (mul == m.captured_nodes.end() || sig == m.captured_nodes.end() ||
        bias == m.captured_nodes.end()) {
      return Status::InvalidArgument("missing captured nodes in swish pattern");
    }
    return ReplaceChain(graph, mul->second, "MusaBiasAddSwish",
                        {mul->second, sig->second, bias->second}, bias->second);
  }

  int GetPriority() const override { return 56; }
  bool IsKernelAvailable() const override {
    return !U::IsTruthyEnvVar(kKillSwitch) &&
           FusionKernelRegistry::GetInstance().IsKernelAvailable(GetName());
  }
  std::string GetName() const override { return "MusaBiasAddSwishFusion"; }
  std::string GetFallbackReason() const override {
    return std::string("disabled by ") + kKillSwitch + " or kernel not registered";
  }
};

}  // namespace

REGISTER_FUSION_PATTERN(MusaBiasAddSwishFusion);
REGISTER_FUSION_KERNEL(MusaBiasAddSwishFusion, []() { return true; });
REGISTER_FUSION_PATTERN(MusaBiasAddReluFusion);
REGISTER_FUSION_KERNEL(MusaBiasAddReluFusion, []() { return true; });
REGISTER_FUSION_PATTERN(MusaBiasAddSigmoidFusion);
REGISTER_FUSION_KERNEL(MusaBiasAddSigmoidFusion, []() { return true; });

// Keeps this translation unit (and its static registrars) in the link.
void LinkBiasAddActivationFusion() {}

}  // namespace musa_graph
