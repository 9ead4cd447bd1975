// A TensorFlow GraphDef as the graph optimizer sees it, read from and written
// to the protobuf wire format without TensorFlow or protobuf headers.
//
// Only what the fusion patterns touch is decoded: GraphDef.node (field 1) and,
// per NodeDef, name (1), op (2), input (3), device (4) and the attr map (5).
// Every other field (versions, function library, debug info, full types, and
// the inside of each AttrValue) is carried through byte for byte, so a graph
// that no pattern matches serialises to an equivalent message.
//
// This stands where the reference uses tensorflow::GraphDef / NodeDef /
// AttrValue (e.g. musa_ext/graph/fusion/fusion_pattern_manager.h:54-66).
#pragma once

#include <cstdint>
#include <map>
#include <string>
#include <vector>

namespace musa_graph {

// tensorflow::DataType values used on this path (types.proto).
enum DataType : int {
  DT_INVALID = 0,
  DT_FLOAT = 1,
  DT_DOUBLE = 2,
  DT_INT32 = 3,
  DT_INT64 = 9,
  DT_BFLOAT16 = 14,
  DT_HALF = 19,
};

const char* DataTypeString(int dt);

// One AttrValue, kept in serialised form.  The accessors decode the scalar
// members of its `value` oneof: s (2), i (3), f (4), b (5), type (6).
class AttrValue {
 public:
  AttrValue() = default;
  static AttrValue FromBytes(std::string bytes);
  static AttrValue Type(int dt);
  static AttrValue Bool(bool b);
  static AttrValue String(const std::string& s);
  static AttrValue Float(float f);
  static AttrValue Int(int64_t i);

  bool GetType(int* dt) const;
  bool GetBool(bool* b) const;
  bool GetString(std::string* s) const;
  bool GetFloat(float* f) const;
  bool GetInt(int64_t* i) const;
  int type_or_invalid() const;

  const std::string& bytes() const { return bytes_; }
  bool operator==(const AttrValue& o) const { return bytes_ == o.bytes_; }

 private:
  std::string bytes_;
};

struct NodeDef {
  std::string name;
  std::string op;
  std::vector<std::string> input;
  std::string device;
  std::map<std::string, AttrValue> attr;
  std::string other_fields;  // undecoded fields, re-emitted verbatim

  int AttrType(const std::string& key) const;  // DT_INVALID when absent
};

struct GraphDef {
  std::vector<NodeDef> node;
  std::string other_fields;  // versions, library, ...

  // False on malformed input; the graph is left empty in that case.
  bool ParseFromArray(const void* data, size_t size);
  std::string SerializeAsString() const;
  int node_size() const { return static_cast<int>(node.size()); }
};

}  // namespace musa_graph
