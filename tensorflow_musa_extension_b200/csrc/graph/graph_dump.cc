// GraphDef dumping around the fusion pass, and the process-wide runtime
// switches that the reference exports next to it.
//
// Configuration: a programmatic override (TFMusaSetGraphDumpConfig) or, without
// one, the environment (MUSA_DUMP_GRAPHDEF, MUSA_DUMP_GRAPHDEF_DIR,
// MUSA_DUMP_GRAPHDEF_TEXT, MUSA_DUMP_GRAPHDEF_SLIM), as in
// musa_ext/mu/optimizer/graph_utils.cc:67-131, :425-500, :552-589.  Files are
// named <dir>/<optimizer>_<id:04>_<stage>.pb (:133-141, :507-524).  The
// binary dump is the GraphDef's wire bytes, unknown fields included.  The
// .pbtxt companion lists name / op / input / device and the scalar attrs of
// every node (the codec keeps other attr kinds as opaque bytes); the .slim.pb
// companion drops every attr that is not a scalar (tensor payloads, shapes,
// lists) and the fields the codec does not decode.
#include "graph_dump.h"

#include <sys/stat.h>

#include <atomic>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <mutex>
#include <sstream>

#include "../../../include/musa_plugin_graph.h"

namespace musa_graph {
namespace {

struct DumpConfig {
  bool has_override = false;
  bool enabled = false;
  bool dump_text = false;
  bool dump_slim = false;
  std::string dump_dir = ".";
};

std::mutex& ConfigMutex() {
  static std::mutex* mu = new std::mutex;
  return *mu;
}
DumpConfig& Config() {
  static DumpConfig* c = new DumpConfig;
  return *c;
}

bool EnvFlag(const char* name) {
  const char* v = std::getenv(name);
  if (v == nullptr) return false;
  const std::string s(v);
  return s == "1" || s == "true" || s == "TRUE" || s == "yes";
}

std::atomic<int> g_dump_counter{0};
std::atomic<bool> g_allow_growth{false};

std::string Escape(const std::string& s) {
  std::string out;
  for (unsigned char ch : s) {
    if (ch == '"' || ch == '\\') {
      out.push_back('\\');
      out.push_back(static_cast<char>(ch));
    } else if (ch < 0x20 || ch >= 0x7f) {
      char buf[8];
      std::snprintf(buf, sizeof(buf), "\\%03o", ch);
      out += buf;
    } else {
      out.push_back(static_cast<char>(ch));
    }
  }
  return out;
}

// Enumerator of tensorflow.DataType as text format spells it; the number for
// a value outside the types this path knows.
std::string EnumName(int dt) {
  switch (dt) {
    case DT_FLOAT: return "DT_FLOAT";
    case DT_DOUBLE: return "DT_DOUBLE";
    case DT_INT32: return "DT_INT32";
    case DT_INT64: return "DT_INT64";
    case DT_BFLOAT16: return "DT_BFLOAT16";
    case DT_HALF: return "DT_HALF";
    default: return std::to_string(dt);
  }
}

// Scalar attr -> text-format body ("type: DT_FLOAT", "s: \"NHWC\"", ...);
// false for the kinds the codec keeps opaque.
bool ScalarAttrText(const AttrValue& v, std::string* out) {
  int dt = 0;
  bool b = false;
  std::string s;
  float f = 0.0f;
  int64_t i = 0;
  std::ostringstream os;
  if (v.GetType(&dt)) {
    os << "type: " << EnumName(dt);
  } else if (v.GetString(&s)) {
    os << "s: \"" << Escape(s) << "\"";
  } else if (v.GetBool(&b)) {
    os << "b: " << (b ? "true" : "false");
  } else if (v.GetInt(&i)) {
    os << "i: " << i;
  } else if (v.GetFloat(&f)) {
    os << "f: " << f;
  } else {
    return false;
  }
  *out = os.str();
  return true;
}

bool WriteFile(const std::string& path, const std::string& bytes) {
  std::ofstream f(path, std::ios::out | std::ios::trunc | std::ios::binary);
  if (!f.is_open()) return false;
  f.write(bytes.data(), static_cast<std::streamsize>(bytes.size()));
  return f.good();
}

}  // namespace

bool IsGraphDefDumpingEnabled() {
  {
    std::lock_guard<std::mutex> l(ConfigMutex());
    if (Config().has_override) return Config().enabled;
  }
  return EnvFlag("MUSA_DUMP_GRAPHDEF");
}

std::string GetDumpDirectory() {
  {
    std::lock_guard<std::mutex> l(ConfigMutex());
    if (Config().has_override) return Config().dump_dir.empty() ? "." : Config().dump_dir;
  }
  const char* d = std::getenv("MUSA_DUMP_GRAPHDEF_DIR");
  return (d != nullptr && d[0] != '\0') ? std::string(d) : std::string(".");
}

bool IsGraphDefTextDumpEnabled() {
  {
    std::lock_guard<std::mutex> l(ConfigMutex());
    if (Config().has_override) return Config().dump_text;
  }
  return EnvFlag("MUSA_DUMP_GRAPHDEF_TEXT");
}

bool IsSlimGraphDefDumpEnabled() {
  {
    std::lock_guard<std::mutex> l(ConfigMutex());
    if (Config().has_override) return Config().dump_slim;
  }
  return EnvFlag("MUSA_DUMP_GRAPHDEF_SLIM");
}

std::string GraphDefToText(const GraphDef& graph) {
  std::ostringstream os;
  for (const NodeDef& n : graph.node) {
    os << "node {\n  name: \"" << Escape(n.name) << "\"\n  op: \"" << Escape(n.op) << "\"\n";
    for (const auto& in : n.input) os << "  input: \"" << Escape(in) << "\"\n";
    if (!n.device.empty()) os << "  device: \"" << Escape(n.device) << "\"\n";
    for (const auto& kv : n.attr) {
      std::string body;
      if (!ScalarAttrText(kv.second, &body)) continue;
      os << "  attr {\n    key: \"" << Escape(kv.first) << "\"\n    value {\n      " << body
         << "\n    }\n  }\n";
    }
    os << "}\n";
  }
  return os.str();
}

GraphDef SlimGraphDef(const GraphDef& graph) {
  GraphDef slim;
  slim.node.reserve(graph.node.size());
  for (const NodeDef& n : graph.node) {
    NodeDef s;
    s.name = n.name;
    s.op = n.op;
    s.input = n.input;
    s.device = n.device;
    for (const auto& kv : n.attr) {
      std::string unused;
      if (ScalarAttrText(kv.second, &unused)) s.attr[kv.first] = kv.second;
    }
    slim.node.push_back(std::move(s));
  }
  return slim;
}

GraphDefDumper::GraphDefDumper(const std::string& optimizer_name)
    : optimizer_name_(optimizer_name), dump_id_(++g_dump_counter) {}

bool GraphDefDumper::DumpAtStage(const GraphDef& graph, const std::string& stage) {
  if (!IsGraphDefDumpingEnabled()) return true;
  const std::string dir = GetDumpDirectory();
  struct stat st;
  if (stat(dir.c_str(), &st) != 0) {
    if (mkdir(dir.c_str(), 0755) != 0 && stat(dir.c_str(), &st) != 0) return false;
  }
  char id[16];
  std::snprintf(id, sizeof(id), "%04d", dump_id_);
  std::string base = dir + "/" + optimizer_name_ + "_" + id;
  if (!stage.empty()) base += "_" + stage;
  // A failed dump never fails the optimisation.
  bool ok = WriteFile(base + ".pb", graph.SerializeAsString());
  if (IsSlimGraphDefDumpEnabled()) {
    ok = WriteFile(base + ".slim.pb", SlimGraphDef(graph).SerializeAsString()) && ok;
  }
  if (IsGraphDefTextDumpEnabled()) {
    ok = WriteFile(base + ".pbtxt", GraphDefToText(graph)) && ok;
  }
  return ok;
}

bool GetAllowGrowth() {
  // TF_FORCE_GPU_ALLOW_GROWTH wins when it parses ("true" / "false"), as in
  // musa_ext/mu/device_register.cc:38-67.
  const char* v = std::getenv("TF_FORCE_GPU_ALLOW_GROWTH");
  if (v != nullptr) {
    if (std::strcmp(v, "true") == 0) return true;
    if (std::strcmp(v, "false") == 0) return false;
  }
  return g_allow_growth.load();
}

void SetAllowGrowth(bool enabled) { g_allow_growth.store(enabled); }

}  // namespace musa_graph

extern "C" {

void TFMusaSetGraphDumpConfig(int enabled, const char* dump_dir, int dump_text,
                              int dump_slim) {
  std::lock_guard<std::mutex> l(musa_graph::ConfigMutex());
  auto& c = musa_graph::Config();
  c.has_override = true;
  c.enabled = enabled != 0;
  c.dump_text = dump_text != 0;
  c.dump_slim = dump_slim != 0;
  c.dump_dir = (dump_dir != nullptr && dump_dir[0] != '\0') ? dump_dir : ".";
}

void TFMusaClearGraphDumpConfig(void) {
  std::lock_guard<std::mutex> l(musa_graph::ConfigMutex());
  musa_graph::Config() = musa_graph::DumpConfig();
}

int TFMusaGraphDumpIsEnabled(void) { return musa_graph::IsGraphDefDumpingEnabled() ? 1 : 0; }

const char* TFMusaGetGraphDumpDirectory(void) {
  static thread_local std::string dir;
  dir = musa_graph::GetDumpDirectory();
  return dir.c_str();
}

int TFMusaGraphDumpTextIsEnabled(void) {
  return musa_graph::IsGraphDefTextDumpEnabled() ? 1 : 0;
}

int TFMusaGraphDumpSlimIsEnabled(void) {
  return musa_graph::IsSlimGraphDefDumpEnabled() ? 1 : 0;
}

void TFMusaSetAllowGrowth(int enabled) { musa_graph::SetAllowGrowth(enabled != 0); }

int TFMusaGetAllowGrowth(void) { return musa_graph::GetAllowGrowth() ? 1 : 0; }

}  // extern "C"
