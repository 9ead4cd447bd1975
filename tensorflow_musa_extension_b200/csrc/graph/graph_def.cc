#include "graph_def.h"

#include <cstring>

namespace musa_graph {
namespace {

// ---- protobuf wire primitives (varint, 64-bit, length-delimited, 32-bit) ---
struct Reader {
  const uint8_t* p;
  const uint8_t* end;
  bool ok = true;

  bool done() const { return p >= end; }

  uint64_t Varint() {
    uint64_t v = 0;
    int shift = 0;
    while (p < end && shift < 64) {
      const uint8_t b = *p++;
      v |= static_cast<uint64_t>(b & 0x7f) << shift;
      if ((b & 0x80) == 0) return v;
      shift += 7;
    }
    ok = false;
    return 0;
  }

  // Reads one field; `payload` covers the value bytes (for LEN: the content).
  // `whole` covers tag + value, for verbatim re-emission.
  bool Field(uint32_t* number, int* wire_type, const uint8_t** payload,
             size_t* payload_size, const uint8_t** whole, size_t* whole_size) {
    const uint8_t* start = p;
    const uint64_t tag = Varint();
    if (!ok) return false;
    *number = static_cast<uint32_t>(tag >> 3);
    *wire_type = static_cast<int>(tag & 7);
    if (*number == 0) return ok = false;
    switch (*wire_type) {
      case 0: {
        *payload = p;
        Varint();
        *payload_size = static_cast<size_t>(p - *payload);
        break;
      }
      case 1:
        if (end - p < 8) return ok = false;
        *payload = p;
        *payload_size = 8;
        p += 8;
        break;
      case 2: {
        const uint64_t n = Varint();
        if (!ok || n > static_cast<uint64_t>(end - p)) return ok = false;
        *payload = p;
        *payload_size = static_cast<size_t>(n);
        p += n;
        break;
      }
      case 5:
        if (end - p < 4) return ok = false;
        *payload = p;
        *payload_size = 4;
        p += 4;
        break;
      default:  // groups are not used by these messages
        return ok = false;
    }
    *whole = start;
    *whole_size = static_cast<size_t>(p - start);
    return ok;
  }
};

void PutVarint(std::string* out, uint64_t v) {
  while (v >= 0x80) {
    out->push_back(static_cast<char>((v & 0x7f) | 0x80));
    v >>= 7;
  }
  out->push_back(static_cast<char>(v));
}

void PutTag(std::string* out, uint32_t number, int wire_type) {
  PutVarint(out, (static_cast<uint64_t>(number) << 3) | wire_type);
}

void PutBytes(std::string* out, uint32_t number, const std::string& s) {
  PutTag(out, number, 2);
  PutVarint(out, s.size());
  out->append(s);
}

uint64_t DecodeVarint(const uint8_t* p, size_t n) {
  Reader r{p, p + n};
  return r.Varint();
}

bool ParseNode(const uint8_t* data, size_t size, NodeDef* node) {
  Reader r{data, data + size};
  while (!r.done()) {
    uint32_t num;
    int wt;
    const uint8_t *payload, *whole;
    size_t psize, wsize;
    if (!r.Field(&num, &wt, &payload, &psize, &whole, &wsize)) return false;
    const char* text = reinterpret_cast<const char*>(payload);
    if (num == 1 && wt == 2) {
      node->name.assign(text, psize);
    } else if (num == 2 && wt == 2) {
      node->op.assign(text, psize);
    } else if (num == 3 && wt == 2) {
      node->input.emplace_back(text, psize);
    } else if (num == 4 && wt == 2) {
      node->device.assign(text, psize);
    } else if (num == 5 && wt == 2) {
      // map<string, AttrValue> entry: key = 1, value = 2
      Reader e{payload, payload + psize};
      std::string key, value;
      while (!e.done()) {
        uint32_t en;
        int ew;
        const uint8_t *ep, *ewh;
        size_t eps, ews;
        if (!e.Field(&en, &ew, &ep, &eps, &ewh, &ews)) return false;
        if (en == 1 && ew == 2) key.assign(reinterpret_cast<const char*>(ep), eps);
        if (en == 2 && ew == 2) value.assign(reinterpret_cast<const char*>(ep), eps);
      }
      node->attr[key] = AttrValue::FromBytes(std::move(value));
    } else {
      node->other_fields.append(reinterpret_cast<const char*>(whole), wsize);
    }
  }
  return r.ok;
}

std::string SerializeNode(const NodeDef& node) {
  std::string out;
  if (!node.name.empty()) PutBytes(&out, 1, node.name);
  if (!node.op.empty()) PutBytes(&out, 2, node.op);
  for (const auto& in : node.input) PutBytes(&out, 3, in);
  if (!node.device.empty()) PutBytes(&out, 4, node.device);
  for (const auto& kv : node.attr) {
    std::string entry;
    PutBytes(&entry, 1, kv.first);
    PutBytes(&entry, 2, kv.second.bytes());
    PutBytes(&out, 5, entry);
  }
  out.append(node.other_fields);
  return out;
}

// Finds the LAST occurrence of a scalar member of AttrValue's oneof (protobuf
// semantics: the last one on the wire wins).
bool FindAttrField(const std::string& bytes, uint32_t want, int want_wt,
                   const uint8_t** payload, size_t* size) {
  Reader r{reinterpret_cast<const uint8_t*>(bytes.data()),
           reinterpret_cast<const uint8_t*>(bytes.data()) + bytes.size()};
  bool found = false;
  while (!r.done()) {
    uint32_t num;
    int wt;
    const uint8_t *p, *w;
    size_t ps, ws;
    if (!r.Field(&num, &wt, &p, &ps, &w, &ws)) return false;
    if (num == want && wt == want_wt) {
      *payload = p;
      *size = ps;
      found = true;
    }
  }
  return found;
}

}  // namespace

const char* DataTypeString(int dt) {
  switch (dt) {
    case DT_FLOAT: return "float";
    case DT_DOUBLE: return "double";
    case DT_INT32: return "int32";
    case DT_INT64: return "int64";
    case DT_BFLOAT16: return "bfloat16";
    case DT_HALF: return "half";
    default: return "invalid";
  }
}

AttrValue AttrValue::FromBytes(std::string bytes) {
  AttrValue a;
  a.bytes_ = std::move(bytes);
  return a;
}
AttrValue AttrValue::Type(int dt) {
  AttrValue a;
  PutTag(&a.bytes_, 6, 0);
  PutVarint(&a.bytes_, static_cast<uint64_t>(dt));
  return a;
}
AttrValue AttrValue::Bool(bool b) {
  AttrValue a;
  PutTag(&a.bytes_, 5, 0);
  PutVarint(&a.bytes_, b ? 1 : 0);
  return a;
}
AttrValue AttrValue::String(const std::string& s) {
  AttrValue a;
  PutBytes(&a.bytes_, 2, s);
  return a;
}
AttrValue AttrValue::Float(float f) {
  AttrValue a;
  PutTag(&a.bytes_, 4, 5);
  char raw[4];
  std::memcpy(raw, &f, 4);
  a.bytes_.append(raw, 4);
  return a;
}
AttrValue AttrValue::Int(int64_t i) {
  AttrValue a;
  PutTag(&a.bytes_, 3, 0);
  PutVarint(&a.bytes_, static_cast<uint64_t>(i));
  return a;
}

bool AttrValue::GetType(int* dt) const {
  const uint8_t* p;
  size_t n;
  if (!FindAttrField(bytes_, 6, 0, &p, &n)) return false;
  *dt = static_cast<int>(DecodeVarint(p, n));
  return true;
}
bool AttrValue::GetBool(bool* b) const {
  const uint8_t* p;
  size_t n;
  if (!FindAttrField(bytes_, 5, 0, &p, &n)) return false;
  *b = DecodeVarint(p, n) != 0;
  return true;
}
bool AttrValue::GetString(std::string* s) const {
  const uint8_t* p;
  size_t n;
  if (!FindAttrField(bytes_, 2, 2, &p, &n)) return false;
  s->assign(reinterpret_cast<const char*>(p), n);
  return true;
}
bool AttrValue::GetFloat(float* f) const {
  const uint8_t* p;
  size_t n;
  if (!FindAttrField(bytes_, 4, 5, &p, &n)) return false;
  std::memcpy(f, p, 4);
  return true;
}
bool AttrValue::GetInt(int64_t* i) const {
  const uint8_t* p;
  size_t n;
  if (!FindAttrField(bytes_, 3, 0, &p, &n)) return false;
  *i = static_cast<int64_t>(DecodeVarint(p, n));
  return true;
}
int AttrValue::type_or_invalid() const {
  int dt = DT_INVALID;
  GetType(&dt);
  return dt;
}

int NodeDef::AttrType(const std::string& key) const {
  const auto it = attr.find(key);
  return it == attr.end() ? DT_INVALID : it->second.type_or_invalid();
}

bool GraphDef::ParseFromArray(const void* data, size_t size) {
  node.clear();
  other_fields.clear();
  const uint8_t* bytes = static_cast<const uint8_t*>(data);
  Reader r{bytes, bytes + size};
  while (!r.done()) {
    uint32_t num;
    int wt;
    const uint8_t *payload, *whole;
    size_t psize, wsize;
    if (!r.Field(&num, &wt, &payload, &psize, &whole, &wsize)) {
      node.clear();
      other_fields.clear();
      return false;
    }
    if (num == 1 && wt == 2) {
      NodeDef n;
      if (!ParseNode(payload, psize, &n)) {
        node.clear();
        other_fields.clear();
        return false;
      }
      node.push_back(std::move(n));
    } else {
      other_fields.append(reinterpret_cast<const char*>(whole), wsize);
    }
  }
  return true;
}

std::string GraphDef::SerializeAsString() const {
  std::string out;
  for (const auto& n : node) PutBytes(&out, 1, SerializeNode(n));
  out.append(other_fields);
  return out;
}

}  // namespace musa_graph
