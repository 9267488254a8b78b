// kq_container — reads karume's distribution format directly: one .safetensors file whose
// __metadata__.karume_ir holds the graph JSON (docs/ir-v1.md, "コンテナ"), so that an exported
// asset feeds kq_weight_upload without a TypeScript hop.
//
// Restates, check for check,
//   packages/runtime/src/format/safetensors.ts:25-50   dtype -> bits and dtype -> alignment tables
//                                                       (I4 = 4 bits per element, tensor start 4-byte aligned)
//   packages/runtime/src/format/safetensors.ts:107-160 one header entry: dtype, shape, data_offsets, exact byte size,
//                                                       an odd number of I4 elements is refused
//   packages/runtime/src/format/safetensors.ts:187-262 the data section is covered exactly: no overlap, no gap, no
//                                                       trailing bytes, every tensor start aligned
//   packages/runtime/src/format/ir.ts:268-306          storage { dtype, scale, group_size }: scale required for i8 / i4,
//                                                       group_size required for i4, a power of two >= 16, refused elsewhere
//   packages/runtime/src/format/ir.ts:617-646          i4: row length (numel / shape[0]) divisible by group_size
//   packages/runtime/src/format/container.ts:180-232   tensor exists, safetensors dtype == storage encoding, shape == declared
//   packages/runtime/src/format/container.ts:337-400   scale tensor: F32; group form [shape[0], row / g] for i4, keepdim
//                                                       broadcast form of the weight's rank for i8
//   packages/runtime/src/format/container.ts:309-320   tensors no initializer refers to are refused
// The graph itself (nodes, symbols, op contracts) stays the host's business: only `initializers` and
// `values` are read.  Everything here is host code; only kq_model_weight touches the GPU.
#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstring>
#include <map>
#include <memory>
#include <string>
#include <vector>

#include "kq_internal.h"

namespace kq {
namespace {

// ---- a small JSON reader (objects, arrays, strings, numbers, true / false / null) ----------
struct Json {
  enum Kind { kNull, kBool, kNumber, kString, kArray, kObject } kind = kNull;
  bool boolean = false;
  double number = 0.0;
  std::string text;
  std::vector<Json> items;
  std::vector<std::pair<std::string, Json>> members;  // declaration order kept

  const Json* get(const char* key) const {
    for (const auto& kv : members)
      if (kv.first == key) return &kv.second;
    return nullptr;
  }
};

struct JsonParser {
  const char* p;
  const char* end;
  std::string error;
  int depth = 0;

  bool fail(const char* what) {
    if (error.empty()) error = what;
    return false;
  }
  void skip() {
    while (p < end && (*p == ' ' || *p == '\t' || *p == '\n' || *p == '\r')) ++p;
  }
  bool parse_string(std::string* out) {
    if (p >= end || *p != '"') return fail("expected a string");
    ++p;
    out->clear();
    while (p < end && *p != '"') {
      unsigned char c = static_cast<unsigned char>(*p++);
      if (c < 0x20) return fail("control character in a string");
      if (c != '\\') {
        out->push_back(static_cast<char>(c));
        continue;
      }
      if (p >= end) return fail("unterminated escape");
      const char e = *p++;
      switch (e) {
        case '"': out->push_back('"'); break;
        case '\\': out->push_back('\\'); break;
        case '/': out->push_back('/'); break;
        case 'b': out->push_back('\b'); break;
        case 'f': out->push_back('\f'); break;
        case 'n': out->push_back('\n'); break;
        case 'r': out->push_back('\r'); break;
        case 't': out->push_back('\t'); break;
        case 'u': {
          if (end - p < 4) return fail("short \\u escape");
          unsigned code = 0;
          for (int i = 0; i < 4; ++i) {
            const char h = *p++;
            code <<= 4;
            if (h >= '0' && h <= '9') code |= static_cast<unsigned>(h - '0');
            else if (h >= 'a' && h <= 'f') code |= static_cast<unsigned>(h - 'a' + 10);
            else if (h >= 'A' && h <= 'F') code |= static_cast<unsigned>(h - 'A' + 10);
            else return fail("bad \\u escape");
          }
          // UTF-8 encode (surrogate pairs are passed through as two 3-byte sequences: names in
          // this format are ASCII and such text is only ever compared, never shown)
          if (code < 0x80) out->push_back(static_cast<char>(code));
          else if (code < 0x800) {
            out->push_back(static_cast<char>(0xC0 | (code >> 6)));
            out->push_back(static_cast<char>(0x80 | (code & 0x3F)));
          } else {
            out->push_back(static_cast<char>(0xE0 | (code >> 12)));
            out->push_back(static_cast<char>(0x80 | ((code >> 6) & 0x3F)));
            out->push_back(static_cast<char>(0x80 | (code & 0x3F)));
          }
          break;
        }
        default: return fail("unknown escape");
      }
    }
    if (p >= end) return fail("unterminated string");
    ++p;
    return true;
  }
  bool parse_value(Json* out) {
    if (++depth > 64) return fail("nesting too deep");
    skip();
    if (p >= end) return fail("unexpected end of JSON");
    bool ok = true;
    const char c = *p;
    if (c == '{') {
      ++p;
      out->kind = Json::kObject;
      skip();
      if (p < end && *p == '}') {
        ++p;
      } else {
        while (ok) {
          skip();
          std::string key;
          if (!parse_string(&key)) { ok = false; break; }
          skip();
          if (p >= end || *p != ':') { ok = fail("expected ':'"); break; }
          ++p;
          Json value;
          if (!parse_value(&value)) { ok = false; break; }
          out->members.emplace_back(std::move(key), std::move(value));
          skip();
          if (p < end && *p == ',') { ++p; continue; }
          if (p < end && *p == '}') { ++p; break; }
          ok = fail("expected ',' or '}'");
        }
      }
    } else if (c == '[') {
      ++p;
      out->kind = Json::kArray;
      skip();
      if (p < end && *p == ']') {
        ++p;
      } else {
        while (ok) {
          Json value;
          if (!parse_value(&value)) { ok = false; break; }
          out->items.push_back(std::move(value));
          skip();
          if (p < end && *p == ',') { ++p; continue; }
          if (p < end && *p == ']') { ++p; break; }
          ok = fail("expected ',' or ']'");
        }
      }
    } else if (c == '"') {
      out->kind = Json::kString;
      ok = parse_string(&out->text);
    } else if (end - p >= 4 && !strncmp(p, "true", 4)) {
      out->kind = Json::kBool; out->boolean = true; p += 4;
    } else if (end - p >= 5 && !strncmp(p, "false", 5)) {
      out->kind = Json::kBool; out->boolean = false; p += 5;
    } else if (end - p >= 4 && !strncmp(p, "null", 4)) {
      out->kind = Json::kNull; p += 4;
    } else if (c == '-' || (c >= '0' && c <= '9')) {
      // JSON numbers only: NaN / Infinity literals do not parse (docs/ir-v1.md forbids them)
      const char* q = p;
      if (*q == '-') ++q;
      if (q >= end || *q < '0' || *q > '9') return fail("malformed number");
      while (q < end && ((*q >= '0' && *q <= '9') || *q == '.' || *q == 'e' || *q == 'E' || *q == '+' || *q == '-')) ++q;
      std::string digits(p, q);
      char* stop = nullptr;
      out->number = strtod(digits.c_str(), &stop);
      if (stop == nullptr || *stop != 0) return fail("malformed number");
      out->kind = Json::kNumber;
      p = q;
    } else {
      ok = fail("unexpected character");
    }
    --depth;
    return ok;
  }
  bool parse_document(Json* out) {
    if (!parse_value(out)) return false;
    skip();
    if (p != end) return fail("trailing characters after the JSON value");
    return true;
  }
};

bool valid_utf8(const uint8_t* s, size_t n) {
  size_t i = 0;
  while (i < n) {
    const uint8_t c = s[i];
    size_t extra;
    if (c < 0x80) extra = 0;
    else if ((c >> 5) == 0x6) extra = 1;
    else if ((c >> 4) == 0xE) extra = 2;
    else if ((c >> 3) == 0x1E) extra = 3;
    else return false;
    if (extra > n - 1 - i) return false;
    for (size_t j = 1; j <= extra; ++j)
      if ((s[i + j] & 0xC0) != 0x80) return false;
    i += extra + 1;
  }
  return true;
}

// ---- safetensors ----------------------------------------------------------------------------
// dtype -> bits per element and -> required alignment of the tensor start
// (packages/runtime/src/format/safetensors.ts:25-50: two tables, because I4 packs two elements
// per byte and is bound as 32-bit words by the consumer).
struct DtypeInfo {
  const char* name;
  uint32_t bits;
  uint32_t align;
};
constexpr DtypeInfo kDtypes[] = {
    {"F32", 32, 4}, {"F16", 16, 2}, {"BF16", 16, 2}, {"I8", 8, 1}, {"I4", 4, 4},
    {"U8", 8, 1},   {"I32", 32, 4}, {"U32", 32, 4},  {"I64", 64, 8}, {"BOOL", 8, 1},
};
const DtypeInfo* find_dtype(const std::string& name) {
  for (const DtypeInfo& d : kDtypes)
    if (name == d.name) return &d;
  return nullptr;
}

struct TensorView {
  std::string name;
  const DtypeInfo* dtype = nullptr;
  std::vector<uint64_t> shape;
  uint64_t begin = 0, end = 0;  // relative to the data section
  uint64_t offset = 0;          // absolute, from the start of the file
  bool referenced = false;
};

constexpr double kMaxSafeInteger = 9007199254740991.0;  // Number.MAX_SAFE_INTEGER

bool as_index(const Json& v, uint64_t* out) {  // a non-negative safe integer
  if (v.kind != Json::kNumber || !(v.number >= 0.0) || v.number > kMaxSafeInteger || std::floor(v.number) != v.number)
    return false;
  *out = static_cast<uint64_t>(v.number);
  return true;
}

struct Initializer {
  std::string name, tensor, scale_key;
  std::string storage;  // "f32" | "f16" | "bf16" | "i8" | "i4" | "i32"
  uint64_t group_size = 0;
  std::vector<uint64_t> shape;  // declared in values{}
};

struct Model {
  std::vector<uint8_t> owned;  // the file, when opened by path
  const uint8_t* bytes = nullptr;
  uint64_t size = 0;
  std::map<std::string, TensorView> tensors;
  std::map<std::string, std::string> metadata;
  std::vector<Initializer> initializers;
  std::vector<std::string> names;  // c_str() storage for kq_model_initializer_name
};

std::string shape_text(const std::vector<uint64_t>& shape) {
  std::string out = "[";
  for (size_t i = 0; i < shape.size(); ++i) out += (i ? "," : "") + std::to_string(shape[i]);
  return out + "]";
}

// packages/runtime/src/format/safetensors.ts:187-262 (parseSafetensors)
bool parse_safetensors(Model* m, std::string* err) {
  char buf[512];
  if (m->size < 8) {
    snprintf(buf, sizeof buf, "file too short: %llu bytes (not even a header length)", (unsigned long long)m->size);
    *err = buf;
    return false;
  }
  uint64_t header_len = 0;
  for (int i = 7; i >= 0; --i) header_len = (header_len << 8) | m->bytes[i];
  if (header_len > static_cast<uint64_t>(kMaxSafeInteger) || 8 + header_len > m->size) {
    snprintf(buf, sizeof buf, "header length %llu exceeds the file length %llu", (unsigned long long)header_len,
             (unsigned long long)m->size);
    *err = buf;
    return false;
  }
  const uint64_t data_start = 8 + header_len;
  if (!valid_utf8(m->bytes + 8, header_len)) {
    *err = "header is not valid UTF-8";
    return false;
  }
  Json header;
  JsonParser parser{reinterpret_cast<const char*>(m->bytes + 8), reinterpret_cast<const char*>(m->bytes + 8 + header_len), "", 0};
  if (!parser.parse_document(&header)) {
    *err = "header JSON does not parse: " + parser.error;
    return false;
  }
  if (header.kind != Json::kObject) {
    *err = "header JSON is not an object";
    return false;
  }
  std::vector<TensorView> declared;
  for (const auto& kv : header.members) {
    if (kv.first == "__metadata__") {
      if (kv.second.kind != Json::kObject) {
        *err = "__metadata__ is not an object";
        return false;
      }
      for (const auto& md : kv.second.members) {
        if (md.second.kind != Json::kString) {
          *err = "__metadata__." + md.first + " is not a string";
          return false;
        }
        m->metadata[md.first] = md.second.text;
      }
      continue;
    }
    const std::string where = "tensor '" + kv.first + "'";
    const Json& raw = kv.second;
    if (raw.kind != Json::kObject) {
      *err = where + ": header entry is not an object";
      return false;
    }
    TensorView view;
    view.name = kv.first;
    const Json* dtype = raw.get("dtype");
    if (!dtype || dtype->kind != Json::kString || !(view.dtype = find_dtype(dtype->text))) {
      *err = where + ": unsupported dtype";
      return false;
    }
    const Json* shape = raw.get("shape");
    if (!shape || shape->kind != Json::kArray) {
      *err = where + ": shape is not an array";
      return false;
    }
    double count = 1.0;
    for (const Json& dim : shape->items) {
      uint64_t d = 0;
      if (!as_index(dim, &d)) {
        *err = where + ": a shape element is not a non-negative integer";
        return false;
      }
      view.shape.push_back(d);
      count *= static_cast<double>(d);
      if (count > kMaxSafeInteger) {
        *err = where + ": element count exceeds the safe integer range";
        return false;
      }
    }
    const Json* offsets = raw.get("data_offsets");
    if (!offsets || offsets->kind != Json::kArray) {
      *err = where + ": data_offsets is not an array";
      return false;
    }
    if (offsets->items.size() != 2) {
      *err = where + ": data_offsets needs exactly 2 elements";
      return false;
    }
    if (!as_index(offsets->items[0], &view.begin) || !as_index(offsets->items[1], &view.end)) {
      *err = where + ": data_offsets are not non-negative integers";
      return false;
    }
    if (view.end < view.begin) {
      *err = where + ": data_offsets are reversed";
      return false;
    }
    const uint64_t numel = static_cast<uint64_t>(count);
    const uint64_t bits = numel * view.dtype->bits;
    if (bits % 8 != 0) {  // an odd number of I4 elements: the tensor's length is not determined by its declaration
      snprintf(buf, sizeof buf, "%s: %s (%u bits per element) with %llu elements does not end on a byte boundary",
               where.c_str(), view.dtype->name, view.dtype->bits, (unsigned long long)numel);
      *err = buf;
      return false;
    }
    if (view.end - view.begin != bits / 8) {
      snprintf(buf, sizeof buf, "%s: size mismatch, offsets span %llu bytes, %s %s needs %llu", where.c_str(),
               (unsigned long long)(view.end - view.begin), view.dtype->name, shape_text(view.shape).c_str(),
               (unsigned long long)(bits / 8));
      *err = buf;
      return false;
    }
    declared.push_back(std::move(view));
  }
  // The declarations must cover the data section exactly: an overlap gives one byte two
  // meanings, a gap or a tail means a declaration was not read.
  std::sort(declared.begin(), declared.end(), [](const TensorView& a, const TensorView& b) {
    return a.begin != b.begin ? a.begin < b.begin : a.end < b.end;
  });
  const uint64_t data_len = m->size - data_start;
  uint64_t cursor = 0;
  for (TensorView& view : declared) {
    const std::string where = "tensor '" + view.name + "'";
    if (view.begin < cursor) {
      *err = where + ": overlaps the tensor before it";
      return false;
    }
    if (view.begin > cursor) {
      snprintf(buf, sizeof buf, "%s: unused bytes [%llu, %llu) in the data section", where.c_str(), (unsigned long long)cursor,
               (unsigned long long)view.begin);
      *err = buf;
      return false;
    }
    if (view.end > data_len) {
      *err = where + ": reaches beyond the data section";
      return false;
    }
    if ((data_start + view.begin) % view.dtype->align != 0) {
      snprintf(buf, sizeof buf, "%s: absolute offset %llu is not aligned to the %u bytes %s needs", where.c_str(),
               (unsigned long long)(data_start + view.begin), view.dtype->align, view.dtype->name);
      *err = buf;
      return false;
    }
    cursor = view.end;
    view.offset = data_start + view.begin;
    m->tensors[view.name] = view;
  }
  if (cursor != data_len) {
    snprintf(buf, sizeof buf, "%llu unused bytes at the end of the data section", (unsigned long long)(data_len - cursor));
    *err = buf;
    return false;
  }
  return true;
}

// ---- karume_ir: the initializer declarations -------------------------------------------------
// storage.dtype -> safetensors dtype (packages/runtime/src/format/container.ts:107-115)
const char* storage_encoding(const std::string& storage) {
  if (storage == "f32") return "F32";
  if (storage == "f16") return "F16";
  if (storage == "bf16") return "BF16";
  if (storage == "i8") return "I8";
  if (storage == "i4") return "I4";
  if (storage == "i32") return "I32";
  return nullptr;
}

bool is_pow2(uint64_t v) { return v && !(v & (v - 1)); }

uint64_t numel_of(const std::vector<uint64_t>& shape) {
  uint64_t n = 1;
  for (uint64_t d : shape) n *= d;
  return n;
}

bool parse_ir(Model* m, std::string* err) {
  auto md = m->metadata.find("karume_ir");
  if (md == m->metadata.end()) {
    *err = "__metadata__.karume_ir is missing (not a karume model)";
    return false;
  }
  Json ir;
  JsonParser parser{md->second.data(), md->second.data() + md->second.size(), "", 0};
  if (!parser.parse_document(&ir) || ir.kind != Json::kObject) {
    *err = "karume_ir does not parse as a JSON object: " + parser.error;
    return false;
  }
  const Json* format = ir.get("format");
  const Json* version = ir.get("version");
  if (!format || format->kind != Json::kString || format->text != "karume-ir" || !version ||
      version->kind != Json::kNumber || version->number != 1.0) {
    *err = "karume_ir: format must be \"karume-ir\" and version 1";
    return false;
  }
  const Json* inits = ir.get("initializers");
  const Json* values = ir.get("values");
  if (!inits || inits->kind != Json::kObject || !values || values->kind != Json::kObject) {
    *err = "karume_ir: initializers and values must be objects";
    return false;
  }
  for (const auto& kv : inits->members) {
    const std::string where = "initializer '" + kv.first + "'";
    Initializer init;
    init.name = kv.first;
    const Json& obj = kv.second;
    const Json* tensor = obj.kind == Json::kObject ? obj.get("tensor") : nullptr;
    const Json* storage = obj.kind == Json::kObject ? obj.get("storage") : nullptr;
    if (!tensor || tensor->kind != Json::kString || tensor->text.empty() || !storage || storage->kind != Json::kObject ||
        obj.members.size() != 2) {
      *err = where + ": needs exactly the keys tensor and storage";
      return false;
    }
    init.tensor = tensor->text;
    // packages/runtime/src/format/ir.ts:268-306 (parseStorage)
    for (const auto& sk : storage->members)
      if (sk.first != "dtype" && sk.first != "scale" && sk.first != "group_size") {
        *err = where + ".storage: unknown key '" + sk.first + "'";
        return false;
      }
    const Json* dtype = storage->get("dtype");
    if (!dtype || dtype->kind != Json::kString || !storage_encoding(dtype->text)) {
      *err = where + ".storage.dtype is not one of f32 / f16 / bf16 / i8 / i4 / i32";
      return false;
    }
    init.storage = dtype->text;
    const bool quantized = init.storage == "i8" || init.storage == "i4";
    const Json* scale = storage->get("scale");
    const Json* group = storage->get("group_size");
    if (!quantized && (scale || group)) {
      *err = where + ".storage: dtype '" + init.storage + "' cannot carry scale / group_size";
      return false;
    }
    if (quantized && !scale) {
      *err = where + ".storage: dtype '" + init.storage + "' needs scale (the key of the scale tensor)";
      return false;
    }
    if (init.storage == "i4" && !group) {
      *err = where + ".storage: dtype 'i4' needs group_size";
      return false;
    }
    if (scale) {
      if (scale->kind != Json::kString || scale->text.empty()) {
        *err = where + ".storage.scale is not a non-empty string";
        return false;
      }
      init.scale_key = scale->text;
    }
    if (group) {
      uint64_t g = 0;
      if (!as_index(*group, &g) || g < 1) {
        *err = where + ".storage.group_size is not a positive integer";
        return false;
      }
      if (init.storage == "i4" && (!is_pow2(g) || g < 16)) {
        *err = where + ".storage.group_size " + std::to_string(g) + " is not a power of two >= 16";
        return false;
      }
      if (init.storage != "i4") {  // group quantisation is stored as i4 only (container.ts:468-506)
        *err = where + ": group quantisation on storage '" + init.storage + "' is not supported (i4 only)";
        return false;
      }
      init.group_size = g;
    }
    const Json* value = values->get(kv.first.c_str());
    const Json* vshape = value && value->kind == Json::kObject ? value->get("shape") : nullptr;
    if (!vshape || vshape->kind != Json::kArray) {
      *err = where + ": no declaration in values{}";
      return false;
    }
    for (const Json& dim : vshape->items) {
      uint64_t d = 0;
      if (!as_index(dim, &d)) {  // initializers have numeric dimensions only
        *err = where + ": a declared dimension is not a non-negative integer";
        return false;
      }
      init.shape.push_back(d);
    }
    if (init.storage == "i4") {  // packages/runtime/src/format/ir.ts:617-646
      if (init.shape.empty() || init.shape[0] == 0) {
        *err = where + ": an i4 weight needs a quantisation axis";
        return false;
      }
      const uint64_t row = numel_of(init.shape) / init.shape[0];
      if (row % init.group_size != 0) {
        *err = where + ": row length " + std::to_string(row) + " is not divisible by group_size " + std::to_string(init.group_size);
        return false;
      }
    }
    m->initializers.push_back(std::move(init));
  }
  // a scale key must not name another initializer's tensor (container.ts:266-283)
  for (const Initializer& a : m->initializers)
    if (!a.scale_key.empty())
      for (const Initializer& b : m->initializers)
        if (b.tensor == a.scale_key) {
          *err = "initializer '" + a.name + "': scale key '" + a.scale_key + "' is also the tensor of initializer '" + b.name + "'";
          return false;
        }
  return true;
}

// Declarations against the tensors of the file (container.ts:180-232, :337-400, :309-320).
bool check_against_file(Model* m, std::string* err) {
  for (const Initializer& init : m->initializers) {
    const std::string where = "initializer '" + init.name + "'";
    auto it = m->tensors.find(init.tensor);
    if (it == m->tensors.end()) {
      *err = where + ": tensor '" + init.tensor + "' is not in the file";
      return false;
    }
    TensorView& view = it->second;
    view.referenced = true;
    if (std::string(view.dtype->name) != storage_encoding(init.storage)) {
      *err = where + ": tensor is " + view.dtype->name + ", storage '" + init.storage + "' needs " + storage_encoding(init.storage);
      return false;
    }
    if (view.shape != init.shape) {
      *err = where + ": tensor shape " + shape_text(view.shape) + " differs from the declared " + shape_text(init.shape);
      return false;
    }
    if (init.scale_key.empty()) continue;
    auto st = m->tensors.find(init.scale_key);
    if (st == m->tensors.end()) {
      *err = where + ": scale tensor '" + init.scale_key + "' is not in the file";
      return false;
    }
    TensorView& scale = st->second;
    scale.referenced = true;
    if (std::string(scale.dtype->name) != "F32") {
      *err = where + ": scale tensor '" + init.scale_key + "' is " + scale.dtype->name + " (F32 needed)";
      return false;
    }
    if (init.group_size != 0) {
      const std::vector<uint64_t> expected = {init.shape[0], numel_of(init.shape) / init.shape[0] / init.group_size};
      if (scale.shape != expected) {
        *err = where + ": scale " + shape_text(scale.shape) + " is not the group form " + shape_text(expected) +
               " (rank 2 whatever the weight's rank, group_size=" + std::to_string(init.group_size) + ")";
        return false;
      }
    } else {
      bool ok = scale.shape.size() == init.shape.size();
      for (size_t axis = 0; ok && axis < init.shape.size(); ++axis)
        ok = scale.shape[axis] == 1 || scale.shape[axis] == init.shape[axis];
      if (!ok) {
        *err = where + ": scale " + shape_text(scale.shape) + " does not broadcast to the weight " + shape_text(init.shape) +
               " (keepdim form of the same rank needed)";
        return false;
      }
    }
  }
  std::string surplus;
  int count = 0;
  for (const auto& kv : m->tensors)
    if (!kv.second.referenced) {
      surplus += (count++ ? ", " : "") + kv.first;
    }
  if (count > 0) {
    *err = "tensors no initializer refers to (" + std::to_string(count) + "): " + surplus;
    return false;
  }
  return true;
}

std::map<uint64_t, std::unique_ptr<Model>>& registry() {
  static std::map<uint64_t, std::unique_ptr<Model>> models;
  return models;
}
uint64_t g_next_model = 1;

Model* find_model(uint64_t handle) {
  auto it = registry().find(handle);
  return it == registry().end() ? nullptr : it->second.get();
}

int open_parsed(std::unique_ptr<Model> m, uint64_t* out, bool with_graph = true) {
  std::string err;
  if (!parse_safetensors(m.get(), &err) || (with_graph && (!parse_ir(m.get(), &err) || !check_against_file(m.get(), &err)))) {
    set_global_error("kq_model_open: " + err);
    return KQ_ERR_SHAPE;
  }
  for (const Initializer& init : m->initializers) m->names.push_back(init.name);
  const uint64_t handle = g_next_model++;
  registry()[handle] = std::move(m);
  *out = handle;
  return KQ_OK;
}

const Initializer* find_initializer(const Model* m, const char* name) {
  for (const Initializer& init : m->initializers)
    if (init.name == name) return &init;
  return nullptr;
}

}  // namespace
}  // namespace kq

extern "C" {

int kq_model_open_memory(const void* bytes, uint64_t size, kq_model* out) {
  if (!bytes || !out) {
    kq::set_global_error("kq_model_open_memory: null argument");
    return KQ_ERR_BAD_ARG;
  }
  *out = 0;
  std::unique_ptr<kq::Model> m(new kq::Model());
  m->owned.assign(static_cast<const uint8_t*>(bytes), static_cast<const uint8_t*>(bytes) + size);
  m->bytes = m->owned.data();
  m->size = size;
  return kq::open_parsed(std::move(m), out);
}

static int open_path(const char* path, kq_model* out, bool with_graph) {
  if (!path || !out) {
    kq::set_global_error("kq_model_open: null argument");
    return KQ_ERR_BAD_ARG;
  }
  *out = 0;
  FILE* f = fopen(path, "rb");
  if (!f) {
    kq::set_global_error(std::string("kq_model_open: cannot open ") + path);
    return KQ_ERR_BAD_ARG;
  }
  std::unique_ptr<kq::Model> m(new kq::Model());
  fseek(f, 0, SEEK_END);
  const long len = ftell(f);
  fseek(f, 0, SEEK_SET);
  m->owned.resize(len > 0 ? static_cast<size_t>(len) : 0);
  const size_t got = m->owned.empty() ? 0 : fread(m->owned.data(), 1, m->owned.size(), f);
  fclose(f);
  if (got != m->owned.size()) {
    kq::set_global_error(std::string("kq_model_open: short read of ") + path);
    return KQ_ERR_BAD_ARG;
  }
  m->bytes = m->owned.data();
  m->size = m->owned.size();
  return kq::open_parsed(std::move(m), out, with_graph);
}

int kq_model_open(const char* path, kq_model* out) { return open_path(path, out, true); }
int kq_tensors_open(const char* path, kq_model* out) { return open_path(path, out, false); }

int kq_model_tensor_info(kq_model model, const char* key, char* dtype8, uint32_t* rank, uint64_t* shape8, const void** data,
                         uint64_t* bytes) {
  const kq::Model* m = kq::find_model(model);
  auto it = m && key ? m->tensors.find(key) : std::map<std::string, kq::TensorView>::const_iterator();
  if (!m || !key || it == m->tensors.end()) {
    kq::set_global_error("kq_model_tensor_info: unknown model handle or tensor key");
    return KQ_ERR_BAD_ARG;
  }
  const kq::TensorView& view = it->second;
  if (dtype8) {
    memset(dtype8, 0, 8);
    strncpy(dtype8, view.dtype->name, 7);
  }
  if (rank) *rank = static_cast<uint32_t>(view.shape.size());
  if (shape8)
    for (size_t i = 0; i < 8; ++i) shape8[i] = i < view.shape.size() ? view.shape[i] : 0;
  if (data) *data = m->bytes + view.offset;
  if (bytes) *bytes = view.end - view.begin;
  return KQ_OK;
}

void kq_model_close(kq_model model) { kq::registry().erase(model); }

uint32_t kq_model_initializer_count(kq_model model) {
  const kq::Model* m = kq::find_model(model);
  return m ? static_cast<uint32_t>(m->initializers.size()) : 0u;
}

const char* kq_model_initializer_name(kq_model model, uint32_t index) {
  const kq::Model* m = kq::find_model(model);
  return m && index < m->names.size() ? m->names[index].c_str() : nullptr;
}

int kq_model_initializer_info(kq_model model, const char* name, uint32_t* storage_bits, uint32_t* rank, uint64_t* shape8,
                              uint32_t* group_size, const void** payload, uint64_t* payload_bytes, const void** scale,
                              uint64_t* scale_bytes) {
  const kq::Model* m = kq::find_model(model);
  const kq::Initializer* init = m && name ? kq::find_initializer(m, name) : nullptr;
  if (!init) {
    kq::set_global_error("kq_model_initializer_info: unknown model handle or initializer name");
    return KQ_ERR_BAD_ARG;
  }
  const kq::TensorView& view = m->tensors.at(init->tensor);
  if (storage_bits) *storage_bits = view.dtype->bits;
  if (rank) *rank = static_cast<uint32_t>(init->shape.size());
  if (shape8)
    for (size_t i = 0; i < 8; ++i) shape8[i] = i < init->shape.size() ? init->shape[i] : 0;
  if (group_size) *group_size = static_cast<uint32_t>(init->group_size);
  if (payload) *payload = m->bytes + view.offset;
  if (payload_bytes) *payload_bytes = view.end - view.begin;
  if (scale) *scale = nullptr;
  if (scale_bytes) *scale_bytes = 0;
  if (!init->scale_key.empty()) {
    const kq::TensorView& sv = m->tensors.at(init->scale_key);
    if (scale) *scale = m->bytes + sv.offset;
    if (scale_bytes) *scale_bytes = sv.end - sv.begin;
  }
  return KQ_OK;
}

int kq_model_weight(kq_ctx* ctx, kq_model model, const char* name, kq_weight* out) {
  if (!ctx || !out) return KQ_ERR_BAD_ARG;
  *out = 0;
  const kq::Model* m = kq::find_model(model);
  const kq::Initializer* init = m && name ? kq::find_initializer(m, name) : nullptr;
  if (!init) return kq::ctx_fail(ctx, KQ_ERR_BAD_ARG, "kq_model_weight: unknown model handle or initializer name");
  if (init->storage != "i4" && init->storage != "i8")
    return kq::ctx_fail(ctx, KQ_ERR_UNSUPPORTED, "kq_model_weight: initializer is stored as '" + init->storage +
                                                     "'; only packed i4 / i8 weights stay resident through this path");
  if (init->shape.size() < 2 || init->shape[0] == 0)
    return kq::ctx_fail(ctx, KQ_ERR_SHAPE, "kq_model_weight: a linear / embedding weight has rank >= 2");
  const kq::TensorView& view = m->tensors.at(init->tensor);
  const kq::TensorView& sv = m->tensors.at(init->scale_key);
  const uint64_t n = init->shape[0], k = kq::numel_of(init->shape) / n;
  if (n > 0xffffffffull || k > 0xffffffffull) return kq::ctx_fail(ctx, KQ_ERR_SHAPE, "kq_model_weight: dimension beyond 32 bits");
  if (init->storage == "i8") {
    // the resident path indexes the scale by output channel (axis 0): every other axis of the
    // keepdim form must be 1 (packages/runtime/src/runtime/executor.ts:830-854)
    for (size_t axis = 1; axis < sv.shape.size(); ++axis)
      if (sv.shape[axis] != 1)
        return kq::ctx_fail(ctx, KQ_ERR_SHAPE, "kq_model_weight: the i8 scale varies along an axis other than the output channel");
    if (sv.shape.empty() || sv.shape[0] != n)
      return kq::ctx_fail(ctx, KQ_ERR_SHAPE, "kq_model_weight: the i8 scale is not per output channel");
  }
  return kq_weight_upload(ctx, init->storage == "i4" ? KQ_STORAGE_I4 : KQ_STORAGE_I8, m->bytes + view.offset,
                          view.end - view.begin, m->bytes + sv.offset, sv.end - sv.begin, KQ_F32, static_cast<uint32_t>(n),
                          static_cast<uint32_t>(k), static_cast<uint32_t>(init->group_size), out);
}

}  // extern "C"
