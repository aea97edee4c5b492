// Reader of the packed expert sidecar (a safetensors file) and its 13-tensor-per-layer schema.
//
// Replaces, for this path, the reference's strict safetensors inspection
// (src/safetensors.cpp, include/gevva/safetensors.hpp:12-27) and the schema check its
// runtime applies to the sidecar (src/runtime.cpp:222-254).  Host code only: the file is
// mapped read-only and tensors are returned as views into the mapping; uploading them is the
// caller's business (the Python mirror does it with one copy per tensor).
//
// File format: 8-byte little-endian header length N, N bytes of JSON
//   { "<name>": {"dtype": "U8", "shape": [..], "data_offsets": [begin, end]}, ...,
//     "__metadata__": {"k": "v", ...} }
// then the data section.  Validation is as strict as the reference's: integers only (no
// fractions, no negatives), known whole-byte dtypes, end-begin = numel*itemsize without
// overflow, and the tensors must tile the data section exactly (no overlap, gap or unclaimed
// byte).  The JSON reader below accepts exactly the subset such headers use.
#include <fcntl.h>
#include <stdint.h>
#include <string.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <map>
#include <string>
#include <vector>

#include "../../include/gevva_moe.h"

namespace {

thread_local std::string g_sidecar_error;

struct Failure {
  std::string what;
};

[[noreturn]] void fail(const std::string& what) { throw Failure{what}; }

// ---------------------------------------------------------------------------
// JSON subset: objects, arrays, strings, non-negative integers.  Any other number form
// (sign, fraction, exponent) is remembered as "not an integer" so that the caller can reject
// it where an integer is required; true/false/null are parsed and never valid where used.
// ---------------------------------------------------------------------------
struct Value {
  enum Kind { kObject, kArray, kString, kInteger, kOtherNumber, kLiteral } kind = kLiteral;
  std::vector<std::pair<std::string, Value>> members;  // object, in file order
  std::vector<Value> items;                            // array
  std::string text;                                    // string
  uint64_t integer = 0;
};

class Parser {
 public:
  Parser(const char* begin, const char* end) : p_(begin), end_(end) {}

  Value document() {
    Value v = value(0);
    skip_space();
    if (p_ != end_) fail("trailing characters after the header object");
    return v;
  }

 private:
  void skip_space() {
    while (p_ != end_ && (*p_ == ' ' || *p_ == '\n' || *p_ == '\r' || *p_ == '\t')) ++p_;
  }
  char peek() {
    if (p_ == end_) fail("header ends inside a value");
    return *p_;
  }
  void expect(char c) {
    if (peek() != c) fail(std::string("expected '") + c + "' in header");
    ++p_;
  }

  Value value(int depth) {
    if (depth > 16) fail("header nested too deeply");
    skip_space();
    const char c = peek();
    Value v;
    if (c == '{') {
      v.kind = Value::kObject;
      ++p_;
      skip_space();
      if (peek() == '}') {
        ++p_;
        return v;
      }
      for (;;) {
        skip_space();
        std::string key = string();
        skip_space();
        expect(':');
        for (const auto& member : v.members)
          if (member.first == key) fail("duplicate key in header: " + key);
        Value inner = value(depth + 1);
        v.members.emplace_back(std::move(key), std::move(inner));
        skip_space();
        if (peek() == ',') {
          ++p_;
          continue;
        }
        expect('}');
        return v;
      }
    }
    if (c == '[') {
      v.kind = Value::kArray;
      ++p_;
      skip_space();
      if (peek() == ']') {
        ++p_;
        return v;
      }
      for (;;) {
        v.items.push_back(value(depth + 1));
        skip_space();
        if (peek() == ',') {
          ++p_;
          continue;
        }
        expect(']');
        return v;
      }
    }
    if (c == '"') {
      v.kind = Value::kString;
      v.text = string();
      return v;
    }
    if (c == '-' || (c >= '0' && c <= '9')) return number();
    for (const char* word : {"true", "false", "null"}) {
      const size_t n = strlen(word);
      if (static_cast<size_t>(end_ - p_) >= n && memcmp(p_, word, n) == 0) {
        p_ += n;
        v.kind = Value::kLiteral;
        return v;
      }
    }
    fail("unexpected character in header");
  }

  Value number() {
    Value v;
    v.kind = Value::kInteger;
    if (*p_ == '-') {
      v.kind = Value::kOtherNumber;
      ++p_;
    }
    if (p_ == end_ || *p_ < '0' || *p_ > '9') fail("malformed number in header");
    if (*p_ == '0' && p_ + 1 != end_ && p_[1] >= '0' && p_[1] <= '9') fail("leading zero in header number");
    bool overflow = false;
    while (p_ != end_ && *p_ >= '0' && *p_ <= '9') {
      const uint64_t digit = static_cast<uint64_t>(*p_ - '0');
      if (v.integer > (UINT64_MAX - digit) / 10) overflow = true;
      v.integer = v.integer * 10 + digit;
      ++p_;
    }
    if (p_ != end_ && (*p_ == '.' || *p_ == 'e' || *p_ == 'E')) {
      v.kind = Value::kOtherNumber;
      while (p_ != end_ && ((*p_ >= '0' && *p_ <= '9') || *p_ == '.' || *p_ == 'e' || *p_ == 'E' ||
                            *p_ == '+' || *p_ == '-'))
        ++p_;
    }
    if (overflow) v.kind = Value::kOtherNumber;
    return v;
  }

  std::string string() {
    expect('"');
    std::string out;
    for (;;) {
      if (p_ == end_) fail("unterminated string in header");
      const unsigned char c = static_cast<unsigned char>(*p_++);
      if (c == '"') return out;
      if (c < 0x20) fail("control character inside a header string");
      if (c != '\\') {
        out.push_back(static_cast<char>(c));
        continue;
      }
      if (p_ == end_) fail("unterminated escape in header");
      const char e = *p_++;
      switch (e) {
        case '"': out.push_back('"'); break;
        case '\\': out.push_back('\\'); break;
        case '/': out.push_back('/'); break;
        case 'b': out.push_back('\b'); break;
        case 'f': out.push_back('\f'); break;
        case 'n': out.push_back('\n'); break;
        case 'r': out.push_back('\r'); break;
        case 't': out.push_back('\t'); break;
        case 'u': {
          if (end_ - p_ < 4) fail("short \\u escape in header");
          unsigned code = 0;
          for (int i = 0; i < 4; ++i) {
            const char h = *p_++;
            code <<= 4;
            if (h >= '0' && h <= '9') code |= static_cast<unsigned>(h - '0');
            else if (h >= 'a' && h <= 'f') code |= static_cast<unsigned>(h - 'a' + 10);
            else if (h >= 'A' && h <= 'F') code |= static_cast<unsigned>(h - 'A' + 10);
            else fail("bad \\u escape in header");
          }
          // tensor names are ASCII in practice; encode the BMP code point as UTF-8
          if (code < 0x80) out.push_back(static_cast<char>(code));
          else if (code < 0x800) {
            out.push_back(static_cast<char>(0xC0 | (code >> 6)));
            out.push_back(static_cast<char>(0x80 | (code & 0x3F)));
          } else {
            out.push_back(static_cast<char>(0xE0 | (code >> 12)));
            out.push_back(static_cast<char>(0x80 | ((code >> 6) & 0x3F)));
            out.push_back(static_cast<char>(0x80 | (code & 0x3F)));
          }
          break;
        }
        default: fail("unknown escape in header string");
      }
    }
  }

  const char* p_;
  const char* end_;
};

// ---------------------------------------------------------------------------
struct Tensor {
  std::string dtype;
  std::vector<uint64_t> shape;
  uint64_t begin = 0, end = 0;
};

int item_bytes(const std::string& dtype) {
  static const std::pair<const char*, int> kTable[] = {
      {"BOOL", 1}, {"U8", 1},   {"I8", 1},   {"F8_E4M3", 1}, {"F8_E5M2", 1}, {"F8_E8M0", 1},
      {"U16", 2},  {"I16", 2},  {"F16", 2},  {"BF16", 2},    {"U32", 4},     {"I32", 4},
      {"F32", 4},  {"U64", 8},  {"I64", 8},  {"F64", 8}};
  for (const auto& entry : kTable)
    if (dtype == entry.first) return entry.second;
  return 0;  // unknown or sub-byte (F4, F6_*) types are refused
}

const Value* member(const Value& object, const char* key) {
  for (const auto& m : object.members)
    if (m.first == key) return &m.second;
  return nullptr;
}

}  // namespace

struct gevva_sidecar {
  int fd = -1;
  const uint8_t* mapping = nullptr;
  uint64_t file_size = 0;
  uint64_t data_begin = 0;  // 8 + header length
  std::map<std::string, Tensor> tensors;
};

namespace {

void parse_header(gevva_sidecar* s) {
  if (s->file_size < 8) fail("file shorter than the 8-byte header length");
  uint64_t header_size = 0;
  for (int i = 0; i < 8; ++i) header_size |= static_cast<uint64_t>(s->mapping[i]) << (8 * i);
  if (header_size > s->file_size - 8) fail("header length exceeds the file");
  s->data_begin = 8 + header_size;
  const uint64_t data_size = s->file_size - s->data_begin;
  const char* text = reinterpret_cast<const char*>(s->mapping + 8);
  Value root = Parser(text, text + header_size).document();
  if (root.kind != Value::kObject) fail("header is not a JSON object");
  for (const auto& entry : root.members) {
    const std::string& name = entry.first;
    const Value& v = entry.second;
    if (name == "__metadata__") {
      if (v.kind != Value::kObject) fail("__metadata__ is not an object");
      for (const auto& m : v.members)
        if (m.second.kind != Value::kString) fail("__metadata__ value is not a string: " + m.first);
      continue;
    }
    if (v.kind != Value::kObject) fail("tensor entry is not an object: " + name);
    const Value* dtype = member(v, "dtype");
    const Value* shape = member(v, "shape");
    const Value* offsets = member(v, "data_offsets");
    if (!dtype || dtype->kind != Value::kString) fail("tensor without a dtype string: " + name);
    if (!shape || shape->kind != Value::kArray) fail("tensor shape is not an array: " + name);
    if (!offsets || offsets->kind != Value::kArray || offsets->items.size() != 2)
      fail("data_offsets is not a pair: " + name);
    Tensor t;
    t.dtype = dtype->text;
    const int item = item_bytes(t.dtype);
    if (item == 0) fail("unknown or sub-byte dtype '" + t.dtype + "': " + name);
    uint64_t elements = 1;
    for (const Value& d : shape->items) {
      if (d.kind != Value::kInteger) fail("shape entry is not a non-negative integer: " + name);
      if (d.integer != 0 && elements > UINT64_MAX / d.integer) fail("shape overflows: " + name);
      elements *= d.integer;
      t.shape.push_back(d.integer);
    }
    if (elements > UINT64_MAX / static_cast<uint64_t>(item)) fail("byte size overflows: " + name);
    for (const Value& o : offsets->items)
      if (o.kind != Value::kInteger) fail("data offset is not a non-negative integer: " + name);
    t.begin = offsets->items[0].integer;
    t.end = offsets->items[1].integer;
    if (t.begin > t.end) fail("data offsets reversed: " + name);
    if (t.end > data_size) fail("tensor lies outside the file: " + name);
    if (t.end - t.begin != elements * static_cast<uint64_t>(item))
      fail("data_offsets do not match shape and dtype: " + name);
    s->tensors.emplace(name, std::move(t));
  }
  // The tensors must tile the data section exactly.
  std::vector<const Tensor*> order;
  for (const auto& entry : s->tensors) order.push_back(&entry.second);
  std::stable_sort(order.begin(), order.end(), [](const Tensor* a, const Tensor* b) {
    return a->begin != b->begin ? a->begin < b->begin : a->end < b->end;
  });
  uint64_t cursor = 0;
  for (const Tensor* t : order) {
    if (t->begin < cursor) fail("tensors overlap in the data section");
    if (t->begin > cursor) fail("gap in the data section");
    cursor = t->end;
  }
  if (cursor != data_size) fail("unclaimed bytes at the end of the data section");
}

struct SchemaEntry {
  const char* suffix;
  const char* dtype;
  int rank;
  uint64_t shape[3];
};

// The thirteen tensors of one layer (src/runtime.cpp:233-252; writer
// tools/pack_trtllm_experts.py:134-148).
const SchemaEntry kLayerSchema[] = {
    {"w13.weight", "U8", 3, {128, 1408, 1408}},
    {"w13.weight_scale", "U8", 3, {128, 1408, 176}},
    {"w2.weight", "U8", 3, {128, 2816, 352}},
    {"w2.weight_scale", "U8", 3, {128, 2816, 44}},
    {"w13.input_scale", "F32", 1, {128, 0, 0}},
    {"w2.input_scale", "F32", 1, {128, 0, 0}},
    {"w13.weight_scale_2", "F32", 2, {128, 2, 0}},
    {"w2.weight_scale_2", "F32", 1, {128, 0, 0}},
    {"g1.alpha", "F32", 1, {128, 0, 0}},
    {"g1.alpha_up", "F32", 1, {128, 0, 0}},
    {"g2.alpha", "F32", 1, {128, 0, 0}},
    {"g1.input_scale_quant", "F32", 1, {128, 0, 0}},
    {"g2.input_scale_quant", "F32", 1, {128, 0, 0}},
};

const Tensor& require(const gevva_sidecar* s, const std::string& name, const SchemaEntry& e) {
  const auto found = s->tensors.find(name);
  if (found == s->tensors.end()) fail("missing packed expert tensor: " + name);
  const Tensor& t = found->second;
  bool ok = t.dtype == e.dtype && static_cast<int>(t.shape.size()) == e.rank;
  for (int i = 0; ok && i < e.rank; ++i) ok = t.shape[i] == e.shape[i];
  if (!ok) fail("invalid packed expert tensor: " + name);
  return t;
}

template <class Body>
int guarded(Body body) {
  try {
    g_sidecar_error.clear();
    return body();
  } catch (const Failure& f) {
    g_sidecar_error = f.what;
    return GEVVA_MOE_BAD_ARGUMENT;
  } catch (const std::exception& e) {
    g_sidecar_error = e.what();
    return GEVVA_MOE_BAD_ARGUMENT;
  }
}

}  // namespace

extern "C" {

int gevva_sidecar_open(gevva_sidecar** out, const char* path) {
  if (!out || !path) return GEVVA_MOE_BAD_ARGUMENT;
  *out = nullptr;
  gevva_sidecar* s = new gevva_sidecar();
  const int status = guarded([&]() {
    s->fd = open(path, O_RDONLY | O_CLOEXEC);
    if (s->fd < 0) fail(std::string("cannot open ") + path);
    struct stat st;
    if (fstat(s->fd, &st) != 0 || st.st_size < 0) fail(std::string("cannot stat ") + path);
    s->file_size = static_cast<uint64_t>(st.st_size);
    if (s->file_size == 0) fail("empty file");
    void* mapping = mmap(nullptr, s->file_size, PROT_READ, MAP_PRIVATE, s->fd, 0);
    if (mapping == MAP_FAILED) fail(std::string("cannot map ") + path);
    s->mapping = static_cast<const uint8_t*>(mapping);
    parse_header(s);
    return static_cast<int>(GEVVA_MOE_OK);
  });
  if (status != GEVVA_MOE_OK) {
    gevva_sidecar_close(s);
    return status;
  }
  *out = s;
  return GEVVA_MOE_OK;
}

void gevva_sidecar_close(gevva_sidecar* s) {
  if (!s) return;
  if (s->mapping) munmap(const_cast<uint8_t*>(s->mapping), s->file_size);
  if (s->fd >= 0) close(s->fd);
  delete s;
}

int gevva_sidecar_tensor_count(const gevva_sidecar* s) {
  return s ? static_cast<int>(s->tensors.size()) : GEVVA_MOE_BAD_ARGUMENT;
}

int gevva_sidecar_tensor(const gevva_sidecar* s, const char* name, gevva_sidecar_view* view) {
  if (!s || !name || !view) return GEVVA_MOE_BAD_ARGUMENT;
  return guarded([&]() {
    const auto found = s->tensors.find(name);
    if (found == s->tensors.end()) fail(std::string("no such tensor: ") + name);
    const Tensor& t = found->second;
    if (t.shape.size() > 8) fail(std::string("more than 8 dimensions: ") + name);
    memset(view, 0, sizeof(*view));
    strncpy(view->dtype, t.dtype.c_str(), sizeof(view->dtype) - 1);
    view->rank = static_cast<int>(t.shape.size());
    for (size_t i = 0; i < t.shape.size(); ++i) view->shape[i] = t.shape[i];
    view->data = s->mapping + s->data_begin + t.begin;
    view->bytes = t.end - t.begin;
    return static_cast<int>(GEVVA_MOE_OK);
  });
}

int gevva_sidecar_check_layers(const gevva_sidecar* s, int layers) {
  if (!s || layers < 0) return GEVVA_MOE_BAD_ARGUMENT;
  return guarded([&]() {
    for (int layer = 0; layer < layers; ++layer) {
      const std::string prefix = "layers." + std::to_string(layer) + ".";
      for (const SchemaEntry& e : kLayerSchema) require(s, prefix + e.suffix, e);
    }
    const size_t expected = static_cast<size_t>(layers) * (sizeof(kLayerSchema) / sizeof(kLayerSchema[0]));
    if (s->tensors.size() != expected) fail("packed expert sidecar has unexpected tensors");
    return static_cast<int>(GEVVA_MOE_OK);
  });
}

int gevva_sidecar_layer_weights(const gevva_sidecar* s, int layer, gevva_moe_weights* host_views) {
  if (!s || !host_views || layer < 0) return GEVVA_MOE_BAD_ARGUMENT;
  return guarded([&]() {
    const std::string prefix = "layers." + std::to_string(layer) + ".";
    const uint8_t* base = s->mapping + s->data_begin;
    auto data = [&](int index) -> const void* {
      return base + require(s, prefix + kLayerSchema[index].suffix, kLayerSchema[index]).begin;
    };
    // the eight tensors the runner reads (src/nvfp4_cutlass.cu:1792-1802)
    host_views->w13 = data(0);
    host_views->w13_sf = data(1);
    host_views->w2 = data(2);
    host_views->w2_sf = data(3);
    host_views->alpha1 = static_cast<const float*>(data(8));
    host_views->alpha2 = static_cast<const float*>(data(10));
    host_views->in_scale_q1 = static_cast<const float*>(data(11));
    host_views->in_scale_q2 = static_cast<const float*>(data(12));
    return static_cast<int>(GEVVA_MOE_OK);
  });
}

// Checkpoint -> sidecar packing of one layer, on the host.  Follows
// tools/pack_trtllm_experts.py:88-148: stack the experts, w13 rows = [up; gate] (:110-113),
// weights copied as they are, each expert's row-major E4M3 block scales put into the 128-row x
// 4-group interleave (:51-65; offset formula src/nvfp4_cutlass.cu:321-323), and the five derived
// vectors (:141-147) computed in fp32 exactly as the script's tensor arithmetic does.
int gevva_moe_pack_checkpoint_layer(const gevva_checkpoint_expert* experts, int expert_count, int hidden,
                                    int intermediate, gevva_sidecar_layer* out) {
  if (!experts || !out || expert_count < 1 || hidden < 64 || intermediate < 64) return GEVVA_MOE_BAD_ARGUMENT;
  return guarded([&]() {
    // rows of a projection fill whole 128-row scale blocks, K whole groups of 4 block scales
    if (hidden % 128 != 0 || intermediate % 64 != 0 || (2 * intermediate) % 128 != 0)
      fail("hidden must be a multiple of 128 and intermediate a multiple of 64");
    void* const outputs[] = {out->w13_weight, out->w13_weight_scale, out->w2_weight, out->w2_weight_scale,
                             out->w13_input_scale, out->w2_input_scale, out->w13_weight_scale_2,
                             out->w2_weight_scale_2, out->g1_alpha, out->g1_alpha_up, out->g2_alpha,
                             out->g1_input_scale_quant, out->g2_input_scale_quant};
    for (void* pointer : outputs)
      if (!pointer) fail("an output tensor pointer is null");
    const size_t in_row = static_cast<size_t>(hidden) / 2, in_groups = static_cast<size_t>(hidden) / 16;
    const size_t mid_row = static_cast<size_t>(intermediate) / 2, mid_groups = static_cast<size_t>(intermediate) / 16;
    auto interleave = [](const uint8_t* row_major, int rows, size_t groups, uint8_t* dst) {
      for (int r = 0; r < rows; ++r)
        for (size_t g = 0; g < groups; ++g)
          dst[static_cast<size_t>(r >> 7) * (128 * groups) + (g >> 2) * 512 + (r & 31) * 16 + ((r >> 5) & 3) * 4 +
              (g & 3)] = row_major[static_cast<size_t>(r) * groups + g];
    };
    for (int e = 0; e < expert_count; ++e) {
      const gevva_checkpoint_expert& x = experts[e];
      const gevva_checkpoint_projection* parts[3] = {&x.gate_proj, &x.up_proj, &x.down_proj};
      for (const gevva_checkpoint_projection* part : parts)
        if (!part->weight || !part->weight_scale) fail("expert " + std::to_string(e) + ": null checkpoint tensor");
      // "gate/up activation scales differ" (tools/pack_trtllm_experts.py:127-128)
      if (memcmp(&x.gate_proj.input_scale, &x.up_proj.input_scale, sizeof(float)) != 0)
        fail("expert " + std::to_string(e) + ": gate/up activation scales differ");
      uint8_t* w13 = static_cast<uint8_t*>(out->w13_weight) + static_cast<size_t>(e) * 2 * intermediate * in_row;
      memcpy(w13, x.up_proj.weight, static_cast<size_t>(intermediate) * in_row);
      memcpy(w13 + static_cast<size_t>(intermediate) * in_row, x.gate_proj.weight,
             static_cast<size_t>(intermediate) * in_row);
      std::vector<uint8_t> stacked(static_cast<size_t>(2) * intermediate * in_groups);
      memcpy(stacked.data(), x.up_proj.weight_scale, static_cast<size_t>(intermediate) * in_groups);
      memcpy(stacked.data() + static_cast<size_t>(intermediate) * in_groups, x.gate_proj.weight_scale,
             static_cast<size_t>(intermediate) * in_groups);
      interleave(stacked.data(), 2 * intermediate, in_groups,
                 static_cast<uint8_t*>(out->w13_weight_scale) + static_cast<size_t>(e) * 2 * intermediate * in_groups);
      memcpy(static_cast<uint8_t*>(out->w2_weight) + static_cast<size_t>(e) * hidden * mid_row, x.down_proj.weight,
             static_cast<size_t>(hidden) * mid_row);
      interleave(static_cast<const uint8_t*>(x.down_proj.weight_scale), hidden, mid_groups,
                 static_cast<uint8_t*>(out->w2_weight_scale) + static_cast<size_t>(e) * hidden * mid_groups);
      const float gate_input = x.gate_proj.input_scale, down_input = x.down_proj.input_scale;
      out->w13_input_scale[e] = gate_input;
      out->w2_input_scale[e] = down_input;
      out->w13_weight_scale_2[2 * e] = x.gate_proj.weight_scale_2;
      out->w13_weight_scale_2[2 * e + 1] = x.up_proj.weight_scale_2;
      out->w2_weight_scale_2[e] = x.down_proj.weight_scale_2;
      out->g1_alpha[e] = gate_input * x.gate_proj.weight_scale_2;
      out->g1_alpha_up[e] = x.up_proj.input_scale * x.up_proj.weight_scale_2;
      out->g2_alpha[e] = down_input * x.down_proj.weight_scale_2;
      out->g1_input_scale_quant[e] = 1.0f / gate_input;
      out->g2_input_scale_quant[e] = 1.0f / down_input;
    }
    return static_cast<int>(GEVVA_MOE_OK);
  });
}

const char* gevva_sidecar_error(void) { return g_sidecar_error.c_str(); }

}  // extern "C"
