// Minimal safetensors reader/writer for the two blobs that cross the worker boundary:
// the per-expert weight bundle (ek-db/src/safetensor/transformer.rs:282-296) and the
// single-tensor "data" blob of ForwardReq/ForwardResp (ek-computation/src/worker/core.rs:52-53,
// ek-computation/src/backend/torch/mod.rs:115-117).
//
// Format: u64 little-endian header length N, N bytes of JSON
//   { "<name>": {"dtype": "...", "shape": [..], "data_offsets": [begin, end]}, ...,
//     "__metadata__": {...} }
// followed by the raw tensor bytes; offsets are relative to the end of the header.
#pragma once
#include <stdint.h>
#include <string.h>

#include <string>
#include <vector>

#include "../../include/ek_b200.h"

namespace ekst {

struct Entry {
  std::string name;
  std::string dtype;
  std::vector<int64_t> shape;
  uint64_t begin = 0, end = 0;
  const uint8_t* data = nullptr;
};

class Parser {
 public:
  Parser(const char* s, size_t n) : s_(s), n_(n) {}
  bool parse(std::vector<Entry>& out, std::string& err) {
    ws();
    if (!eat('{')) return fail(err, "header is not a JSON object");
    ws();
    if (peek() == '}') { ++i_; return true; }
    while (true) {
      std::string key;
      if (!str(key)) return fail(err, "bad key");
      ws();
      if (!eat(':')) return fail(err, "missing ':'");
      ws();
      if (key == "__metadata__") {
        if (!skip_value()) return fail(err, "bad __metadata__");
      } else {
        Entry e;
        e.name = key;
        if (!tensor(e)) return fail(err, "bad tensor entry '" + key + "'");
        out.push_back(e);
      }
      ws();
      if (eat(',')) { ws(); continue; }
      if (eat('}')) return true;
      return fail(err, "expected ',' or '}'");
    }
  }

 private:
  const char* s_;
  size_t n_, i_ = 0;
  static bool fail(std::string& err, const std::string& m) { err = m; return false; }
  char peek() const { return i_ < n_ ? s_[i_] : '\0'; }
  bool eat(char c) { if (peek() == c) { ++i_; return true; } return false; }
  void ws() { while (i_ < n_ && (s_[i_] == ' ' || s_[i_] == '\n' || s_[i_] == '\t' || s_[i_] == '\r')) ++i_; }
  bool str(std::string& out) {
    if (!eat('"')) return false;
    out.clear();
    while (i_ < n_ && s_[i_] != '"') {
      if (s_[i_] == '\\' && i_ + 1 < n_) { out.push_back(s_[i_ + 1]); i_ += 2; }
      else out.push_back(s_[i_++]);
    }
    return eat('"');
  }
  bool num(int64_t& v) {
    size_t st = i_;
    bool neg = eat('-');
    int64_t x = 0;
    while (i_ < n_ && s_[i_] >= '0' && s_[i_] <= '9') x = x * 10 + (s_[i_++] - '0');
    if (i_ == st + (neg ? 1 : 0)) return false;
    v = neg ? -x : x;
    return true;
  }
  bool num_array(std::vector<int64_t>& out) {
    if (!eat('[')) return false;
    ws();
    if (eat(']')) return true;
    while (true) {
      int64_t v;
      ws();
      if (!num(v)) return false;
      out.push_back(v);
      ws();
      if (eat(',')) continue;
      return eat(']');
    }
  }
  bool skip_value() {
    ws();
    char c = peek();
    if (c == '"') { std::string t; return str(t); }
    if (c == '{' || c == '[') {
      char open = c, close = c == '{' ? '}' : ']';
      int depth = 0;
      while (i_ < n_) {
        char d = s_[i_];
        if (d == '"') { std::string t; if (!str(t)) return false; continue; }
        if (d == open) ++depth;
        if (d == close) { --depth; ++i_; if (depth == 0) return true; continue; }
        ++i_;
      }
      return false;
    }
    while (i_ < n_ && s_[i_] != ',' && s_[i_] != '}' && s_[i_] != ']') ++i_;
    return true;
  }
  bool tensor(Entry& e) {
    if (!eat('{')) return false;
    while (true) {
      ws();
      std::string k;
      if (!str(k)) return false;
      ws();
      if (!eat(':')) return false;
      ws();
      if (k == "dtype") { if (!str(e.dtype)) return false; }
      else if (k == "shape") { if (!num_array(e.shape)) return false; }
      else if (k == "data_offsets") {
        std::vector<int64_t> o;
        if (!num_array(o) || o.size() != 2) return false;
        e.begin = (uint64_t)o[0];
        e.end = (uint64_t)o[1];
      } else if (!skip_value()) return false;
      ws();
      if (eat(',')) continue;
      return eat('}');
    }
  }
};

inline int dtype_from_string(const std::string& s) {
  if (s == "BF16") return EK_BF16;
  if (s == "F32") return EK_F32;
  if (s == "F8_E4M3") return EK_F8_E4M3;
  if (s == "I8") return EK_I8;
  if (s == "I32") return EK_I32;
  if (s == "F16") return EK_F16;
  if (s == "U8") return EK_U8;
  if (s == "I64") return EK_I64;
  return -1;
}
inline int dtype_size(int dt) {
  switch (dt) {
    case EK_BF16: case EK_F16: return 2;
    case EK_F32: case EK_I32: return 4;
    case EK_F8_E4M3: case EK_I8: case EK_U8: return 1;
    case EK_I64: return 8;
  }
  return 0;
}

// Parses a blob; entries point into `blob`.
inline bool parse_blob(const void* blob, size_t len, std::vector<Entry>& out, std::string& err) {
  if (len < 8) { err = "blob shorter than its length prefix"; return false; }
  uint64_t n;
  memcpy(&n, blob, 8);
  if (n > len - 8 || n > (100u << 20)) { err = "header length out of range"; return false; }
  const char* hdr = reinterpret_cast<const char*>(blob) + 8;
  Parser p(hdr, (size_t)n);
  if (!p.parse(out, err)) return false;
  const uint8_t* base = reinterpret_cast<const uint8_t*>(blob) + 8 + n;
  const uint64_t avail = len - 8 - n;
  for (auto& e : out) {
    if (e.begin > e.end || e.end > avail) { err = "data_offsets out of range for '" + e.name + "'"; return false; }
    int dt = dtype_from_string(e.dtype);
    if (dt < 0) { err = "unsupported dtype '" + e.dtype + "'"; return false; }
    // element count with refusal of negative dimensions and of products that leave 64 bits
    uint64_t cnt = 1;
    bool dims_ok = true;
    for (auto d : e.shape) {
      if (d < 0 || (d > 0 && cnt > (UINT64_MAX / 16) / (uint64_t)d)) { dims_ok = false; break; }
      cnt *= (uint64_t)d;
    }
    if (!dims_ok) { err = "shape of '" + e.name + "' is negative or too large"; return false; }
    if (cnt * dtype_size(dt) != e.end - e.begin) { err = "size mismatch for '" + e.name + "'"; return false; }
    e.data = base + e.begin;
  }
  return true;
}

// Header of a blob holding the single BF16 tensor "data" of shape [n, h]; padded to 8 bytes.
inline std::string single_header(int64_t n, int64_t h) {
  std::string j = "{\"data\":{\"dtype\":\"BF16\",\"shape\":[" + std::to_string(n) + "," + std::to_string(h) +
                  "],\"data_offsets\":[0," + std::to_string(n * h * 2) + "]}}";
  while (j.size() % 8) j.push_back(' ');
  return j;
}

}  // namespace ekst
