// Minimal JSON value, parser and writer, plus SHA-256, for the node CLI (no third-party code).
#pragma once
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <map>
#include <memory>
#include <string>
#include <vector>

namespace mj {

struct Value;
using Ptr = std::shared_ptr<Value>;

struct Value {
  enum Kind { Null, Bool, Num, Str, Arr, Obj } kind = Null;
  bool b = false;
  double num = 0;
  std::string raw_num;  // number text as written (large integers keep their digits)
  std::string str;
  std::vector<Ptr> arr;
  std::vector<std::pair<std::string, Ptr>> obj;  // insertion order kept

  const Value* get(const std::string& k) const {
    for (auto& kv : obj)
      if (kv.first == k) return kv.second.get();
    return nullptr;
  }
  bool is_str() const { return kind == Str; }
  bool is_bool() const { return kind == Bool; }
};

struct Parser {
  const char* p;
  const char* end;
  std::string err;

  void ws() {
    while (p < end && (*p == ' ' || *p == '\n' || *p == '\t' || *p == '\r')) p++;
  }
  bool lit(const char* s) {
    size_t n = std::strlen(s);
    if ((size_t)(end - p) >= n && std::memcmp(p, s, n) == 0) {
      p += n;
      return true;
    }
    return false;
  }
  Ptr fail(const char* m) {
    if (err.empty()) err = m;
    return nullptr;
  }
  Ptr string_value() {
    auto v = std::make_shared<Value>();
    v->kind = Value::Str;
    p++;  // opening quote
    while (p < end && *p != '"') {
      if (*p == '\\') {
        if (++p >= end) return fail("bad escape");
        switch (*p) {
          case 'n': v->str.push_back('\n'); break;
          case 't': v->str.push_back('\t'); break;
          case 'r': v->str.push_back('\r'); break;
          case 'b': v->str.push_back('\b'); break;
          case 'f': v->str.push_back('\f'); break;
          case 'u': {
            if (end - p < 5) return fail("bad \\u escape");
            unsigned cp = 0;
            for (int i = 1; i <= 4; i++) {
              char c = p[i];
              cp = cp * 16 + (c >= '0' && c <= '9' ? c - '0' : (c | 32) >= 'a' && (c | 32) <= 'f' ? (c | 32) - 'a' + 10 : 0);
            }
            p += 4;
            if (cp < 0x80) {
              v->str.push_back((char)cp);
            } else if (cp < 0x800) {
              v->str.push_back((char)(0xC0 | (cp >> 6)));
              v->str.push_back((char)(0x80 | (cp & 0x3F)));
            } else {
              v->str.push_back((char)(0xE0 | (cp >> 12)));
              v->str.push_back((char)(0x80 | ((cp >> 6) & 0x3F)));
              v->str.push_back((char)(0x80 | (cp & 0x3F)));
            }
            break;
          }
          default: v->str.push_back(*p);
        }
        p++;
      } else {
        v->str.push_back(*p++);
      }
    }
    if (p >= end) return fail("unterminated string");
    p++;
    return v;
  }
  Ptr value() {
    ws();
    if (p >= end) return fail("unexpected end");
    if (*p == '"') return string_value();
    auto v = std::make_shared<Value>();
    if (*p == '{') {
      v->kind = Value::Obj;
      p++;
      ws();
      if (p < end && *p == '}') {
        p++;
        return v;
      }
      while (true) {
        ws();
        if (p >= end || *p != '"') return fail("object key expected");
        Ptr k = string_value();
        if (!k) return nullptr;
        ws();
        if (p >= end || *p != ':') return fail("':' expected");
        p++;
        Ptr x = value();
        if (!x) return nullptr;
        v->obj.emplace_back(k->str, x);
        ws();
        if (p < end && *p == ',') {
          p++;
          continue;
        }
        if (p < end && *p == '}') {
          p++;
          return v;
        }
        return fail("',' or '}' expected");
      }
    }
    if (*p == '[') {
      v->kind = Value::Arr;
      p++;
      ws();
      if (p < end && *p == ']') {
        p++;
        return v;
      }
      while (true) {
        Ptr x = value();
        if (!x) return nullptr;
        v->arr.push_back(x);
        ws();
        if (p < end && *p == ',') {
          p++;
          continue;
        }
        if (p < end && *p == ']') {
          p++;
          return v;
        }
        return fail("',' or ']' expected");
      }
    }
    if (lit("true")) {
      v->kind = Value::Bool;
      v->b = true;
      return v;
    }
    if (lit("false")) {
      v->kind = Value::Bool;
      return v;
    }
    if (lit("null")) return v;
    const char* s = p;
    while (p < end && (std::strchr("+-.eE", *p) || (*p >= '0' && *p <= '9'))) p++;
    if (p == s) return fail("unexpected character");
    v->kind = Value::Num;
    v->raw_num.assign(s, p - s);
    v->num = std::strtod(v->raw_num.c_str(), nullptr);
    return v;
  }
};

inline Ptr parse(const std::string& text, std::string* err) {
  Parser ps{text.data(), text.data() + text.size(), {}};
  Ptr v = ps.value();
  if (v) {
    ps.ws();
    if (ps.p != ps.end) {
      v = nullptr;
      ps.err = "trailing characters";
    }
  }
  if (!v && err) *err = ps.err;
  return v;
}

inline void escape(const std::string& s, std::string& out) {
  out.push_back('"');
  for (unsigned char c : s) {
    if (c == '"') out += "\\\"";
    else if (c == '\\') out += "\\\\";
    else if (c == '\n') out += "\\n";
    else if (c == '\t') out += "\\t";
    else if (c == '\r') out += "\\r";
    else if (c < 0x20) {
      char buf[8];
      std::snprintf(buf, sizeof buf, "\\u%04x", c);
      out += buf;
    } else out.push_back((char)c);
  }
  out.push_back('"');
}

inline void write(const Value& v, std::string& out) {
  switch (v.kind) {
    case Value::Null: out += "null"; break;
    case Value::Bool: out += v.b ? "true" : "false"; break;
    case Value::Num: out += v.raw_num; break;
    case Value::Str: escape(v.str, out); break;
    case Value::Arr:
      out.push_back('[');
      for (size_t i = 0; i < v.arr.size(); i++) {
        if (i) out.push_back(',');
        write(*v.arr[i], out);
      }
      out.push_back(']');
      break;
    case Value::Obj:
      out.push_back('{');
      for (size_t i = 0; i < v.obj.size(); i++) {
        if (i) out.push_back(',');
        escape(v.obj[i].first, out);
        out.push_back(':');
        write(*v.obj[i].second, out);
      }
      out.push_back('}');
      break;
  }
}

// ---------------------------------------------------------------- SHA-256
inline std::string sha256_hex(const std::string& data) {
  static const uint32_t K[64] = {
      0x428a2f98, 0x71374491, 0xb5c0fbcf, 0xe9b5dba5, 0x3956c25b, 0x59f111f1, 0x923f82a4, 0xab1c5ed5, 0xd807aa98, 0x12835b01,
      0x243185be, 0x550c7dc3, 0x72be5d74, 0x80deb1fe, 0x9bdc06a7, 0xc19bf174, 0xe49b69c1, 0xefbe4786, 0x0fc19dc6, 0x240ca1cc,
      0x2de92c6f, 0x4a7484aa, 0x5cb0a9dc, 0x76f988da, 0x983e5152, 0xa831c66d, 0xb00327c8, 0xbf597fc7, 0xc6e00bf3, 0xd5a79147,
      0x06ca6351, 0x14292967, 0x27b70a85, 0x2e1b2138, 0x4d2c6dfc, 0x53380d13, 0x650a7354, 0x766a0abb, 0x81c2c92e, 0x92722c85,
      0xa2bfe8a1, 0xa81a664b, 0xc24b8b70, 0xc76c51a3, 0xd192e819, 0xd6990624, 0xf40e3585, 0x106aa070, 0x19a4c116, 0x1e376c08,
      0x2748774c, 0x34b0bcb5, 0x391c0cb3, 0x4ed8aa4a, 0x5b9cca4f, 0x682e6ff3, 0x748f82ee, 0x78a5636f, 0x84c87814, 0x8cc70208,
      0x90befffa, 0xa4506ceb, 0xbef9a3f7, 0xc67178f2};
  uint32_t h[8] = {0x6a09e667, 0xbb67ae85, 0x3c6ef372, 0xa54ff53a, 0x510e527f, 0x9b05688c, 0x1f83d9ab, 0x5be0cd19};
  std::string m = data;
  uint64_t bits = (uint64_t)data.size() * 8;
  m.push_back((char)0x80);
  while (m.size() % 64 != 56) m.push_back(0);
  for (int i = 7; i >= 0; i--) m.push_back((char)(bits >> (8 * i)));
  auto rotr = [](uint32_t x, int n) { return (x >> n) | (x << (32 - n)); };
  for (size_t off = 0; off < m.size(); off += 64) {
    uint32_t w[64];
    for (int i = 0; i < 16; i++)
      w[i] = ((uint32_t)(uint8_t)m[off + 4 * i] << 24) | ((uint32_t)(uint8_t)m[off + 4 * i + 1] << 16) |
             ((uint32_t)(uint8_t)m[off + 4 * i + 2] << 8) | (uint32_t)(uint8_t)m[off + 4 * i + 3];
    for (int i = 16; i < 64; i++) {
      uint32_t s0 = rotr(w[i - 15], 7) ^ rotr(w[i - 15], 18) ^ (w[i - 15] >> 3);
      uint32_t s1 = rotr(w[i - 2], 17) ^ rotr(w[i - 2], 19) ^ (w[i - 2] >> 10);
      w[i] = w[i - 16] + s0 + w[i - 7] + s1;
    }
    uint32_t a = h[0], b = h[1], c = h[2], d = h[3], e = h[4], f = h[5], g = h[6], hh = h[7];
    for (int i = 0; i < 64; i++) {
      uint32_t S1 = rotr(e, 6) ^ rotr(e, 11) ^ rotr(e, 25);
      uint32_t ch = (e & f) ^ (~e & g);
      uint32_t t1 = hh + S1 + ch + K[i] + w[i];
      uint32_t S0 = rotr(a, 2) ^ rotr(a, 13) ^ rotr(a, 22);
      uint32_t mj_ = (a & b) ^ (a & c) ^ (b & c);
      uint32_t t2 = S0 + mj_;
      hh = g; g = f; f = e; e = d + t1; d = c; c = b; b = a; a = t1 + t2;
    }
    h[0] += a; h[1] += b; h[2] += c; h[3] += d; h[4] += e; h[5] += f; h[6] += g; h[7] += hh;
  }
  char buf[65];
  for (int i = 0; i < 8; i++) std::snprintf(buf + 8 * i, 9, "%08x", h[i]);
  return std::string(buf, 64);
}

}  // namespace mj
