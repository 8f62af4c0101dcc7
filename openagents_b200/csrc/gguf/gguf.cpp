// GGUF v3 container: memory-mapped reader and streaming writer, exported as a C API.
//
// The reference model server loads GGUF artifacts and detects the family from
// `general.architecture` (docs/muse/muse-glimmer.md:118-126); the container layout itself is the
// public GGUF specification.  Metadata is handed to Python as one JSON document so the binding
// stays a handful of calls.
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstring>
#include <exception>
#include <string>
#include <vector>

#include "quant.h"

namespace b200 {

enum GgufValueType : uint32_t {
  GV_U8 = 0, GV_I8 = 1, GV_U16 = 2, GV_I16 = 3, GV_U32 = 4, GV_I32 = 5, GV_F32 = 6,
  GV_BOOL = 7, GV_STRING = 8, GV_ARRAY = 9, GV_U64 = 10, GV_I64 = 11, GV_F64 = 12,
};

struct TensorInfo {
  std::string name;
  std::vector<uint64_t> dims;  // fastest-varying first, as stored
  uint32_t type = 0;
  uint64_t offset = 0;         // relative to the data section
  uint64_t nbytes = 0;
};

struct Reader {
  int fd = -1;
  const uint8_t* base = nullptr;
  size_t size = 0;
  uint32_t version = 0;
  uint64_t alignment = 32;
  uint64_t data_start = 0;
  std::vector<TensorInfo> tensors;
  std::string meta_json;
  std::string error;
};

struct Cursor {
  const uint8_t* p;
  const uint8_t* end;
  bool ok = true;
  template <class T>
  T get() {
    T v{};
    if (p + sizeof(T) > end) {
      ok = false;
      return v;
    }
    std::memcpy(&v, p, sizeof(T));
    p += sizeof(T);
    return v;
  }
  std::string str() {
    uint64_t n = get<uint64_t>();
    if (!ok || n > (uint64_t)(end - p)) {
      ok = false;
      return {};
    }
    std::string s((const char*)p, (size_t)n);
    p += n;
    return s;
  }
};

static void json_escape(const std::string& s, std::string& out) {
  out.push_back('"');
  for (unsigned char c : s) {
    switch (c) {
      case '"': out += "\\\""; break;
      case '\\': out += "\\\\"; break;
      case '\n': out += "\\n"; break;
      case '\r': out += "\\r"; break;
      case '\t': out += "\\t"; break;
      default:
        if (c < 0x20) {
          char buf[8];
          std::snprintf(buf, sizeof buf, "\\u%04x", c);
          out += buf;
        } else {
          out.push_back((char)c);
        }
    }
  }
  out.push_back('"');
}

static void json_float(double v, std::string& out) {
  if (std::isnan(v) || std::isinf(v)) {
    out += "null";
    return;
  }
  char buf[40];
  std::snprintf(buf, sizeof buf, "%.17g", v);
  out += buf;
  // keep floats recognisable as floats after a JSON round trip
  if (!std::strpbrk(buf, ".eE")) out += ".0";
}

static bool json_value(Cursor& c, uint32_t type, std::string& out) {
  switch (type) {
    case GV_U8: out += std::to_string(c.get<uint8_t>()); break;
    case GV_I8: out += std::to_string(c.get<int8_t>()); break;
    case GV_U16: out += std::to_string(c.get<uint16_t>()); break;
    case GV_I16: out += std::to_string(c.get<int16_t>()); break;
    case GV_U32: out += std::to_string(c.get<uint32_t>()); break;
    case GV_I32: out += std::to_string(c.get<int32_t>()); break;
    case GV_U64: out += std::to_string(c.get<uint64_t>()); break;
    case GV_I64: out += std::to_string(c.get<int64_t>()); break;
    case GV_F32: json_float(c.get<float>(), out); break;
    case GV_F64: json_float(c.get<double>(), out); break;
    case GV_BOOL: out += c.get<uint8_t>() ? "true" : "false"; break;
    case GV_STRING: json_escape(c.str(), out); break;
    case GV_ARRAY: {
      uint32_t et = c.get<uint32_t>();
      uint64_t n = c.get<uint64_t>();
      if (!c.ok || et == GV_ARRAY) return false;
      out.push_back('[');
      for (uint64_t i = 0; i < n && c.ok; i++) {
        if (i) out.push_back(',');
        if (!json_value(c, et, out)) return false;
      }
      out.push_back(']');
      break;
    }
    default:
      return false;
  }
  return c.ok;
}

static Reader* open_reader(const char* path) {
  Reader* r = new Reader();
  r->fd = ::open(path, O_RDONLY);
  if (r->fd < 0) {
    r->error = std::string("cannot open ") + path;
    return r;
  }
  struct stat st;
  if (fstat(r->fd, &st) != 0 || st.st_size < 24) {
    r->error = "file too small for a GGUF header";
    return r;
  }
  r->size = (size_t)st.st_size;
  void* m = mmap(nullptr, r->size, PROT_READ, MAP_PRIVATE, r->fd, 0);
  if (m == MAP_FAILED) {
    r->error = "mmap failed";
    return r;
  }
  r->base = (const uint8_t*)m;
  Cursor c{r->base, r->base + r->size};
  if (std::memcmp(c.p, "GGUF", 4) != 0) {
    r->error = "bad magic";
    return r;
  }
  c.p += 4;
  r->version = c.get<uint32_t>();
  if (r->version < 2 || r->version > 3) {
    r->error = "unsupported GGUF version " + std::to_string(r->version);
    return r;
  }
  uint64_t n_tensors = c.get<uint64_t>();
  uint64_t n_kv = c.get<uint64_t>();
  // A header cannot promise more entries than the file has room for: a key/value pair takes at least 12 bytes (empty
  // key, type, one byte of value), a tensor record at least 24 (empty name, no dimensions, type, offset).
  if (n_kv > r->size / 12 || n_tensors > r->size / 24) {
    r->error = "header counts exceed the file size";
    return r;
  }
  std::string js = "{";
  for (uint64_t i = 0; i < n_kv && c.ok; i++) {
    std::string key = c.str();
    uint32_t vt = c.get<uint32_t>();
    if (i) js.push_back(',');
    json_escape(key, js);
    js.push_back(':');
    const uint8_t* before = c.p;
    if (!json_value(c, vt, js)) {
      r->error = "bad metadata value for key " + key;
      return r;
    }
    if (key == "general.alignment" && vt == GV_U32) {
      uint32_t a;
      std::memcpy(&a, before, 4);
      if (a) r->alignment = a;
    }
  }
  js.push_back('}');
  if (!c.ok) {
    r->error = "truncated metadata";
    return r;
  }
  r->meta_json = js;
  r->tensors.resize((size_t)n_tensors);
  for (auto& t : r->tensors) {
    t.name = c.str();
    uint32_t nd = c.get<uint32_t>();
    if (!c.ok || nd > 8) {
      r->error = "bad tensor info";
      return r;
    }
    t.dims.resize(nd);
    uint64_t n = 1;
    bool overflow = false;
    for (auto& d : t.dims) {
      d = c.get<uint64_t>();
      overflow |= __builtin_mul_overflow(n, d, &n);
    }
    if (overflow || n > (uint64_t)1 << 48) {
      r->error = "tensor " + t.name + " has an impossible element count";
      return r;
    }
    t.type = c.get<uint32_t>();
    t.offset = c.get<uint64_t>();
    const TypeTraits* tt = type_traits(t.type);
    if (!c.ok || !tt) {
      r->error = "tensor " + t.name + " has unsupported type " + std::to_string(t.type);
      return r;
    }
    if (t.dims.empty() || t.dims[0] % tt->block_elems) {
      r->error = "tensor " + t.name + " row length is not a multiple of its block size";
      return r;
    }
    t.nbytes = tensor_bytes(t.type, n);
  }
  uint64_t pos = (uint64_t)(c.p - r->base);
  r->data_start = (pos + r->alignment - 1) / r->alignment * r->alignment;
  if (r->data_start > r->size) {
    r->error = "data section starts past the end of the file";
    return r;
  }
  const uint64_t room = r->size - r->data_start;
  for (auto& t : r->tensors) {
    if (t.offset > room || t.nbytes > room - t.offset) {      // written so that nothing can wrap around
      r->error = "tensor " + t.name + " runs past the end of the file";
      return r;
    }
  }
  return r;
}

// ---------------------------------------------------------------- writer

struct PendingTensor {
  TensorInfo info;
  const void* data;
};

struct Writer {
  std::string path;
  uint64_t alignment = 32;
  uint64_t n_kv = 0;
  std::string kv;  // serialized key/value section
  std::vector<PendingTensor> tensors;
  std::string error;
};

template <class T>
static void put(std::string& s, T v) {
  s.append((const char*)&v, sizeof(T));
}
static void put_str(std::string& s, const char* p, size_t n) {
  put<uint64_t>(s, n);
  s.append(p, n);
}

}  // namespace b200

using namespace b200;

extern "C" {

// ---- quantization helpers
int b200_type_info(uint32_t type, uint32_t* block_elems, uint32_t* block_bytes) {
  const TypeTraits* t = type_traits(type);
  if (!t) return -1;
  *block_elems = t->block_elems;
  *block_bytes = t->block_bytes;
  return 0;
}
const char* b200_type_name(uint32_t type) {
  const TypeTraits* t = type_traits(type);
  return t ? t->name : nullptr;
}
int b200_dequantize(uint32_t type, const void* src, float* dst, uint64_t n) {
  return dequantize(type, src, dst, n);
}
int b200_quantize(uint32_t type, const float* src, void* dst, uint64_t n) {
  return quantize(type, src, dst, n);
}

// ---- reader
// Never lets an exception cross the C boundary: a file whose header makes the parser run out of memory or trip a
// length check comes back as a reader with an error message, like any other malformed file.
void* b200_gguf_open(const char* path) {
  try {
    return open_reader(path);
  } catch (const std::exception& e) {
    Reader* r = new Reader();
    r->error = std::string("malformed file: ") + e.what();
    return r;
  } catch (...) {
    Reader* r = new Reader();
    r->error = "malformed file";
    return r;
  }
}
const char* b200_gguf_error(void* h) {
  Reader* r = (Reader*)h;
  return r->error.empty() ? nullptr : r->error.c_str();
}
void b200_gguf_close(void* h) {
  Reader* r = (Reader*)h;
  if (r->base) munmap((void*)r->base, r->size);
  if (r->fd >= 0) ::close(r->fd);
  delete r;
}
uint32_t b200_gguf_version(void* h) { return ((Reader*)h)->version; }
uint64_t b200_gguf_alignment(void* h) { return ((Reader*)h)->alignment; }
const char* b200_gguf_meta_json(void* h) { return ((Reader*)h)->meta_json.c_str(); }
uint64_t b200_gguf_n_tensors(void* h) { return ((Reader*)h)->tensors.size(); }
const char* b200_gguf_tensor_name(void* h, uint64_t i) {
  return ((Reader*)h)->tensors[i].name.c_str();
}
uint32_t b200_gguf_tensor_type(void* h, uint64_t i) { return ((Reader*)h)->tensors[i].type; }
uint32_t b200_gguf_tensor_ndim(void* h, uint64_t i) {
  return (uint32_t)((Reader*)h)->tensors[i].dims.size();
}
uint64_t b200_gguf_tensor_dim(void* h, uint64_t i, uint32_t d) {
  return ((Reader*)h)->tensors[i].dims[d];
}
uint64_t b200_gguf_tensor_nbytes(void* h, uint64_t i) { return ((Reader*)h)->tensors[i].nbytes; }
uint64_t b200_gguf_tensor_offset(void* h, uint64_t i) { return ((Reader*)h)->tensors[i].offset; }
const void* b200_gguf_tensor_data(void* h, uint64_t i) {
  Reader* r = (Reader*)h;
  return r->base + r->data_start + r->tensors[i].offset;
}

// ---- writer
void* b200_gguf_writer_new(const char* path, uint32_t alignment) {
  Writer* w = new Writer();
  w->path = path;
  if (alignment) w->alignment = alignment;
  put_str(w->kv, "general.alignment", 17);
  put<uint32_t>(w->kv, GV_U32);
  put<uint32_t>(w->kv, (uint32_t)w->alignment);
  w->n_kv = 1;
  return w;
}
static void kv_head(Writer* w, const char* key, uint32_t vt) {
  put_str(w->kv, key, std::strlen(key));
  put<uint32_t>(w->kv, vt);
  w->n_kv++;
}
void b200_gguf_writer_kv_u32(void* h, const char* key, uint32_t v) {
  Writer* w = (Writer*)h;
  kv_head(w, key, GV_U32);
  put(w->kv, v);
}
void b200_gguf_writer_kv_i32(void* h, const char* key, int32_t v) {
  Writer* w = (Writer*)h;
  kv_head(w, key, GV_I32);
  put(w->kv, v);
}
void b200_gguf_writer_kv_u64(void* h, const char* key, uint64_t v) {
  Writer* w = (Writer*)h;
  kv_head(w, key, GV_U64);
  put(w->kv, v);
}
void b200_gguf_writer_kv_f32(void* h, const char* key, float v) {
  Writer* w = (Writer*)h;
  kv_head(w, key, GV_F32);
  put(w->kv, v);
}
void b200_gguf_writer_kv_bool(void* h, const char* key, int v) {
  Writer* w = (Writer*)h;
  kv_head(w, key, GV_BOOL);
  put<uint8_t>(w->kv, v ? 1 : 0);
}
void b200_gguf_writer_kv_str(void* h, const char* key, const char* v, uint64_t n) {
  Writer* w = (Writer*)h;
  kv_head(w, key, GV_STRING);
  put_str(w->kv, v, (size_t)n);
}
// Array of strings: `blob` is the concatenation, `lens[i]` the byte length of element i.
void b200_gguf_writer_kv_str_array(void* h, const char* key, const char* blob,
                                   const uint64_t* lens, uint64_t n) {
  Writer* w = (Writer*)h;
  kv_head(w, key, GV_ARRAY);
  put<uint32_t>(w->kv, GV_STRING);
  put<uint64_t>(w->kv, n);
  size_t off = 0;
  for (uint64_t i = 0; i < n; i++) {
    put_str(w->kv, blob + off, (size_t)lens[i]);
    off += (size_t)lens[i];
  }
}
// Array of a fixed-width scalar type (`elem_type` one of the GGUF scalar ids).
void b200_gguf_writer_kv_array(void* h, const char* key, uint32_t elem_type, const void* data,
                               uint64_t n, uint32_t elem_size) {
  Writer* w = (Writer*)h;
  kv_head(w, key, GV_ARRAY);
  put<uint32_t>(w->kv, elem_type);
  put<uint64_t>(w->kv, n);
  w->kv.append((const char*)data, (size_t)(n * elem_size));
}
// The data pointer must stay valid until b200_gguf_writer_finish.
int b200_gguf_writer_tensor(void* h, const char* name, uint32_t type, uint32_t ndim,
                            const uint64_t* dims, const void* data) {
  Writer* w = (Writer*)h;
  const TypeTraits* tt = type_traits(type);
  if (!tt || ndim == 0 || dims[0] % tt->block_elems) {
    w->error = std::string("bad tensor ") + name;
    return -1;
  }
  PendingTensor p;
  p.info.name = name;
  p.info.type = type;
  uint64_t n = 1;
  for (uint32_t i = 0; i < ndim; i++) {
    p.info.dims.push_back(dims[i]);
    n *= dims[i];
  }
  p.info.nbytes = tensor_bytes(type, n);
  p.data = data;
  w->tensors.push_back(p);
  return 0;
}
int b200_gguf_writer_finish(void* h) {
  Writer* w = (Writer*)h;
  std::string head;
  head.append("GGUF", 4);
  put<uint32_t>(head, 3);
  put<uint64_t>(head, w->tensors.size());
  put<uint64_t>(head, w->n_kv);
  head += w->kv;
  uint64_t off = 0;
  for (auto& t : w->tensors) {
    t.info.offset = off;
    put_str(head, t.info.name.data(), t.info.name.size());
    put<uint32_t>(head, (uint32_t)t.info.dims.size());
    for (auto d : t.info.dims) put<uint64_t>(head, d);
    put<uint32_t>(head, t.info.type);
    put<uint64_t>(head, off);
    off += (t.info.nbytes + w->alignment - 1) / w->alignment * w->alignment;
  }
  std::string tmp = w->path + ".tmp";
  FILE* f = std::fopen(tmp.c_str(), "wb");
  int rc = 0;
  if (!f) {
    w->error = "cannot create " + tmp;
    rc = -1;
  } else {
    static const char zeros[256] = {0};
    auto pad_to = [&](uint64_t pos) {
      uint64_t want = (pos + w->alignment - 1) / w->alignment * w->alignment;
      for (uint64_t left = want - pos; left;) {
        size_t n = (size_t)std::min<uint64_t>(left, sizeof zeros);
        if (std::fwrite(zeros, 1, n, f) != n) rc = -1;
        left -= n;
      }
    };
    if (std::fwrite(head.data(), 1, head.size(), f) != head.size()) rc = -1;
    pad_to(head.size());
    for (auto& t : w->tensors) {
      if (t.info.nbytes && std::fwrite(t.data, 1, t.info.nbytes, f) != t.info.nbytes) rc = -1;
      pad_to(t.info.nbytes);
    }
    if (std::fclose(f) != 0) rc = -1;
    if (rc == 0 && std::rename(tmp.c_str(), w->path.c_str()) != 0) rc = -1;
    if (rc != 0) w->error = "write failed for " + w->path;
  }
  return rc;
}
const char* b200_gguf_writer_error(void* h) {
  Writer* w = (Writer*)h;
  return w->error.empty() ? nullptr : w->error.c_str();
}
void b200_gguf_writer_free(void* h) { delete (Writer*)h; }

}  // extern "C"
