// GGUF container reader (host side, no device code): header parse + mapped tensor bytes.
//
// Follows the reference's `Content::read` (fuel-formats/src/gguf.rs:385-462) in what it accepts and how it reads
// it — versions 1..3, u32 vs u64 counts, strings with trailing NULs dropped, the 13 value types, dimension lists
// reversed, data offset rounded up to general.alignment (default 32) — and the loaders' slicing rule
// (fuel-core/src/lazy_quantized_llama.rs:251-260). Unlike the reference, which reads through a std::io::Read and
// fails on a short read, every access here is bounds-checked against the mapping first, so a truncated or hostile
// file is an error return, never a fault.
#include <cuda_runtime.h>
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cerrno>
#include <cstdio>
#include <cstring>
#include <string>
#include <unordered_map>
#include <vector>

#include "../../include/fuelq.h"
#include "../../include/fuelq_gguf.h"
#include "host.hpp"

namespace {

using fuelq::Error;

struct DTypeInfo {
  int32_t id;
  uint32_t block, bytes;
};
// GgmlDType::{from_u32, type_size, block_size}, fuel-ir/src/quantized.rs:35-103
constexpr DTypeInfo kDTypes[] = {{0, 1, 4},     {1, 1, 2},     {2, 32, 18},    {3, 32, 20},    {6, 32, 22},
                                 {7, 32, 24},   {8, 32, 34},   {9, 32, 36},    {10, 256, 84},  {11, 256, 110},
                                 {12, 256, 144}, {13, 256, 176}, {14, 256, 210}, {15, 256, 292}, {30, 1, 2}};
const DTypeInfo* dtype_info(uint32_t id) {
  for (const DTypeInfo& d : kDTypes)
    if ((uint32_t)d.id == id) return &d;
  return nullptr;
}

struct Value {
  std::string key;
  int32_t type = 0, elem_type = 0;
  uint64_t len = 0;  // string bytes or array elements
  int64_t i = 0;
  double f = 0;
  const char* s = nullptr;
  const void* array = nullptr;
  std::vector<std::pair<const char*, uint64_t>> strings;  // array of strings
};

struct Tensor {
  std::string name;
  int32_t ggml_type = 0, n_dims = 0;
  int64_t dims[8] = {};
  uint64_t offset = 0, nbytes = 0;
};

[[noreturn]] void bad(const std::string& msg) { throw Error("gguf: " + msg, FUELQ_INVALID_PROBLEM); }

// Bounds-checked little-endian cursor over the file image.
class Cursor {
 public:
  Cursor(const uint8_t* base, size_t len) : base_(base), len_(len) {}
  size_t pos() const { return pos_; }
  const uint8_t* take(uint64_t n) {
    if (n > len_ - pos_) bad("unexpected end of file");
    const uint8_t* p = base_ + pos_;
    pos_ += (size_t)n;
    return p;
  }
  template <typename T>
  T get() {
    T v;
    std::memcpy(&v, take(sizeof(T)), sizeof(T));  // the host is little-endian, as is the file
    return v;
  }
  // v1: u32 counts and lengths; v2, v3: u64 (gguf.rs:69-74, 392-403)
  uint64_t count(int version) { return version == 1 ? (uint64_t)get<uint32_t>() : get<uint64_t>(); }
  // read_string, gguf.rs:68-83
  std::pair<const char*, uint64_t> str(int version) {
    uint64_t n = count(version);
    const char* p = reinterpret_cast<const char*>(take(n));
    while (n > 0 && p[n - 1] == 0) --n;
    return {p, n};
  }

 private:
  const uint8_t* base_;
  size_t len_, pos_ = 0;
};

size_t scalar_size(int32_t t) {
  switch (t) {
    case FUELQ_GGUF_U8: case FUELQ_GGUF_I8: case FUELQ_GGUF_BOOL: return 1;
    case FUELQ_GGUF_U16: case FUELQ_GGUF_I16: return 2;
    case FUELQ_GGUF_U32: case FUELQ_GGUF_I32: case FUELQ_GGUF_F32: return 4;
    case FUELQ_GGUF_U64: case FUELQ_GGUF_I64: case FUELQ_GGUF_F64: return 8;
    default: return 0;
  }
}

int32_t value_type(uint32_t v) {  // ValueType::from_u32, gguf.rs:124-142
  if (v > 12) {
    char buf[64];
    std::snprintf(buf, sizeof buf, "unrecognized value-type %#08x", v);
    bad(buf);
  }
  return (int32_t)v;
}

// Value::read, gguf.rs:296-335. depth bounds nested arrays (the format does not, a hostile file could).
void read_value(Cursor& c, int version, int32_t type, Value& out, int depth) {
  out.type = type;
  switch (type) {
    case FUELQ_GGUF_U8: out.i = c.get<uint8_t>(); break;
    case FUELQ_GGUF_I8: out.i = c.get<int8_t>(); break;
    case FUELQ_GGUF_U16: out.i = c.get<uint16_t>(); break;
    case FUELQ_GGUF_I16: out.i = c.get<int16_t>(); break;
    case FUELQ_GGUF_U32: out.i = c.get<uint32_t>(); break;
    case FUELQ_GGUF_I32: out.i = c.get<int32_t>(); break;
    case FUELQ_GGUF_U64: out.i = (int64_t)c.get<uint64_t>(); break;
    case FUELQ_GGUF_I64: out.i = c.get<int64_t>(); break;
    case FUELQ_GGUF_F32: out.f = c.get<float>(); break;
    case FUELQ_GGUF_F64: out.f = c.get<double>(); break;
    case FUELQ_GGUF_BOOL: {
      const uint8_t b = c.get<uint8_t>();
      if (b > 1) bad("unexpected bool value " + std::to_string(b));
      out.i = b;
      break;
    }
    case FUELQ_GGUF_STRING: {
      const auto s = c.str(version);
      out.s = s.first, out.len = s.second;
      break;
    }
    case FUELQ_GGUF_ARRAY: {
      out.elem_type = value_type(c.get<uint32_t>());
      out.len = c.count(version);
      const size_t es = scalar_size(out.elem_type);
      if (es) {
        if (out.len > UINT64_MAX / es) bad("unexpected end of file");
        const uint8_t* p = c.take(out.len * es);
        if (out.elem_type == FUELQ_GGUF_BOOL)
          for (uint64_t j = 0; j < out.len; ++j)
            if (p[j] > 1) bad("unexpected bool value " + std::to_string(p[j]));
        out.array = p;
      } else if (out.elem_type == FUELQ_GGUF_STRING) {
        for (uint64_t j = 0; j < out.len; ++j) out.strings.push_back(c.str(version));  // each str() is bounds-checked
      } else {  // array of arrays: walked for its extent only
        if (depth >= 4) bad("arrays nested too deeply");
        for (uint64_t j = 0; j < out.len; ++j) {
          Value inner;
          read_value(c, version, FUELQ_GGUF_ARRAY, inner, depth + 1);
        }
      }
      break;
    }
    default: bad("unrecognized value-type");
  }
}

}  // namespace

struct fuelq_gguf {
  const uint8_t* base = nullptr;
  size_t len = 0;
  bool mapped = false;
  int version = 0;
  uint64_t alignment = 32, data_offset = 0;
  std::vector<Value> meta;
  std::vector<Tensor> tensors;
  std::unordered_map<std::string, size_t> meta_index, tensor_index;

  ~fuelq_gguf() {
    if (mapped && base) munmap(const_cast<uint8_t*>(base), len);
  }

  void parse() {
    Cursor c(base, len);
    // VersionedMagic::read, gguf.rs:45-58 (either byte order of the four tag characters is accepted, :29)
    const uint32_t magic = c.get<uint32_t>();
    if (magic != 0x46554747u && magic != 0x47475546u) {
      char buf[48];
      std::snprintf(buf, sizeof buf, "unknown magic 0x%08x", magic);
      throw Error(buf, FUELQ_INVALID_PROBLEM);
    }
    const uint32_t ver = c.get<uint32_t>();
    if (ver < 1 || ver > 3) bad("unsupported magic/version Gguf/" + std::to_string(ver));
    version = (int)ver;
    const uint64_t tensor_count = c.count(version), kv_count = c.count(version);

    for (uint64_t n = 0; n < kv_count; ++n) {
      const auto key = c.str(version);
      Value v;
      v.key.assign(key.first, key.second);
      read_value(c, version, value_type(c.get<uint32_t>()), v, 0);
      const auto it = meta_index.find(v.key);  // HashMap::insert: a repeated key keeps its last value
      if (it != meta_index.end()) {
        meta[it->second] = std::move(v);
      } else {
        meta_index.emplace(v.key, meta.size());
        meta.push_back(std::move(v));
      }
    }
    for (uint64_t n = 0; n < tensor_count; ++n) {
      const auto name = c.str(version);
      Tensor t;
      t.name.assign(name.first, name.second);
      const uint32_t nd = c.get<uint32_t>();
      if (nd > 8) bad("tensor " + t.name + " has " + std::to_string(nd) + " dimensions");
      t.n_dims = (int32_t)nd;
      uint64_t elems = 1;
      for (uint32_t d = 0; d < nd; ++d) {
        const uint64_t e = version == 1 ? (uint64_t)c.get<uint32_t>() : c.get<uint64_t>();
        if (e > (uint64_t)INT64_MAX || (e != 0 && elems > (uint64_t)INT64_MAX / e)) bad("tensor " + t.name + " is too large");
        elems *= e;
        t.dims[nd - 1 - d] = (int64_t)e;  // dimensions.reverse(), gguf.rs:431
      }
      const uint32_t dt = c.get<uint32_t>();
      const DTypeInfo* di = dtype_info(dt);
      if (!di) throw Error("unknown dtype for tensor " + std::to_string(dt), FUELQ_INVALID_PROBLEM);
      t.ggml_type = di->id;
      t.offset = c.get<uint64_t>();
      // elems / block * bytes as in lazy_quantized_llama.rs:255-257, but a header is not trusted: a count that is
      // not whole blocks, or a byte size that wraps or exceeds the file, is an error here, not a short tensor
      if (elems % di->block) bad("tensor " + t.name + ": " + std::to_string(elems) + " elements is not a whole number of blocks");
      const uint64_t nblocks = elems / di->block;
      if (nblocks > (uint64_t)len / di->bytes) bad("tensor " + t.name + " is larger than the file");
      t.nbytes = nblocks * di->bytes;
      const auto it = tensor_index.find(t.name);
      if (it != tensor_index.end()) {
        tensors[it->second] = std::move(t);
      } else {
        tensor_index.emplace(t.name, tensors.size());
        tensors.push_back(std::move(t));
      }
    }
    // gguf.rs:443-453
    const auto al = meta_index.find("general.alignment");
    if (al != meta_index.end()) {
      const Value& v = meta[al->second];
      const bool is_unsigned = v.type == FUELQ_GGUF_U8 || v.type == FUELQ_GGUF_U16 || v.type == FUELQ_GGUF_U32;
      const bool is_signed = v.type == FUELQ_GGUF_I8 || v.type == FUELQ_GGUF_I16 || v.type == FUELQ_GGUF_I32;
      if (is_unsigned || (is_signed && v.i >= 0)) alignment = (uint64_t)v.i;
    }
    if (alignment == 0) bad("general.alignment is 0");  // the reference divides by it
    data_offset = (c.pos() + alignment - 1) / alignment * alignment;
  }

  // a tensor's bytes must lie inside the file (checked on use, as the reference's slice is)
  const uint8_t* tensor_data(const Tensor& t) const {
    if (data_offset > len || t.offset > len - data_offset || t.nbytes > len - data_offset - t.offset)
      bad("tensor " + t.name + " lies outside the file");
    return base + data_offset + t.offset;
  }
};

namespace {
template <typename F>
int32_t guarded(F&& f) {
  try {
    f();
    return FUELQ_OK;
  } catch (const Error& e) {
    fuelq::set_last_error(e.what());
    return e.status();
  } catch (const std::exception& e) {
    fuelq::set_last_error(e.what());
    return FUELQ_INVALID_PROBLEM;
  }
}
int32_t open_image(const uint8_t* base, size_t len, bool mapped, fuelq_gguf** out) {
  fuelq_gguf* g = new fuelq_gguf;
  g->base = base, g->len = len, g->mapped = mapped;
  const int32_t st = guarded([&] { g->parse(); });
  if (st != FUELQ_OK) {
    delete g;
    return st;
  }
  *out = g;
  return FUELQ_OK;
}
}  // namespace

extern "C" {

int32_t fuelq_gguf_open(const char* path, fuelq_gguf** out) {
  if (!path || !out) return FUELQ_INVALID_PROBLEM;
  *out = nullptr;
  const int fd = ::open(path, O_RDONLY | O_CLOEXEC);
  if (fd < 0) {
    fuelq::set_last_error(std::string("gguf: cannot open ") + path + ": " + std::strerror(errno));
    return FUELQ_INVALID_PROBLEM;
  }
  struct stat sb;
  if (fstat(fd, &sb) != 0 || sb.st_size <= 0) {
    ::close(fd);
    fuelq::set_last_error(std::string("gguf: unexpected end of file (empty) ") + path);
    return FUELQ_INVALID_PROBLEM;
  }
  void* m = mmap(nullptr, (size_t)sb.st_size, PROT_READ, MAP_PRIVATE, fd, 0);
  ::close(fd);
  if (m == MAP_FAILED) {
    fuelq::set_last_error(std::string("gguf: cannot map ") + path + ": " + std::strerror(errno));
    return FUELQ_INVALID_PROBLEM;
  }
  const int32_t st = open_image((const uint8_t*)m, (size_t)sb.st_size, true, out);
  if (st != FUELQ_OK) munmap(m, (size_t)sb.st_size);
  return st;
}

int32_t fuelq_gguf_open_memory(const void* bytes, size_t len, fuelq_gguf** out) {
  if (!bytes || !out) return FUELQ_INVALID_PROBLEM;
  *out = nullptr;
  return open_image((const uint8_t*)bytes, len, false, out);
}

int32_t fuelq_gguf_close(fuelq_gguf* g) {
  delete g;
  return FUELQ_OK;
}

int32_t fuelq_gguf_version(const fuelq_gguf* g) { return g ? g->version : 0; }
uint64_t fuelq_gguf_alignment(const fuelq_gguf* g) { return g ? g->alignment : 0; }
uint64_t fuelq_gguf_tensor_data_offset(const fuelq_gguf* g) { return g ? g->data_offset : 0; }
int64_t fuelq_gguf_tensor_count(const fuelq_gguf* g) { return g ? (int64_t)g->tensors.size() : 0; }
int64_t fuelq_gguf_meta_count(const fuelq_gguf* g) { return g ? (int64_t)g->meta.size() : 0; }

int64_t fuelq_gguf_find_tensor(const fuelq_gguf* g, const char* name) {
  if (!g || !name) return -1;
  const auto it = g->tensor_index.find(name);
  return it == g->tensor_index.end() ? -1 : (int64_t)it->second;
}

int64_t fuelq_gguf_find_meta(const fuelq_gguf* g, const char* key) {
  if (!g || !key) return -1;
  const auto it = g->meta_index.find(key);
  return it == g->meta_index.end() ? -1 : (int64_t)it->second;
}

int32_t fuelq_gguf_tensor_at(const fuelq_gguf* g, int64_t index, fuelq_gguf_tensor* out) {
  if (!g || !out || index < 0 || index >= (int64_t)g->tensors.size()) return FUELQ_INVALID_PROBLEM;
  return guarded([&] {
    const Tensor& t = g->tensors[(size_t)index];
    out->name = t.name.c_str();
    out->ggml_type = t.ggml_type, out->n_dims = t.n_dims;
    std::memcpy(out->dims, t.dims, sizeof t.dims);
    out->offset = t.offset, out->nbytes = t.nbytes;
    out->data = nullptr;
    out->data = g->tensor_data(t);
  });
}

int32_t fuelq_gguf_meta_at(const fuelq_gguf* g, int64_t index, fuelq_gguf_value* out) {
  if (!g || !out || index < 0 || index >= (int64_t)g->meta.size()) return FUELQ_INVALID_PROBLEM;
  const Value& v = g->meta[(size_t)index];
  out->key = v.key.c_str();
  out->type = v.type, out->elem_type = v.elem_type, out->len = v.len;
  out->i = v.i, out->f = v.f, out->s = v.s, out->array = v.array;
  return FUELQ_OK;
}

int32_t fuelq_gguf_meta_array_string(const fuelq_gguf* g, int64_t index, uint64_t elem, const char** s, uint64_t* len) {
  if (!g || !s || !len || index < 0 || index >= (int64_t)g->meta.size()) return FUELQ_INVALID_PROBLEM;
  const Value& v = g->meta[(size_t)index];
  if (v.type != FUELQ_GGUF_ARRAY || v.elem_type != FUELQ_GGUF_STRING || elem >= v.strings.size()) return FUELQ_INVALID_PROBLEM;
  *s = v.strings[(size_t)elem].first, *len = v.strings[(size_t)elem].second;
  return FUELQ_OK;
}

int32_t fuelq_gguf_load_tensor(const fuelq_gguf* g, int64_t index, uint64_t byte_offset, uint64_t nbytes, void* device_dst,
                               void* stream) {
  if (!g || index < 0 || index >= (int64_t)g->tensors.size()) return FUELQ_INVALID_PROBLEM;
  return guarded([&] {
    const Tensor& t = g->tensors[(size_t)index];
    const uint8_t* src = g->tensor_data(t);
    if (byte_offset > t.nbytes || nbytes > t.nbytes - byte_offset) bad("byte range outside tensor " + t.name);
    if (nbytes == 0) return;
    if (!device_dst) bad("null destination");
    const cudaError_t e = cudaMemcpyAsync(device_dst, src + byte_offset, (size_t)nbytes, cudaMemcpyHostToDevice, (cudaStream_t)stream);
    if (e != cudaSuccess) throw Error(std::string("gguf: copy of ") + t.name + ": " + cudaGetErrorString(e), FUELQ_LAUNCH_FAILURE);
  });
}

}  // extern "C"
