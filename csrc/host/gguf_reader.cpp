// GGUF v3 reader: memory-maps the file, parses the header, the metadata key/values and the tensor
// directory, and hands out raw tensor payload pointers (no copies).  Little endian only.
// Block formats understood downstream: F32, F16, BF16, Q8_0 (34 B / 32 values), Q2_K (84 B / 256),
// IQ2_XXS (66 B / 256), I32.  Tensor dims are stored innermost first.
// Behavioural reference: vllm/model_executor/models/deepseek_v4_flash/gguf_reader.py:13-366.
#include <fcntl.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <new>
#include <string>
#include <vector>

namespace {

struct TensorInfo {
  std::string name;
  uint32_t n_dims;
  uint64_t dims[4];
  uint32_t type;
  uint64_t offset;   // relative to the data section
  uint64_t nbytes;
};

struct Gguf {
  int fd = -1;
  uint8_t* base = nullptr;
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
  template <typename T> T get() {
    T v{};
    if (!ok || sizeof(T) > static_cast<size_t>(end - p)) { ok = false; return v; }
    memcpy(&v, p, sizeof(T));
    p += sizeof(T);
    return v;
  }
  std::string str() {
    uint64_t n = get<uint64_t>();
    // sizes are compared, never pointers: a length near 2^64 must not wrap `p + n` past `end`
    if (!ok || n > static_cast<uint64_t>(end - p)) { ok = false; return ""; }
    std::string s(reinterpret_cast<const char*>(p), n);
    p += n;
    return s;
  }
};

void json_escape(const std::string& s, std::string& out) {
  out.push_back('"');
  for (unsigned char c : s) {
    if (c == '"' || c == '\\') { out.push_back('\\'); out.push_back(c); }
    else if (c < 0x20) { char b[8]; snprintf(b, sizeof b, "\\u%04x", c); out += b; }
    else out.push_back(c);
  }
  out.push_back('"');
}

// type ids of GGUF metadata values
enum { U8 = 0, I8, U16, I16, U32, I32, F32, BOOL, STR, ARR, U64, I64, F64 };

bool value_to_json(Cursor& c, uint32_t type, std::string& out, int depth) {
  char b[64];
  switch (type) {
    case U8: snprintf(b, sizeof b, "%u", c.get<uint8_t>()); out += b; break;
    case I8: snprintf(b, sizeof b, "%d", c.get<int8_t>()); out += b; break;
    case U16: snprintf(b, sizeof b, "%u", c.get<uint16_t>()); out += b; break;
    case I16: snprintf(b, sizeof b, "%d", c.get<int16_t>()); out += b; break;
    case U32: snprintf(b, sizeof b, "%u", c.get<uint32_t>()); out += b; break;
    case I32: snprintf(b, sizeof b, "%d", c.get<int32_t>()); out += b; break;
    case F32: snprintf(b, sizeof b, "%.9g", c.get<float>()); out += b; break;
    case BOOL: out += c.get<uint8_t>() ? "true" : "false"; break;
    case STR: json_escape(c.str(), out); break;
    case U64: snprintf(b, sizeof b, "%llu", (unsigned long long)c.get<uint64_t>()); out += b; break;
    case I64: snprintf(b, sizeof b, "%lld", (long long)c.get<int64_t>()); out += b; break;
    case F64: snprintf(b, sizeof b, "%.17g", c.get<double>()); out += b; break;
    case ARR: {
      if (depth > 2) return false;
      uint32_t et = c.get<uint32_t>();
      uint64_t n = c.get<uint64_t>();
      // long arrays (tokenizer vocabularies) are summarised, not expanded
      const bool expand = n <= 4096 && et != ARR;
      std::string tmp;
      out += expand ? "[" : "{\"__array_len__\":";
      if (!expand) { snprintf(b, sizeof b, "%llu}", (unsigned long long)n); out += b; }
      for (uint64_t i = 0; i < n && c.ok; ++i) {
        tmp.clear();
        if (!value_to_json(c, et, tmp, depth + 1)) return false;
        if (expand) { if (i) out += ","; out += tmp; }
      }
      if (expand) out += "]";
      break;
    }
    default: return false;
  }
  return c.ok;
}

uint64_t type_nbytes(uint32_t type, uint64_t n_elems) {
  switch (type) {
    case 0: return n_elems * 4;                 // F32
    case 1: return n_elems * 2;                 // F16
    case 8: return n_elems / 32 * 34;           // Q8_0
    case 10: return n_elems / 256 * 84;         // Q2_K
    case 16: return n_elems / 256 * 66;         // IQ2_XXS
    case 26: return n_elems * 4;                // I32
    case 30: return n_elems * 2;                // BF16
    case 2: return n_elems / 32 * 18;           // Q4_0
    case 12: return n_elems / 256 * 144;        // Q4_K
    case 14: return n_elems / 256 * 210;        // Q6_K
    default: return 0;
  }
}

}  // namespace

extern "C" {

static void* gguf_open_impl(const char* path, char* err, int err_cap, Gguf* g);

// The file is untrusted input: every size in it is checked with overflow-aware arithmetic and no C++
// exception (a huge length reaching std::string, a failed reserve) may cross this C boundary.
void* fi_gguf_open(const char* path, char* err, int err_cap) {
  Gguf* g = new (std::nothrow) Gguf();
  if (g == nullptr) return nullptr;
  try {
    return gguf_open_impl(path, err, err_cap, g);
  } catch (...) {
    if (err && err_cap > 0) snprintf(err, err_cap, "%s", "malformed GGUF file (allocation or length error while parsing)");
    if (g->base) munmap(g->base, g->size);
    if (g->fd >= 0) close(g->fd);
    delete g;
    return nullptr;
  }
}

static void* gguf_open_impl(const char* path, char* err, int err_cap, Gguf* g) {
  auto fail = [&](const char* msg) -> void* {
    if (err && err_cap > 0) snprintf(err, err_cap, "%s", msg);
    if (g->base) munmap(g->base, g->size);
    if (g->fd >= 0) close(g->fd);
    delete g;
    return nullptr;
  };
  g->fd = open(path, O_RDONLY);
  if (g->fd < 0) return fail("cannot open file");
  struct stat st;
  if (fstat(g->fd, &st) != 0 || st.st_size < 24) return fail("file too small for a GGUF header");
  g->size = static_cast<size_t>(st.st_size);
  g->base = static_cast<uint8_t*>(mmap(nullptr, g->size, PROT_READ, MAP_PRIVATE, g->fd, 0));
  if (g->base == MAP_FAILED) { g->base = nullptr; return fail("mmap failed"); }
  Cursor c{g->base, g->base + g->size};
  if (c.get<uint32_t>() != 0x46554747u) return fail("bad magic (not a GGUF file)");
  g->version = c.get<uint32_t>();
  if (g->version != 3) return fail("only GGUF version 3 is supported");
  const uint64_t n_tensors = c.get<uint64_t>();
  const uint64_t n_kv = c.get<uint64_t>();
  // a directory entry takes at least 32 bytes and a key/value at least 13, so the file size bounds both
  if (n_tensors > (1u << 24) || n_kv > (1u << 20) || n_tensors > g->size / 32 || n_kv > g->size / 13)
    return fail("implausible header counts");
  g->meta_json = "{";
  for (uint64_t i = 0; i < n_kv; ++i) {
    std::string key = c.str();
    uint32_t type = c.get<uint32_t>();
    if (!c.ok) return fail("truncated metadata");
    std::string val;
    const uint8_t* before = c.p;
    if (!value_to_json(c, type, val, 0)) return fail("unsupported or truncated metadata value");
    if (key == "general.alignment" && (type == U32 || type == U64)) {
      Cursor c2{before, c.end};
      g->alignment = type == U32 ? c2.get<uint32_t>() : c2.get<uint64_t>();
    }
    if (i) g->meta_json += ",";
    json_escape(key, g->meta_json);
    g->meta_json += ":";
    g->meta_json += val;
  }
  g->meta_json += "}";
  if (g->alignment == 0 || (g->alignment & (g->alignment - 1))) return fail("alignment must be a power of two");
  g->tensors.reserve(n_tensors);
  for (uint64_t i = 0; i < n_tensors; ++i) {
    TensorInfo t;
    t.name = c.str();
    t.n_dims = c.get<uint32_t>();
    if (!c.ok || t.n_dims == 0 || t.n_dims > 4) return fail("bad tensor rank");
    uint64_t n = 1;
    for (uint32_t d = 0; d < 4; ++d) t.dims[d] = 1;
    bool overflow = false;
    for (uint32_t d = 0; d < t.n_dims; ++d) {
      t.dims[d] = c.get<uint64_t>();
      overflow |= __builtin_mul_overflow(n, t.dims[d], &n);
    }
    if (overflow || n > (1ull << 48)) return fail("tensor element count overflows");
    t.type = c.get<uint32_t>();
    t.offset = c.get<uint64_t>();
    if (!c.ok) return fail("truncated tensor directory");
    t.nbytes = type_nbytes(t.type, n);
    if (t.nbytes == 0 && n != 0) return fail("unsupported tensor type");
    g->tensors.push_back(t);
  }
  const uint64_t pos = static_cast<uint64_t>(c.p - g->base);
  g->data_start = (pos + g->alignment - 1) / g->alignment * g->alignment;
  for (const auto& t : g->tensors) {
    if (t.offset % g->alignment != 0) return fail("tensor offset is not aligned");
    uint64_t end_off = 0;
    if (__builtin_add_overflow(g->data_start, t.offset, &end_off) ||
        __builtin_add_overflow(end_off, t.nbytes, &end_off) || end_off > g->size)
      return fail("tensor payload runs past the end of the file");
  }
  return g;
}

void fi_gguf_close(void* h) {
  Gguf* g = static_cast<Gguf*>(h);
  if (!g) return;
  if (g->base) munmap(g->base, g->size);
  if (g->fd >= 0) close(g->fd);
  delete g;
}

long fi_gguf_num_tensors(void* h) { return static_cast<long>(static_cast<Gguf*>(h)->tensors.size()); }
long fi_gguf_alignment(void* h) { return static_cast<long>(static_cast<Gguf*>(h)->alignment); }
long fi_gguf_meta_json_len(void* h) { return static_cast<long>(static_cast<Gguf*>(h)->meta_json.size()); }

int fi_gguf_meta_json(void* h, char* out, long cap) {
  const std::string& s = static_cast<Gguf*>(h)->meta_json;
  if (static_cast<long>(s.size()) + 1 > cap) return -1;
  memcpy(out, s.c_str(), s.size() + 1);
  return 0;
}

// dims_out: 4 values (innermost first); info_out: {n_dims, type}; sizes_out: {absolute file offset, nbytes}
int fi_gguf_tensor_info(void* h, long i, char* name_out, long name_cap, long* dims_out, int* info_out,
                        long* sizes_out) {
  Gguf* g = static_cast<Gguf*>(h);
  if (i < 0 || i >= static_cast<long>(g->tensors.size())) return -1;
  const TensorInfo& t = g->tensors[i];
  if (static_cast<long>(t.name.size()) + 1 > name_cap) return -2;
  memcpy(name_out, t.name.c_str(), t.name.size() + 1);
  for (int d = 0; d < 4; ++d) dims_out[d] = static_cast<long>(t.dims[d]);
  info_out[0] = static_cast<int>(t.n_dims);
  info_out[1] = static_cast<int>(t.type);
  sizes_out[0] = static_cast<long>(g->data_start + t.offset);
  sizes_out[1] = static_cast<long>(t.nbytes);
  return 0;
}

void* fi_gguf_base(void* h) { return static_cast<Gguf*>(h)->base; }

}  // extern "C"
