// GGUF v3 reader and the bridge from a model file to resident packed matrices.
//
// Restates the parsing rules of langtax/src/gguf.rs:714-806 (`parse_gguf`): magic, version 3, signed counts,
// the thirteen metadata value types with nested arrays, `general.alignment` (default 32), one to four positive
// dimensions per tensor, the accepted / removed ggml type ids (:117-119, :165-204) with their block layouts
// (:248-283), tensor payload = blocks of the element count, payload range inside the file.  A tensor is a byte
// range of the file image (`blob_range`, :435); nothing is copied while parsing.
//
// The second half is what the crate's loader does with such ranges (langtax/src/decode.rs:476-485 `QuantMat`,
// :9612-9675 `quant_mat`, :9680-9713 `quant_mat_rows`): a 2-D weight, one expert part of a 3-D `*_exps` tensor, or a
// run of rows of either is a contiguous byte range, which goes to the device packed (llr_matrix_upload) or into a
// product with residency keyed by that range (llr_matmul_keyed): a model file is immutable, so (file, offset)
// names the bytes and a hit reads none of them.
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <atomic>
#include <cstring>
#include <string>
#include <unordered_map>
#include <vector>

#include "../../include/llama_rust_b200.h"

namespace {

struct Layout { int id; int block_bytes; int block_elems; int llr_dtype; };
// ggml type id, bytes per block, elements per block (gguf.rs:248-283, quant.rs:86-183), executor tag or -1
constexpr Layout kLayouts[] = {
    {0, 4, 1, LLR_DTYPE_F32},   {1, 2, 1, LLR_DTYPE_F16},    {30, 2, 1, LLR_DTYPE_BF16},  {2, 18, 32, LLR_DTYPE_Q4_0},
    {3, 20, 32, LLR_DTYPE_Q4_1},          {6, 22, 32, LLR_DTYPE_Q5_0}, {7, 24, 32, LLR_DTYPE_Q5_1}, {8, 34, 32, LLR_DTYPE_Q8_0},
    {9, 36, 32, -1},            {10, 84, 256, -1},           {11, 110, 256, -1},          {12, 144, 256, LLR_DTYPE_Q4_K},
    {13, 176, 256, LLR_DTYPE_Q5_K},       {14, 210, 256, LLR_DTYPE_Q6_K}, {15, 292, 256, -1},       {16, 66, 256, -1},
    {17, 74, 256, -1},          {18, 98, 256, -1},           {19, 50, 256, -1},           {20, 18, 32, -1},
    {21, 110, 256, -1},         {22, 82, 256, -1},           {23, 136, 256, -1},          {29, 56, 256, -1},
    {34, 54, 256, -1},          {35, 66, 256, -1},           {39, 17, 32, -1},            {40, 36, 64, -1},
    {41, 18, 128, -1},          {42, 18, 64, -1},
};
const Layout* layout_of(int id) {
  for (const Layout& l : kLayouts)
    if (l.id == id) return &l;
  return nullptr;
}
bool removed_type(int id) {  // gguf.rs:117-119
  return id == 4 || id == 5 || id == 31 || id == 32 || id == 33 || id == 36 || id == 37 || id == 38;
}

struct Kv {
  int type = -1;        // gguf_type of the value
  uint64_t bits = 0;    // scalars: the value's bits, zero- or sign-extended
  std::string str;      // strings
  int elem = -1;        // arrays: element type
  std::vector<Kv> items;
};

struct TensorInfo {
  std::string name;
  int ggml_type;
  uint32_t n_dims;
  uint64_t shape[4];
  uint64_t start, end;
};

std::atomic<uint64_t> g_next_file_id{1};

}  // namespace

struct llr_gguf {
  const uint8_t* bytes = nullptr;
  size_t len = 0;
  void* mapping = nullptr;  // non-null when this object owns an mmap of the file
  size_t alignment = 32;
  uint64_t file_id = 0;     // high half of the residency key of every tensor range
  std::unordered_map<std::string, Kv> kv;
  std::vector<TensorInfo> tensors;
  std::string error;
};

namespace {

struct Reader {
  const uint8_t* p;
  size_t len, pos = 0;
  int err = LLR_OK;
  int detail = 0;
  bool take(size_t n, const uint8_t** out) {
    if (n > len - pos) { err = LLR_GGUF_TRUNCATED; return false; }
    *out = p + pos;
    pos += n;
    return true;
  }
  template <typename T> bool num(T* v) {
    const uint8_t* s;
    if (!take(sizeof(T), &s)) return false;
    std::memcpy(v, s, sizeof(T));  // the format is little-endian, as is every machine this runs on
    return true;
  }
  bool str(std::string* out) {
    uint64_t n;
    if (!num(&n)) return false;
    const uint8_t* s;
    if (n > len - pos) { err = LLR_GGUF_TRUNCATED; return false; }
    if (!take((size_t)n, &s)) return false;
    if (!valid_utf8(s, (size_t)n)) { err = LLR_GGUF_UTF8; return false; }
    out->assign((const char*)s, (size_t)n);
    return true;
  }
  static bool valid_utf8(const uint8_t* s, size_t n) {
    size_t i = 0;
    while (i < n) {
      const uint8_t c = s[i];
      if (c < 0x80) { ++i; continue; }
      int extra; uint32_t cp;
      if ((c & 0xE0) == 0xC0) { extra = 1; cp = c & 0x1F; }
      else if ((c & 0xF0) == 0xE0) { extra = 2; cp = c & 0x0F; }
      else if ((c & 0xF8) == 0xF0) { extra = 3; cp = c & 0x07; }
      else return false;
      if ((size_t)extra > n - 1 - i) return false;
      for (int k = 1; k <= extra; ++k) {
        if ((s[i + k] & 0xC0) != 0x80) return false;
        cp = cp << 6 | (s[i + k] & 0x3F);
      }
      if ((extra == 1 && cp < 0x80) || (extra == 2 && cp < 0x800) || (extra == 3 && cp < 0x10000)) return false;
      if (cp > 0x10FFFF || (cp >= 0xD800 && cp <= 0xDFFF)) return false;
      i += extra + 1;
    }
    return true;
  }
  bool value(int type, Kv* out, int depth) {  // gguf.rs:925-950
    out->type = type;
    switch (type) {
      case 0: { uint8_t v; if (!num(&v)) return false; out->bits = v; return true; }
      case 1: { int8_t v; if (!num(&v)) return false; out->bits = (uint64_t)(int64_t)v; return true; }
      case 2: { uint16_t v; if (!num(&v)) return false; out->bits = v; return true; }
      case 3: { int16_t v; if (!num(&v)) return false; out->bits = (uint64_t)(int64_t)v; return true; }
      case 4: { uint32_t v; if (!num(&v)) return false; out->bits = v; return true; }
      case 5: { int32_t v; if (!num(&v)) return false; out->bits = (uint64_t)(int64_t)v; return true; }
      case 6: { uint32_t v; if (!num(&v)) return false; out->bits = v; return true; }
      case 7: { uint8_t v; if (!num(&v)) return false; out->bits = v != 0; return true; }
      case 8: return str(&out->str);
      case 9: {
        int32_t elem; uint64_t n;
        if (!num(&elem) || !num(&n)) return false;
        if (depth > 64) { err = LLR_GGUF_TRUNCATED; return false; }
        out->elem = elem;
        for (uint64_t i = 0; i < n; ++i) {
          out->items.emplace_back();
          if (!value(elem, &out->items.back(), depth + 1)) return false;
        }
        return true;
      }
      case 10: { uint64_t v; if (!num(&v)) return false; out->bits = v; return true; }
      case 11: { int64_t v; if (!num(&v)) return false; out->bits = (uint64_t)v; return true; }
      case 12: { uint64_t v; if (!num(&v)) return false; out->bits = v; return true; }
      default: err = LLR_GGUF_KV_TYPE; detail = type; return false;
    }
  }
};

int parse(llr_gguf* g) {
  Reader r{g->bytes, g->len};
  const uint8_t* magic;
  if (!r.take(4, &magic)) return r.err;
  if (std::memcmp(magic, "GGUF", 4) != 0) return LLR_GGUF_MAGIC;
  uint32_t version;
  if (!r.num(&version)) return r.err;
  if (version != 3) { g->error = "unsupported GGUF version " + std::to_string(version); return LLR_GGUF_VERSION; }
  int64_t n_tensors, n_kv;
  if (!r.num(&n_tensors) || !r.num(&n_kv)) return r.err;
  if (n_tensors < 0 || n_kv < 0) return LLR_GGUF_TRUNCATED;
  for (int64_t i = 0; i < n_kv; ++i) {
    std::string key;
    int32_t type;
    Kv v;
    if (!r.str(&key) || !r.num(&type) || !r.value(type, &v, 0)) {
      if (r.err == LLR_GGUF_KV_TYPE) g->error = "unsupported GGUF kv type " + std::to_string(r.detail);
      return r.err;
    }
    g->kv[key] = std::move(v);  // the last value of a repeated key wins
  }
  auto al = g->kv.find("general.alignment");
  if (al != g->kv.end() && al->second.type == 4 && al->second.bits > 0) g->alignment = (size_t)al->second.bits;
  struct Raw { std::string name; uint32_t n_dims; uint64_t shape[4]; int type; uint64_t offset; };
  std::vector<Raw> raw;
  for (int64_t i = 0; i < n_tensors; ++i) {
    Raw t{};
    if (!r.str(&t.name) || !r.num(&t.n_dims)) return r.err;
    if (t.n_dims == 0 || t.n_dims > 4) return LLR_GGUF_SHAPE;
    for (uint32_t d = 0; d < t.n_dims; ++d) {
      int64_t v;
      if (!r.num(&v)) return r.err;
      if (v <= 0) return LLR_GGUF_SHAPE;
      t.shape[d] = (uint64_t)v;
    }
    int32_t type;
    if (!r.num(&type)) return r.err;
    if (removed_type(type)) { g->error = "ggml-removed type " + std::to_string(type); return LLR_GGUF_REMOVED_TYPE; }
    if (!layout_of(type)) { g->error = "unsupported ggml type " + std::to_string(type); return LLR_GGUF_TYPE; }
    t.type = type;
    if (!r.num(&t.offset)) return r.err;
    raw.push_back(std::move(t));
  }
  const size_t a = g->alignment;
  if (r.pos > SIZE_MAX - a) return LLR_GGUF_TRUNCATED;
  const size_t data_start = (r.pos + a - 1) / a * a;
  for (Raw& t : raw) {
    unsigned __int128 n_el = 1;
    for (uint32_t d = 0; d < t.n_dims; ++d) {
      n_el *= t.shape[d];
      if (n_el > (unsigned __int128)UINT64_MAX) return LLR_GGUF_SHAPE;
    }
    const Layout* l = layout_of(t.type);
    if ((uint64_t)n_el % (uint64_t)l->block_elems) return LLR_GGUF_SHAPE;
    const unsigned __int128 nbytes = n_el / l->block_elems * l->block_bytes;
    const unsigned __int128 start = (unsigned __int128)data_start + t.offset;
    const unsigned __int128 end = start + nbytes;
    if (end > g->len) return LLR_GGUF_TRUNCATED;
    TensorInfo info{std::move(t.name), t.type, t.n_dims, {1, 1, 1, 1}, (uint64_t)start, (uint64_t)end};
    for (uint32_t d = 0; d < t.n_dims; ++d) info.shape[d] = t.shape[d];
    g->tensors.push_back(std::move(info));
  }
  return LLR_OK;
}

const char* code_text(int rc) {
  switch (rc) {
    case LLR_GGUF_MAGIC: return "not a GGUF file";
    case LLR_GGUF_TRUNCATED: return "truncated GGUF";
    case LLR_GGUF_UTF8: return "non-utf8 GGUF string";
    case LLR_GGUF_SHAPE: return "invalid GGUF tensor shape";
    default: return "";
  }
}

int finish_open(llr_gguf* g, llr_gguf** out) {
  const int rc = parse(g);
  if (rc != LLR_OK && g->error.empty()) g->error = code_text(rc);
  g->file_id = g_next_file_id.fetch_add(1);
  *out = g;  // also on failure, so that the caller can read the message; llr_gguf_close releases it
  return rc;
}

const TensorInfo* find(const llr_gguf* g, const char* name) {
  for (const TensorInfo& t : g->tensors)  // the first tensor of that name (gguf.rs:534-539)
    if (t.name == name) return &t;
  return nullptr;
}

void fill(const TensorInfo& t, llr_gguf_tensor* out) {
  out->name = t.name.c_str();
  out->ggml_type = t.ggml_type;
  out->dtype = layout_of(t.ggml_type)->llr_dtype;
  out->n_dims = t.n_dims;
  for (int d = 0; d < 4; ++d) out->shape[d] = t.shape[d];
  out->start = t.start;
  out->end = t.end;
  out->name_len = t.name.size();
}

// The byte range of rows [first_row, first_row + n_rows) of part `part` (decode.rs:9612-9713); n_rows 0 = all rows.
int slice_of(llr_gguf* g, const char* name, size_t part, size_t first_row, size_t n_rows, const TensorInfo** t_out,
             uint64_t* start, size_t* rows, size_t* cols, size_t* bytes) {
  const TensorInfo* t = g && name ? find(g, name) : nullptr;
  if (!t) { if (g) g->error = std::string("no tensor named ") + (name ? name : "(null)"); return LLR_ERR_INVALID; }
  const Layout* l = layout_of(t->ggml_type);
  if (l->llr_dtype < 0) { g->error = "the executor has no kernel for ggml type " + std::to_string(t->ggml_type); return LLR_ERR_DTYPE; }
  if (t->n_dims > 3) { g->error = "a weight has at most three dimensions"; return LLR_ERR_INVALID; }
  const uint64_t n_cols = t->shape[0], n_rows_all = t->n_dims > 1 ? t->shape[1] : 1, n_parts = t->n_dims > 2 ? t->shape[2] : 1;
  if (n_cols % (uint64_t)l->block_elems) { g->error = "columns are not a multiple of the block"; return LLR_ERR_UNALIGNED; }
  const uint64_t row_bytes = n_cols / l->block_elems * l->block_bytes;
  if (part >= n_parts) { g->error = "part out of range"; return LLR_ERR_INVALID; }
  if (n_rows == 0) { if (first_row != 0) { g->error = "row range out of bounds"; return LLR_ERR_INVALID; } n_rows = (size_t)n_rows_all; }
  if (first_row > n_rows_all || n_rows > n_rows_all - first_row) { g->error = "row range out of bounds"; return LLR_ERR_INVALID; }
  *t_out = t;
  *start = t->start + (part * n_rows_all + first_row) * row_bytes;
  *rows = n_rows;
  *cols = (size_t)n_cols;
  *bytes = (size_t)(n_rows * row_bytes);
  return *start + *bytes <= t->end ? LLR_OK : LLR_ERR_INVALID;
}

}  // namespace

extern "C" {

int llr_gguf_open_bytes(const void* bytes, size_t len, llr_gguf** out) {
  if (!out || (!bytes && len)) return LLR_ERR_INVALID;
  llr_gguf* g = new llr_gguf;
  g->bytes = (const uint8_t*)bytes;
  g->len = len;
  return finish_open(g, out);
}

int llr_gguf_open(const char* path, llr_gguf** out) {
  if (!out || !path) return LLR_ERR_INVALID;
  llr_gguf* g = new llr_gguf;
  const int fd = ::open(path, O_RDONLY);
  struct stat st;
  if (fd < 0 || fstat(fd, &st) != 0) {
    if (fd >= 0) ::close(fd);
    g->error = std::string("cannot open ") + path;
    *out = g;
    return LLR_ERR_INVALID;
  }
  g->len = (size_t)st.st_size;
  if (g->len) {
    void* m = mmap(nullptr, g->len, PROT_READ, MAP_PRIVATE, fd, 0);
    if (m == MAP_FAILED) { ::close(fd); g->error = std::string("cannot map ") + path; g->len = 0; *out = g; return LLR_ERR_INVALID; }
    g->mapping = m;
    g->bytes = (const uint8_t*)m;
  }
  ::close(fd);
  return finish_open(g, out);
}

void llr_gguf_close(llr_gguf* g) {
  if (!g) return;
  if (g->mapping) munmap(g->mapping, g->len);
  delete g;
}

const char* llr_gguf_last_error(const llr_gguf* g) { return g ? g->error.c_str() : ""; }

int llr_gguf_info(const llr_gguf* g, size_t* n_tensors, size_t* alignment, size_t* file_bytes) {
  if (!g) return LLR_ERR_INVALID;
  if (n_tensors) *n_tensors = g->tensors.size();
  if (alignment) *alignment = g->alignment;
  if (file_bytes) *file_bytes = g->len;
  return LLR_OK;
}

int llr_gguf_tensor_at(const llr_gguf* g, size_t index, llr_gguf_tensor* out) {
  if (!g || !out || index >= g->tensors.size()) return LLR_ERR_INVALID;
  fill(g->tensors[index], out);
  return LLR_OK;
}

int llr_gguf_find(const llr_gguf* g, const char* name, llr_gguf_tensor* out) {
  const TensorInfo* t = g && name ? find(g, name) : nullptr;
  if (!t || !out) return LLR_ERR_INVALID;
  fill(*t, out);
  return LLR_OK;
}

int llr_gguf_read(const llr_gguf* g, uint64_t start, size_t len, void* out) {
  if (!g || (!out && len) || start > g->len || len > g->len - start) return LLR_ERR_INVALID;
  if (len) std::memcpy(out, g->bytes + start, len);
  return LLR_OK;
}

// Typed metadata readers: the value must have exactly the asked type, as in gguf.rs:571-628.
int llr_gguf_kv_u32(const llr_gguf* g, const char* key, uint32_t* out) {
  if (!g || !key || !out) return LLR_ERR_INVALID;
  auto it = g->kv.find(key);
  if (it == g->kv.end() || it->second.type != 4) return LLR_ERR_INVALID;
  *out = (uint32_t)it->second.bits;
  return LLR_OK;
}

int llr_gguf_kv_f32(const llr_gguf* g, const char* key, float* out) {
  if (!g || !key || !out) return LLR_ERR_INVALID;
  auto it = g->kv.find(key);
  if (it == g->kv.end() || it->second.type != 6) return LLR_ERR_INVALID;
  const uint32_t b = (uint32_t)it->second.bits;
  std::memcpy(out, &b, 4);
  return LLR_OK;
}

int llr_gguf_kv_bool(const llr_gguf* g, const char* key, int* out) {
  if (!g || !key || !out) return LLR_ERR_INVALID;
  auto it = g->kv.find(key);
  if (it == g->kv.end() || it->second.type != 7) return LLR_ERR_INVALID;
  *out = (int)it->second.bits;
  return LLR_OK;
}

int llr_gguf_kv_string(const llr_gguf* g, const char* key, const char** out, size_t* len) {
  if (!g || !key || !out) return LLR_ERR_INVALID;
  auto it = g->kv.find(key);
  if (it == g->kv.end() || it->second.type != 8) return LLR_ERR_INVALID;
  *out = it->second.str.c_str();
  if (len) *len = it->second.str.size();
  return LLR_OK;
}

// Any scalar value as raw bits (integers sign- or zero-extended, floats as their IEEE bits) with its type.
int llr_gguf_kv_bits(const llr_gguf* g, const char* key, uint64_t* bits, int* type) {
  if (!g || !key || !bits) return LLR_ERR_INVALID;
  auto it = g->kv.find(key);
  if (it == g->kv.end() || it->second.type == 8 || it->second.type == 9) return LLR_ERR_INVALID;
  *bits = it->second.bits;
  if (type) *type = it->second.type;
  return LLR_OK;
}

int llr_gguf_kv_type(const llr_gguf* g, const char* key, int* type, int* elem_type, size_t* n_items) {
  if (!g || !key) return LLR_ERR_INVALID;
  auto it = g->kv.find(key);
  if (it == g->kv.end()) return LLR_ERR_INVALID;
  if (type) *type = it->second.type;
  if (elem_type) *elem_type = it->second.elem;
  if (n_items) *n_items = it->second.items.size();
  return LLR_OK;
}

// An array whose every element is INT32 (gguf.rs:611-628); returns the count, copies at most cap values.
int llr_gguf_kv_i32s(const llr_gguf* g, const char* key, int32_t* out, size_t cap, size_t* n) {
  if (!g || !key || !n) return LLR_ERR_INVALID;
  auto it = g->kv.find(key);
  if (it == g->kv.end() || it->second.type != 9) return LLR_ERR_INVALID;
  for (const Kv& v : it->second.items)
    if (v.type != 5) return LLR_ERR_INVALID;
  *n = it->second.items.size();
  for (size_t i = 0; i < *n && i < cap && out; ++i) out[i] = (int32_t)it->second.items[i].bits;
  return LLR_OK;
}

int llr_gguf_upload(llr_exec* exec, llr_gguf* g, const char* name, size_t part, size_t first_row, size_t n_rows,
                    llr_matrix** out) {
  const TensorInfo* t;
  uint64_t start;
  size_t rows, cols, bytes;
  const int rc = slice_of(g, name, part, first_row, n_rows, &t, &start, &rows, &cols, &bytes);
  if (rc != LLR_OK) return rc;
  return llr_matrix_upload(exec, (uint8_t)layout_of(t->ggml_type)->llr_dtype, rows, cols, g->bytes + start, bytes, out);
}

int llr_gguf_key(llr_gguf* g, const char* name, size_t part, size_t first_row, size_t n_rows, uint64_t* key_hi,
                 uint64_t* key_lo) {
  const TensorInfo* t;
  uint64_t start;
  size_t rows, cols, bytes;
  const int rc = slice_of(g, name, part, first_row, n_rows, &t, &start, &rows, &cols, &bytes);
  if (rc != LLR_OK) return rc;
  if (key_hi) *key_hi = g->file_id;
  if (key_lo) *key_lo = start;
  return LLR_OK;
}

int llr_gguf_matmul(llr_exec* exec, llr_gguf* g, const char* name, size_t part, size_t first_row, size_t n_rows,
                    size_t tokens, const float* x, size_t x_len, float* y, size_t y_len) {
  const TensorInfo* t;
  uint64_t start;
  size_t rows, cols, bytes;
  const int rc = slice_of(g, name, part, first_row, n_rows, &t, &start, &rows, &cols, &bytes);
  if (rc != LLR_OK) return rc;
  return llr_matmul_keyed(exec, g->file_id, start, (uint8_t)layout_of(t->ggml_type)->llr_dtype, rows, cols, tokens,
                          g->bytes + start, bytes, x, x_len, y, y_len);
}

}  // extern "C"
