// C ABI of the matrix executor: validation, device residency of packed
// weights, host<->device staging and kernel dispatch.
//
// Plays the role of two reference components at once: the `CudaGemv` executor
// (native-cuda/src/gpu.rs:126-418: context, stream, scratch reuse, upload,
// gemv/gemm_resident) and the crate-side dispatcher `native_gpu::matmul`
// (langtax/src/native_gpu.rs:124-214: content-identity residency with a byte
// budget).  Differences by design: weights stay packed on the device (the
// reference expands to F32 on a miss), identity is a 128-bit content hash
// instead of a retained host copy of every matrix, and the budget counts
// packed bytes only.
#include <cuda_runtime.h>

#include <algorithm>
#include <cmath>
#include <cstdlib>
#include <atomic>
#include <cstring>
#include <list>
#include <memory>
#include <new>
#include <string>
#include <unordered_set>
#include <vector>

#include "../../include/llama_rust_b200.h"
#include "llr_formats.cuh"
#include "llr_kernels.cuh"

using namespace llr;

struct llr_matrix {
  llr_exec* owner;   // null once the owning executor is gone
  uint8_t* dev;
  size_t bytes;      // packed bytes (allocation is padded beyond this)
  int dtype;
  int64_t rows, cols, row_bytes;
  int f16_ok = -1;   // operand choice of the tensor-core GEMM, from the block headers at upload (-1: not examined)
};

namespace {

constexpr size_t PAD = 256;  // readable slack after the last row (16-byte copy windows)
constexpr size_t MIN_HEADROOM = 512ull << 20;  // native_gpu.rs:16

struct Hash128 {
  uint64_t a, b;
  bool operator==(const Hash128& o) const { return a == o.a && b == o.b; }
};

inline uint64_t rotl(uint64_t v, int s) { return (v << s) | (v >> (64 - s)); }
inline uint64_t fmix(uint64_t k) {
  k ^= k >> 33; k *= 0xff51afd7ed558ccdull; k ^= k >> 33; k *= 0xc4ceb9fe1a85ec53ull; k ^= k >> 33;
  return k;
}

// 128-bit content fingerprint of the packed bytes: four multiply-rotate lanes over 32-byte strides; every round folds
// each lane into its neighbour, so a change in any word reaches all four lanes (independent lanes would let two inputs
// that differ in the words of one lane collide with 64-bit strength only), then the length and a final avalanche.
Hash128 content_hash(const uint8_t* p, size_t n) {
  uint64_t l0 = 0x9E3779B97F4A7C15ull, l1 = 0xC2B2AE3D27D4EB4Full, l2 = 0x165667B19E3779F9ull,
           l3 = 0x27D4EB2F165667C5ull;
  auto round = [&](const uint64_t (&w)[4]) {
    l0 = rotl((l0 ^ w[0]) * 0x9FB21C651E98DF25ull, 29) + l3;
    l1 = rotl((l1 ^ w[1]) * 0xD6E8FEB86659FD93ull, 31) + l0;
    l2 = rotl((l2 ^ w[2]) * 0xA0761D6478BD642Full, 27) + l1;
    l3 = rotl((l3 ^ w[3]) * 0xE7037ED1A0B428DBull, 33) + l2;
  };
  size_t i = 0;
  for (; i + 32 <= n; i += 32) {
    uint64_t w[4];
    std::memcpy(w, p + i, 32);
    round(w);
  }
  if (i < n) {
    uint8_t tail[32] = {0};
    std::memcpy(tail, p + i, n - i);
    uint64_t w[4];
    std::memcpy(w, tail, 32);
    round(w);
  }
  Hash128 h;
  h.a = fmix(l0 ^ rotl(l1, 17) ^ (uint64_t)n) + fmix(l2 + 0x52DCE729ull);
  h.b = fmix(l3 ^ rotl(l2, 23) ^ ((uint64_t)n * 0x9E3779B97F4A7C15ull)) + fmix(l1 ^ l0);
  return h;
}

struct CacheEntry {
  int dtype;
  int64_t rows, cols;
  size_t len;
  Hash128 hash;   // content fingerprint, or the caller's key when keyed
  bool keyed;     // identity is a caller-supplied stable key (llr_matmul_keyed), not the content
  bool pinned;    // never evicted to make room (llr_exec_pin_key)
  llr_matrix* mat;
};

thread_local std::string g_create_error;

struct DeviceGuard {
  int prev = -1;
  explicit DeviceGuard(int dev) {
    cudaGetDevice(&prev);
    if (prev != dev) cudaSetDevice(dev);
    else prev = -1;
  }
  ~DeviceGuard() {
    if (prev >= 0) cudaSetDevice(prev);
  }
};

}  // namespace

struct llr_exec {
  int device = 0;
  int sm_count = 148;
  cudaStream_t stream = nullptr;
  std::string err;
  llr_counters ctr{};
  int path = PATH_AUTO;
  int poll_limit = 1 << 20;  // iterations a device-side wait for another CTA's or rank's data may take
  int* err_flag = nullptr;  // device alias of err_pinned: set by a kernel whose bounded wait ran out
  volatile int* err_pinned = nullptr;  // the same word, mapped pinned host memory
  struct PinSeen { const void* p; bool pinned; } pin_seen[8] = {};
  int pin_next = 0;
  // result delivery by the kernel (HostOut): completion word (mapped pinned, after the error word),
  // its device alias, a device counter of finished CTAs, the ticket of the last such launch
  volatile int* done_pinned = nullptr;
  int* done_dev = nullptr;
  unsigned int* done_count = nullptr;
  int ticket = 0;
  bool host_delivery = true;
  unsigned int* bound_dev = nullptr;  // result word of the weight range check
  unsigned int* done_count_base = nullptr;
  bool verify_hits = false;  // LLAMA_CUDA_CACHE_VERIFY: compare all bytes on a fingerprint hit
  unsigned int* bound_word() { return done_count_base + 1; }
  // activation / result staging
  float* pin_x = nullptr; size_t pin_x_cap = 0;
  float* pin_y = nullptr;
  void* pin_y_alias = nullptr;      // device alias of pin_y, valid while pin_y_alias_of == pin_y
  const float* pin_y_alias_of = nullptr; size_t pin_y_cap = 0;
  float* dev_x = nullptr; size_t dev_x_cap = 0;
  float* dev_y = nullptr; size_t dev_y_cap = 0;
  float* dev_moe = nullptr; size_t dev_moe_cap = 0;  // workspace of the routed-expert layer
  uint8_t* dev_s = nullptr; size_t dev_s_cap = 0;  // kernel scratch (bf16 activations of the tensor-core GEMM)
  // residency
  std::list<CacheEntry> cache;  // front = least recently used
  bool limit_resolved = false;
  size_t limit = 0;
  std::unordered_set<llr_matrix*> live;
};

namespace {

int fail(llr_exec* e, int code, const std::string& msg) {
  if (e) e->err = msg;
  return code;
}
int fail_cuda(llr_exec* e, cudaError_t ce, const char* what) {
  cudaGetLastError();  // clear the sticky-less error state
  const int code = ce == cudaErrorMemoryAllocation ? LLR_ERR_OOM : LLR_ERR_CUDA;
  return fail(e, code, std::string(what) + ": " + cudaGetErrorString(ce));
}

bool mul_ok(size_t a, size_t b, size_t* out) {
  if (a != 0 && b > SIZE_MAX / a) return false;
  *out = a * b;
  return true;
}

int row_bytes_checked(int dtype, size_t cols, size_t* out, std::string* msg) {
  const int be = block_elems(dtype);
  if (be == 0) {
    *msg = "unsupported dtype tag " + std::to_string(dtype) + " (no CPU fallback)";
    return LLR_ERR_DTYPE;
  }
  if (cols % (size_t)be != 0) {
    *msg = "n_cols " + std::to_string(cols) + " is not a multiple of the block width " +
           std::to_string(be);
    return LLR_ERR_UNALIGNED;
  }
  if (!mul_ok(cols / (size_t)be, (size_t)block_bytes(dtype), out)) {
    *msg = "weight shape overflow";
    return LLR_ERR_OVERFLOW;
  }
  return LLR_OK;
}

template <class T>
cudaError_t grow_pinned(T** p, size_t* cap, size_t need) {
  if (need <= *cap) return cudaSuccess;
  size_t ncap = *cap ? *cap : 4096;
  while (ncap < need) ncap *= 2;
  T* np_ = nullptr;
  cudaError_t ce = cudaMallocHost((void**)&np_, ncap * sizeof(T));
  if (ce != cudaSuccess) return ce;
  if (*p) cudaFreeHost(*p);
  *p = np_;
  *cap = ncap;
  return cudaSuccess;
}

template <class T>
cudaError_t grow_device(T** p, size_t* cap, size_t need) {
  if (need <= *cap) return cudaSuccess;
  size_t ncap = *cap ? *cap : 4096;
  while (ncap < need) ncap *= 2;
  T* np_ = nullptr;
  cudaError_t ce = cudaMalloc((void**)&np_, ncap * sizeof(T));
  if (ce != cudaSuccess) return ce;
  if (*p) cudaFree(*p);
  *p = np_;
  *cap = ncap;
  return cudaSuccess;
}

void drop_entry(llr_exec* e, std::list<CacheEntry>::iterator it) {
  e->ctr.resident_bytes -= it->len;
  ++e->ctr.evictions;
  llr_matrix* m = it->mat;
  e->cache.erase(it);
  e->live.erase(m);
  cudaFree(m->dev);
  delete m;
}

void drop_all_cached(llr_exec* e) {
  while (!e->cache.empty()) drop_entry(e, e->cache.begin());
}

// LLAMA_CUDA_CACHE_BYTES, native_gpu.rs:19-54
int resolve_limit(llr_exec* e) {
  if (e->limit_resolved) return LLR_OK;
  const char* v = std::getenv("LLAMA_CUDA_CACHE_BYTES");
  if (v && std::strcmp(v, "auto") != 0) {
    const size_t n = std::strlen(v);
    bool digits = n > 0;
    for (size_t i = 0; i < n; ++i) digits = digits && v[i] >= '0' && v[i] <= '9';
    if (!digits)
      return fail(e, LLR_ERR_CONFIG,
                  "LLAMA_CUDA_CACHE_BYTES must be auto or a nonnegative decimal byte count");
    size_t acc = 0;
    for (size_t i = 0; i < n; ++i) {
      const size_t dg = (size_t)(v[i] - '0');
      if (acc > (SIZE_MAX - dg) / 10)
        return fail(e, LLR_ERR_CONFIG, "LLAMA_CUDA_CACHE_BYTES exceeds addressable memory");
      acc = acc * 10 + dg;
    }
    e->limit = acc;
  } else {
    size_t fr = 0, tot = 0;
    cudaError_t ce = cudaMemGetInfo(&fr, &tot);
    if (ce != cudaSuccess) return fail_cuda(e, ce, "cudaMemGetInfo");
    const size_t avail = fr < tot ? fr : tot;  // native_gpu.rs:34-40
    const size_t reserve = avail / 4 > MIN_HEADROOM ? avail / 4 : MIN_HEADROOM;
    e->limit = avail > reserve ? avail - reserve : 0;
  }
  e->limit_resolved = true;
  e->ctr.cache_limit = e->limit;
  return LLR_OK;
}

int alloc_matrix(llr_exec* e, int dtype, size_t rows, size_t cols, size_t rb, size_t bytes,
                 llr_matrix** out) {
  uint8_t* dev = nullptr;
  cudaError_t ce = cudaMalloc((void**)&dev, bytes + PAD);
  if (ce == cudaErrorMemoryAllocation) {
    // cached weights must never keep an otherwise viable matrix from fitting (gpu.rs:198-210)
    cudaGetLastError();
    drop_all_cached(e);
    ce = cudaMalloc((void**)&dev, bytes + PAD);
  }
  if (ce != cudaSuccess) return fail_cuda(e, ce, "device allocation for packed weights");
  ce = cudaMemsetAsync(dev + bytes, 0, PAD, e->stream);
  if (ce != cudaSuccess) { cudaFree(dev); return fail_cuda(e, ce, "cudaMemsetAsync"); }
  llr_matrix* m = new (std::nothrow) llr_matrix{e, dev, bytes, dtype, (int64_t)rows, (int64_t)cols,
                                                (int64_t)rb};
  if (!m) { cudaFree(dev); return fail(e, LLR_ERR_OOM, "host allocation failed"); }
  e->live.insert(m);
  *out = m;
  return LLR_OK;
}

void release_matrix(llr_exec* e, llr_matrix* m) {
  e->live.erase(m);
  cudaFree(m->dev);
  delete m;
}

int check_matrix(llr_exec* e, const llr_matrix* m) {
  if (!m) return fail(e, LLR_ERR_INVALID, "null matrix");
  if (m->owner != e) return fail(e, LLR_ERR_FOREIGN, "CUDA matrix belongs to a different executor");
  return LLR_OK;
}

MatView view_of(const llr_matrix* m) {
  return MatView{m->dev, m->dtype, m->rows, m->cols, m->row_bytes, m->f16_ok};
}

// scratch for the tensor-core GEMM; growing frees the old buffer, which synchronizes the device
cudaError_t ensure_scratch(llr_exec* e, const llr_matrix* m, size_t tokens, void** out) {
  *out = nullptr;
  const MatView v = view_of(m);
  if (!matmul_wants_tc(v, (int64_t)tokens, e->path)) return cudaSuccess;
  cudaError_t ce = grow_device(&e->dev_s, &e->dev_s_cap, gemm_tc_scratch_bytes(v, (int64_t)tokens));
  if (ce == cudaSuccess) *out = e->dev_s;
  return ce;
}

// Is p pinned host memory, and where can kernels of this device address it?  Asked of the driver on
// every call: the answer decides whether a kernel stores through the alias, and a remembered
// answer for memory that has since been freed would turn into a wild store.
bool pinned_alias(const void* p, void** alias) {
  cudaPointerAttributes a{};
  *alias = nullptr;
  if (cudaPointerGetAttributes(&a, p) != cudaSuccess) { cudaGetLastError(); return false; }
  if (a.type != cudaMemoryTypeHost) return false;
  *alias = a.devicePointer;
  return true;
}

// Same question for buffers that are only copied from or to.  Remembers the answer for the last few
// pointers: callers reuse their buffers, and a stale answer is harmless here (a pageable buffer taken
// for pinned is still copied correctly, only slower; a pinned one taken for pageable goes through
// the staging buffer).
bool is_pinned_host(llr_exec* e, const void* p) {
  for (const auto& s : e->pin_seen)
    if (s.p == p) return s.pinned;
  void* unused = nullptr;
  const bool pinned = pinned_alias(p, &unused);
  e->pin_seen[e->pin_next] = {p, pinned};
  e->pin_next = (e->pin_next + 1) % 8;
  return pinned;
}

// after a synchronize: non-zero when a device-side wait gave up since the last check
int take_device_error(llr_exec* e) {
  const int v = *e->err_pinned;
  if (v != 0) *e->err_pinned = 0;
  return v;
}

// Tensor-core GEMM operand choice for a freshly filled matrix: enqueues the header scan; the caller
// synchronizes the stream anyway and then calls finish_range_check.
cudaError_t begin_range_check(llr_exec* e, llr_matrix* m, unsigned int* host_word) {
  const MatView v = view_of(m);
  if (!gemm_tc_supported(v, 64) || !e->bound_dev) return cudaSuccess;
  cudaError_t ce = launch_weight_bound(v, e->bound_dev, e->stream, &e->ctr.launches);
  if (ce == cudaSuccess) ce = cudaMemcpyAsync(host_word, e->bound_dev, sizeof(unsigned int), cudaMemcpyDeviceToHost, e->stream);
  return ce;
}
void finish_range_check(llr_matrix* m, unsigned int host_word, bool examined) {
  if (examined) m->f16_ok = weight_bound_allows_f16(host_word) ? 1 : 0;
}

// H2D of the activations, launch, D2H of the result, synchronize (gpu.rs:301-334,
// 381-416).  `y` is written only after everything succeeded.
int run_host(llr_exec* e, const llr_matrix* m, size_t tokens, const float* x, float* y) {
  const size_t nx = tokens * (size_t)m->cols, ny = tokens * (size_t)m->rows;
  cudaError_t ce;
  if ((ce = grow_device(&e->dev_x, &e->dev_x_cap, nx)) != cudaSuccess) return fail_cuda(e, ce, "activation scratch");
  if ((ce = grow_device(&e->dev_y, &e->dev_y_cap, ny)) != cudaSuccess) return fail_cuda(e, ce, "result scratch");
  const float* src = x;
  if (!is_pinned_host(e, x)) {
    if ((ce = grow_pinned(&e->pin_x, &e->pin_x_cap, nx)) != cudaSuccess) return fail_cuda(e, ce, "pinned activation staging");
    std::memcpy(e->pin_x, x, nx * sizeof(float));
    src = e->pin_x;
  }
  void* y_alias = nullptr;
  const bool y_pinned = pinned_alias(y, &y_alias);
  float* dst = y;
  if (!y_pinned) {
    if ((ce = grow_pinned(&e->pin_y, &e->pin_y_cap, ny)) != cudaSuccess) return fail_cuda(e, ce, "pinned result staging");
    dst = e->pin_y;
    if (e->pin_y_alias_of != e->pin_y) {  // the staging buffer moved (it grows in several entry points)
      void* a = nullptr;
      e->pin_y_alias = cudaHostGetDevicePointer(&a, e->pin_y, 0) == cudaSuccess ? a : nullptr;
      if (!e->pin_y_alias) cudaGetLastError();
      e->pin_y_alias_of = e->pin_y;
    }
    y_alias = e->pin_y_alias;
  }
  void* scratch = nullptr;
  if ((ce = ensure_scratch(e, m, tokens, &scratch)) != cudaSuccess) return fail_cuda(e, ce, "kernel scratch");
  if ((ce = cudaMemcpyAsync(e->dev_x, src, nx * sizeof(float), cudaMemcpyHostToDevice, e->stream)) != cudaSuccess)
    return fail_cuda(e, ce, "activation upload");
  const MatView v = view_of(m);
  // Decode-sized calls on the streaming kernel: the kernel stores the result into the host buffer and
  // raises a completion word that this thread polls: no device-to-host copy, no stream synchronize.
  const bool deliver = e->host_delivery && y_alias && !scratch && (e->path == PATH_AUTO || e->path == PATH_MMA) &&
                       gemv_mma_hostout_ok(v, (int64_t)tokens);
  if (deliver) {
    const int ticket = ++e->ticket;
    HostOut ho{(long long)((char*)y_alias - (char*)e->dev_y), e->done_dev, e->done_count, ticket};
    if ((ce = launch_gemv_mma_hostout(v, e->dev_x, e->dev_y, (int64_t)tokens, ho, e->stream, e->sm_count, e->err_flag,
                                      &e->ctr.launches)) != cudaSuccess)
      return fail_cuda(e, ce, "kernel launch");
    bool done = false;
    for (uint64_t spins = 1; !done; ++spins) {
      if (*e->done_pinned == ticket) { done = true; break; }
      if ((spins & 4095) == 0) {  // a kernel that failed or was never run must not hang the caller
        const cudaError_t q = cudaStreamQuery(e->stream);
        if (q == cudaErrorNotReady) continue;
        if (q != cudaSuccess) return fail_cuda(e, q, "kernel execution");
        done = *e->done_pinned == ticket;
        break;
      }
    }
    std::atomic_thread_fence(std::memory_order_acquire);
    if (!done) return fail(e, LLR_ERR_CUDA, "the kernel finished without delivering its result");
  } else {
    if ((ce = launch_matmul(v, e->dev_x, e->dev_y, (int64_t)tokens, e->stream, e->path,
                            e->sm_count, e->err_flag, scratch, &e->ctr.launches)) != cudaSuccess)
      return fail_cuda(e, ce, "kernel launch");
    if ((ce = cudaMemcpyAsync(dst, e->dev_y, ny * sizeof(float), cudaMemcpyDeviceToHost, e->stream)) != cudaSuccess)
      return fail_cuda(e, ce, "result download");
    if ((ce = cudaStreamSynchronize(e->stream)) != cudaSuccess) return fail_cuda(e, ce, "stream synchronize");
  }
  if (take_device_error(e) != 0) {
    return fail(e, LLR_ERR_CUDA, "a device-side wait ran out of iterations (copy engine did not deliver a weight tile)");
  }
  if (!y_pinned) std::memcpy(y, e->pin_y, ny * sizeof(float));
  e->ctr.h2d_bytes += nx * sizeof(float);
  e->ctr.d2h_bytes += ny * sizeof(float);
  return LLR_OK;
}

}  // namespace

namespace llr {

bool matmul_wants_tc(const MatView& m, int64_t tokens, int path) {
  if (path == PATH_TC) return gemm_tc_supported(m, tokens);
  return path == PATH_AUTO && tokens >= TC_MIN_TOKENS && gemm_tc_supported(m, tokens);
}

cudaError_t launch_matmul(const MatView& m, const float* x, float* y, int64_t tokens,
                          cudaStream_t stream, int path, int sm_count, int* err_flag,
                          void* scratch, uint64_t* launches) {
  const bool x_aligned = ((uintptr_t)x & 15) == 0 && (m.cols % 4 == 0);
  if (scratch && err_flag && x_aligned && matmul_wants_tc(m, tokens, path))
    return launch_gemm_tc(m, x, y, tokens, scratch, gemm_tc_scratch_bytes(m, tokens), stream, err_flag, launches);
  if (path == PATH_TC) path = PATH_AUTO;
  if ((path == PATH_AUTO || path == PATH_MMA) && x_aligned && err_flag && gemv_mma_supported(m))
    return launch_gemv_mma(m, x, y, tokens, stream, sm_count, err_flag, launches);
  if (path == PATH_AUTO && x_aligned && gemv_rows_supported(m) && tokens <= 32)
    return launch_gemv_rows(m, x, y, tokens, stream, sm_count, launches);
  if (path != PATH_GENERIC && x_aligned && gemv_staged_supported(m))
    return launch_gemv_staged(m, x, y, tokens, stream, sm_count, launches);
  return launch_gemv_generic(m, x, y, tokens, stream, launches);
}

}  // namespace llr

extern "C" {

int llr_exec_create(int device, llr_exec** out) {
  if (!out) { g_create_error = "null output pointer"; return LLR_ERR_INVALID; }
  *out = nullptr;
  int n = 0;
  cudaError_t ce = cudaGetDeviceCount(&n);
  if (ce != cudaSuccess) {
    cudaGetLastError();
    g_create_error = std::string("no usable CUDA device: ") + cudaGetErrorString(ce);
    return LLR_ERR_CUDA;
  }
  if (device < 0 || device >= n) {
    g_create_error = "device ordinal " + std::to_string(device) + " out of range";
    return LLR_ERR_INVALID;
  }
  DeviceGuard guard(device);
  llr_exec* e = new (std::nothrow) llr_exec();
  if (!e) { g_create_error = "host allocation failed"; return LLR_ERR_OOM; }
  e->device = device;
  cudaDeviceProp prop{};
  if ((ce = cudaGetDeviceProperties(&prop, device)) != cudaSuccess ||
      (ce = cudaStreamCreateWithFlags(&e->stream, cudaStreamNonBlocking)) != cudaSuccess) {
    cudaGetLastError();
    g_create_error = std::string("CUDA initialisation failed: ") + cudaGetErrorString(ce);
    delete e;
    return LLR_ERR_CUDA;
  }
  if (prop.major < 10) {
    g_create_error = std::string("device ") + prop.name + " is sm_" + std::to_string(prop.major) +
                     std::to_string(prop.minor) + "; this library is built for sm_100a only";
    cudaStreamDestroy(e->stream);
    delete e;
    return LLR_ERR_CUDA;
  }
  e->sm_count = prop.multiProcessorCount;
  void* err_host = nullptr;
  if ((ce = cudaHostAlloc(&err_host, 2 * sizeof(int), cudaHostAllocMapped)) == cudaSuccess) {
    ((int*)err_host)[0] = ((int*)err_host)[1] = 0;
    e->err_pinned = (volatile int*)err_host;
    e->done_pinned = (volatile int*)err_host + 1;
    ce = cudaHostGetDevicePointer((void**)&e->err_flag, err_host, 0);
    e->done_dev = e->err_flag + 1;
  }
  if (ce == cudaSuccess && (ce = cudaMalloc((void**)&e->done_count, 2 * sizeof(unsigned int))) == cudaSuccess) {
    ce = cudaMemset(e->done_count, 0, 2 * sizeof(unsigned int));
    e->bound_dev = e->done_count + 1;
    e->done_count_base = e->done_count;
  }
  if (const char* bf = std::getenv("LLR_GEMM_BF16")) { if (std::strcmp(bf, "0") != 0) e->bound_dev = nullptr; }  // keep bfloat16 operands
  if (const char* vh = std::getenv("LLAMA_CUDA_CACHE_VERIFY")) e->verify_hits = std::strcmp(vh, "0") != 0;
  if (const char* hd = std::getenv("LLR_HOST_DELIVERY")) e->host_delivery = std::strcmp(hd, "0") != 0;
  if (ce != cudaSuccess) {
    if (err_host) cudaFreeHost(err_host);
    cudaGetLastError();
    g_create_error = std::string("CUDA initialisation failed: ") + cudaGetErrorString(ce);
    cudaStreamDestroy(e->stream);
    delete e;
    return LLR_ERR_CUDA;
  }
  if (const char* p = std::getenv("LLR_GEMV_PATH")) {
    if (!std::strcmp(p, "generic")) e->path = PATH_GENERIC;
    else if (!std::strcmp(p, "staged")) e->path = PATH_STAGED;
    else if (!std::strcmp(p, "mma")) e->path = PATH_MMA;
    else if (!std::strcmp(p, "tc")) e->path = PATH_TC;
  }
  *out = e;
  return LLR_OK;
}

int llr_exec_destroy(llr_exec* e) {
  if (!e) return LLR_OK;
  DeviceGuard guard(e->device);
  cudaStreamSynchronize(e->stream);
  drop_all_cached(e);
  for (llr_matrix* m : e->live) {  // handles the caller still holds: free the device side
    cudaFree(m->dev);
    m->dev = nullptr;
    m->owner = nullptr;
  }
  if (e->pin_x) cudaFreeHost(e->pin_x);
  if (e->pin_y) cudaFreeHost(e->pin_y);
  if (e->dev_x) cudaFree(e->dev_x);
  if (e->dev_y) cudaFree(e->dev_y);
  if (e->dev_s) cudaFree(e->dev_s);
  if (e->dev_moe) cudaFree(e->dev_moe);
  if (e->err_pinned) cudaFreeHost((void*)e->err_pinned);
  if (e->done_count) cudaFree(e->done_count);
  cudaStreamDestroy(e->stream);
  cudaGetLastError();
  delete e;
  return LLR_OK;
}

int llr_exec_mem_info(llr_exec* e, size_t* free_bytes, size_t* total_bytes) {
  if (!e || !free_bytes || !total_bytes) return fail(e, LLR_ERR_INVALID, "null argument");
  DeviceGuard guard(e->device);
  cudaError_t ce = cudaMemGetInfo(free_bytes, total_bytes);
  if (ce != cudaSuccess) return fail_cuda(e, ce, "cudaMemGetInfo");
  return LLR_OK;
}

const char* llr_exec_last_error(const llr_exec* e) { return e ? e->err.c_str() : g_create_error.c_str(); }

int llr_exec_counters(const llr_exec* e, llr_counters* out) {
  if (!e || !out) return LLR_ERR_INVALID;
  *out = e->ctr;
  return LLR_OK;
}

int llr_exec_set_path(llr_exec* e, int path) {
  if (!e || path < PATH_AUTO || path > PATH_TC) return LLR_ERR_INVALID;
  e->path = path;
  return LLR_OK;
}

int llr_row_bytes(uint8_t dtype, size_t cols, size_t* out) {
  if (!out) return LLR_ERR_INVALID;
  std::string msg;
  return row_bytes_checked(dtype, cols, out, &msg);
}

static int upload_common(llr_exec* e, uint8_t dtype, size_t rows, size_t cols, const void* packed,
                         size_t packed_len, bool from_device, llr_matrix** out) {
  if (!e) return LLR_ERR_INVALID;
  if (!out) return fail(e, LLR_ERR_INVALID, "null output pointer");
  *out = nullptr;
  if (rows == 0 || cols == 0) return fail(e, LLR_ERR_INVALID, "GEMV dimensions must be positive");
  size_t rb = 0, expect = 0;
  std::string msg;
  int rc = row_bytes_checked(dtype, cols, &rb, &msg);
  if (rc) return fail(e, rc, msg);
  if (!mul_ok(rb, rows, &expect)) return fail(e, LLR_ERR_OVERFLOW, "GEMV shape overflow");
  if (packed_len != expect || !packed)
    return fail(e, LLR_ERR_INVALID, "GEMV buffer lengths do not match shape");
  DeviceGuard guard(e->device);
  llr_matrix* m = nullptr;
  if ((rc = alloc_matrix(e, dtype, rows, cols, rb, expect, &m)) != LLR_OK) return rc;
  cudaError_t ce = cudaMemcpyAsync(m->dev, packed, expect,
                                   from_device ? cudaMemcpyDeviceToDevice : cudaMemcpyHostToDevice,
                                   e->stream);
  unsigned int bound = 0;
  const bool examine = gemm_tc_supported(view_of(m), 64) && e->bound_dev != nullptr;
  if (ce == cudaSuccess) ce = begin_range_check(e, m, &bound);
  if (ce == cudaSuccess) ce = cudaStreamSynchronize(e->stream);
  if (ce != cudaSuccess) { release_matrix(e, m); return fail_cuda(e, ce, "weight upload"); }
  finish_range_check(m, bound, examine);
  ++e->ctr.uploads;
  e->ctr.upload_bytes += expect;
  *out = m;
  return LLR_OK;
}

int llr_matrix_upload(llr_exec* e, uint8_t dtype, size_t rows, size_t cols, const void* packed,
                      size_t packed_len, llr_matrix** out) {
  return upload_common(e, dtype, rows, cols, packed, packed_len, false, out);
}

int llr_matrix_upload_device(llr_exec* e, uint8_t dtype, size_t rows, size_t cols,
                             const void* packed_dev, size_t packed_len, llr_matrix** out) {
  return upload_common(e, dtype, rows, cols, packed_dev, packed_len, true, out);
}

int llr_matrix_free(llr_matrix* m) {
  if (!m) return LLR_OK;
  if (m->owner) {
    DeviceGuard guard(m->owner->device);
    cudaStreamSynchronize(m->owner->stream);
    release_matrix(m->owner, m);
  } else {
    delete m;
  }
  return LLR_OK;
}

int llr_matrix_info(const llr_matrix* m, uint8_t* dtype, size_t* rows, size_t* cols,
                    size_t* packed_bytes) {
  if (!m) return LLR_ERR_INVALID;
  if (dtype) *dtype = (uint8_t)m->dtype;
  if (rows) *rows = (size_t)m->rows;
  if (cols) *cols = (size_t)m->cols;
  if (packed_bytes) *packed_bytes = m->bytes;
  return LLR_OK;
}

int llr_gemm_resident(llr_exec* e, const llr_matrix* m, size_t tokens, const float* x, size_t x_len,
                      float* y, size_t y_len) {
  if (!e) return LLR_ERR_INVALID;
  int rc = check_matrix(e, m);
  if (rc) return rc;
  size_t nx = 0, ny = 0;
  if (!mul_ok(tokens, (size_t)m->cols, &nx)) return fail(e, LLR_ERR_OVERFLOW, "CUDA GEMM input shape overflow");
  if (!mul_ok(tokens, (size_t)m->rows, &ny)) return fail(e, LLR_ERR_OVERFLOW, "CUDA GEMM output shape overflow");
  if (tokens == 0 || x_len != nx || y_len != ny || !x || !y)
    return fail(e, LLR_ERR_INVALID, "CUDA GEMM buffer lengths do not match shape");
  DeviceGuard guard(e->device);
  return run_host(e, m, tokens, x, y);
}

int llr_gemv_resident(llr_exec* e, const llr_matrix* m, const float* x, size_t x_len, float* y,
                      size_t y_len) {
  if (!e) return LLR_ERR_INVALID;
  int rc = check_matrix(e, m);
  if (rc) return rc;
  if (x_len != (size_t)m->cols || y_len != (size_t)m->rows || !x || !y)
    return fail(e, LLR_ERR_INVALID, "CUDA GEMV vector lengths do not match resident matrix");
  DeviceGuard guard(e->device);
  return run_host(e, m, 1, x, y);
}

static int matmul_cached(llr_exec* e, const Hash128* key, uint8_t dtype, size_t rows, size_t cols, size_t tokens,
                         const void* packed, size_t packed_len, const float* x, size_t x_len, float* y, size_t y_len) {
  if (!e) return LLR_ERR_INVALID;
  // native_matmul, quant.rs:6698-6745
  if (tokens == 0 || cols == 0 || y_len % tokens != 0)
    return fail(e, LLR_ERR_INVALID, "matrix dimensions must be positive and token-aligned");
  size_t nx = 0;
  if (!mul_ok(tokens, cols, &nx)) return fail(e, LLR_ERR_OVERFLOW, "input shape overflow");
  if (x_len != nx)
    return fail(e, LLR_ERR_INVALID, "X F32 elems: expected " + std::to_string(nx) + ", got " + std::to_string(x_len));
  if (y_len / tokens != rows)
    return fail(e, LLR_ERR_INVALID, "Y F32 elems do not match rows x tokens");
  size_t rb = 0, expect = 0;
  std::string msg;
  int rc = row_bytes_checked(dtype, cols, &rb, &msg);
  if (rc) return fail(e, rc, msg);
  if (!mul_ok(rb, rows, &expect)) return fail(e, LLR_ERR_OVERFLOW, "weight shape overflow");
  if (packed_len != expect)
    return fail(e, LLR_ERR_INVALID, "W bytes: expected " + std::to_string(expect) + ", got " + std::to_string(packed_len));
  if (rows == 0) return LLR_OK;
  if (!packed || !x || !y) return fail(e, LLR_ERR_INVALID, "null buffer");

  DeviceGuard guard(e->device);
  if ((rc = resolve_limit(e)) != LLR_OK) return rc;

  // Identity: the caller's stable key when given (immutable model weights: nothing is read but the key), else a
  // 128-bit fingerprint of all packed bytes.  The reference compares every byte on a hit (native_gpu.rs:96-98);
  // LLAMA_CUDA_CACHE_VERIFY=1 restores that guarantee for fingerprint hits: the caller's bytes are uploaded beside the
  // resident copy and compared on the device, and a difference is treated as a miss.
  const bool keyed = key != nullptr;
  const Hash128 h = keyed ? *key : content_hash((const uint8_t*)packed, packed_len);
  for (auto it = e->cache.begin(); it != e->cache.end(); ++it) {
    if (it->keyed == keyed && it->dtype == dtype && it->rows == (int64_t)rows && it->cols == (int64_t)cols &&
        it->len == packed_len && it->hash == h) {
      if (!keyed && e->verify_hits) {
        int differ = 0;
        cudaError_t ve = grow_device(&e->dev_s, &e->dev_s_cap, packed_len + 256);
        if (ve == cudaSuccess) ve = cudaMemcpyAsync(e->dev_s, packed, packed_len, cudaMemcpyHostToDevice, e->stream);
        if (ve == cudaSuccess) ve = launch_bytes_differ(e->dev_s, it->mat->dev, packed_len, (int*)e->bound_word(), e->stream, &e->ctr.launches);
        if (ve == cudaSuccess) ve = cudaMemcpyAsync(&differ, e->bound_word(), sizeof(int), cudaMemcpyDeviceToHost, e->stream);
        if (ve == cudaSuccess) ve = cudaStreamSynchronize(e->stream);
        if (ve != cudaSuccess) return fail_cuda(e, ve, "residency verification");
        if (differ) { drop_entry(e, it); break; }  // a fingerprint collision: the resident copy is not this matrix
      }
      e->cache.splice(e->cache.end(), e->cache, it);  // most recently used
      ++e->ctr.cache_hits;
      return run_host(e, e->cache.back().mat, tokens, x, y);
    }
  }
  ++e->ctr.cache_misses;
  // native_gpu.rs:42-44, 178-185: evict the oldest entries (pinned ones stay) until the newcomer fits
  for (auto it = e->cache.begin(); it != e->cache.end() && (expect > e->limit || e->ctr.resident_bytes > e->limit - expect);) {
    if (it->pinned) { ++it; continue; }
    auto victim = it++;
    drop_entry(e, victim);
  }
  llr_matrix* m = nullptr;
  if ((rc = alloc_matrix(e, dtype, rows, cols, rb, expect, &m)) != LLR_OK) return rc;
  cudaError_t ce = cudaMemcpyAsync(m->dev, packed, expect, cudaMemcpyHostToDevice, e->stream);
  // Operand choice of the tensor-core GEMM, as llr_matrix_upload makes it: a scan of the block headers behind
  // the upload.  Without it every product that arrives here with 64 or more activation rows would take the
  // bfloat16 operands (8 significant bits) although the weights fit binary16 (11 bits).  The scan's answer is
  // needed only when this very call runs the GEMM; otherwise it is collected without an extra wait: the
  // host-pointer product below synchronizes with the stream before it returns.
  unsigned int bound = 0;
  const bool examine = gemm_tc_supported(view_of(m), 64) && e->bound_dev != nullptr;
  if (ce == cudaSuccess) ce = begin_range_check(e, m, &bound);
  if (ce == cudaSuccess && examine && matmul_wants_tc(view_of(m), (int64_t)tokens, e->path)) {
    ce = cudaStreamSynchronize(e->stream);
    if (ce == cudaSuccess) finish_range_check(m, bound, true);
  }
  if (ce != cudaSuccess) { cudaStreamSynchronize(e->stream); release_matrix(e, m); return fail_cuda(e, ce, "weight upload"); }
  ++e->ctr.uploads;
  e->ctr.upload_bytes += expect;
  rc = run_host(e, m, tokens, x, y);
  if (rc == LLR_OK && examine && m->f16_ok < 0) {
    cudaStreamSynchronize(e->stream);  // decode-sized calls return on a completion word, not on the stream
    finish_range_check(m, bound, true);
  }
  if (rc != LLR_OK) { cudaStreamSynchronize(e->stream); cudaGetLastError(); release_matrix(e, m); return rc; }
  // matrices that do not fit the budget (beside what is pinned) run once and are released (native_gpu.rs:199-211)
  if (expect <= e->limit && e->ctr.resident_bytes <= e->limit - expect) {
    e->cache.push_back(CacheEntry{dtype, (int64_t)rows, (int64_t)cols, packed_len, h, keyed, false, m});
    e->ctr.resident_bytes += expect;
  } else {
    release_matrix(e, m);
  }
  return LLR_OK;
}

int llr_matmul(llr_exec* e, uint8_t dtype, size_t rows, size_t cols, size_t tokens, const void* packed, size_t packed_len,
               const float* x, size_t x_len, float* y, size_t y_len) {
  return matmul_cached(e, nullptr, dtype, rows, cols, tokens, packed, packed_len, x, x_len, y, y_len);
}

int llr_matmul_keyed(llr_exec* e, uint64_t key_hi, uint64_t key_lo, uint8_t dtype, size_t rows, size_t cols, size_t tokens,
                     const void* packed, size_t packed_len, const float* x, size_t x_len, float* y, size_t y_len) {
  const Hash128 key{key_hi, key_lo};
  return matmul_cached(e, &key, dtype, rows, cols, tokens, packed, packed_len, x, x_len, y, y_len);
}

int llr_exec_pin_key(llr_exec* e, uint64_t key_hi, uint64_t key_lo, int pinned) {
  if (!e) return LLR_ERR_INVALID;
  const Hash128 key{key_hi, key_lo};
  bool found = false;
  for (auto& ent : e->cache)
    if (ent.keyed && ent.hash == key) { ent.pinned = pinned != 0; found = true; }
  if (!found) return fail(e, LLR_ERR_INVALID, "no resident matrix carries this key");
  return LLR_OK;
}

// plan_placement (expertvm/src/planner.rs:332-349): move the expert's weights once, or ship activations on every use.
int llr_plan_placement(uint64_t expert_bytes, uint64_t activation_bytes, uint64_t fan_in, uint64_t reuse, uint64_t link_bps) {
  // nanoseconds to carry bytes at bps, floored, saturating at 2^64-1 (gpu-sim/src/profile.rs:718-727)
  auto ns_for_bytes = [](uint64_t bytes, uint64_t bps) -> uint64_t {
    if (bps == 0) return UINT64_MAX;
    const unsigned __int128 n = (unsigned __int128)bytes * 1000000000ull / bps;
    return n > (unsigned __int128)UINT64_MAX ? UINT64_MAX : (uint64_t)n;
  };
  auto sat_mul = [](uint64_t a, uint64_t b) { return a != 0 && b > UINT64_MAX / a ? UINT64_MAX : a * b; };
  const uint64_t dispatch = sat_mul(sat_mul(activation_bytes, fan_in ? fan_in : 1), reuse ? reuse : 1);
  return ns_for_bytes(expert_bytes, link_bps) <= ns_for_bytes(dispatch, link_bps) ? LLR_PLACE_MOVE_WEIGHTS : LLR_PLACE_DISPATCH_ACTIVATIONS;
}

int llr_matmul_device(llr_exec* e, const llr_matrix* m, size_t tokens, const float* x_dev,
                      float* y_dev, void* stream) {
  if (!e) return LLR_ERR_INVALID;
  int rc = check_matrix(e, m);
  if (rc) return rc;
  if (tokens == 0 || !x_dev || !y_dev)
    return fail(e, LLR_ERR_INVALID, "CUDA GEMM buffer lengths do not match shape");
  DeviceGuard guard(e->device);
  cudaStream_t s = stream ? (cudaStream_t)stream : e->stream;
  void* scratch = nullptr;
  cudaError_t ce = ensure_scratch(e, m, tokens, &scratch);
  if (ce != cudaSuccess) return fail_cuda(e, ce, "kernel scratch");
  ce = launch_matmul(view_of(m), x_dev, y_dev, (int64_t)tokens, s, e->path, e->sm_count, e->err_flag,
                     scratch, &e->ctr.launches);
  if (ce != cudaSuccess) return fail_cuda(e, ce, "kernel launch");
  return LLR_OK;
}

int llr_gemm_device_noalloc(llr_exec* e, const llr_matrix* m, size_t tokens, const float* x_dev,
                            float* y_dev, void* stream) {
  if (!e) return LLR_ERR_INVALID;
  int rc = check_matrix(e, m);
  if (rc) return rc;
  if (tokens == 0 || !x_dev || !y_dev || ((uintptr_t)x_dev & 15) != 0)
    return fail(e, LLR_ERR_INVALID, "CUDA GEMM buffer lengths do not match shape (x must be 16-byte aligned)");
  const MatView v = view_of(m);
  if (!gemm_tc_supported(v, (int64_t)tokens))
    return fail(e, LLR_ERR_INVALID,
                "the allocation-free GEMM takes the block-quantized formats with cols % 256 == 0 (Q6_K: % 2048) and at least 16 activation rows");
  size_t need = 0;
  if (!mul_ok(tokens, (size_t)v.cols, &need) || !mul_ok(need, 2, &need) || need > gemm_tc_static_scratch_limit())
    return fail(e, LLR_ERR_INVALID, "tokens * cols * 2 = " + std::to_string(need) + " bytes exceeds the built-in staging area of " +
                                        std::to_string(gemm_tc_static_scratch_limit()) + " bytes; split the batch or use llr_matmul_device");
  DeviceGuard guard(e->device);
  cudaStream_t s = stream ? (cudaStream_t)stream : e->stream;
  cudaError_t ce = launch_gemm_tc_static(e->device, v, x_dev, y_dev, (int64_t)tokens, s, e->err_flag, &e->ctr.launches);
  if (ce != cudaSuccess) return fail_cuda(e, ce, "kernel launch");
  return LLR_OK;
}

int llr_exec_synchronize(llr_exec* e) {
  if (!e) return LLR_ERR_INVALID;
  DeviceGuard guard(e->device);
  cudaError_t ce = cudaStreamSynchronize(e->stream);
  if (ce != cudaSuccess) return fail_cuda(e, ce, "stream synchronize");
  if (take_device_error(e) != 0) {
    return fail(e, LLR_ERR_CUDA, "a device-side wait ran out of iterations (copy engine did not deliver a weight tile)");
  }
  return LLR_OK;
}

// ---------------------------------------------------------------- routed experts
namespace {

// Grouped expert products: with the automatic choice the tensor-core GEMM takes over from 16 routed
// rows (two passes of the 8-row decode kernel already cost more than one GEMM launch); below that,
// and for formats the GEMM does not take, the f32-faithful decode kernels run.
int expert_path(const llr_exec* e, size_t n_rows) { return e->path == PATH_AUTO && n_rows >= 16 ? PATH_TC : e->path; }

cudaError_t matmul_dev(llr_exec* e, const llr_matrix* m, size_t tokens, const float* x, float* y, int path) {
  void* scratch = nullptr;
  const int saved = e->path;
  e->path = path;
  cudaError_t ce = ensure_scratch(e, m, tokens, &scratch);
  if (ce == cudaSuccess)
    ce = launch_matmul(view_of(m), x, y, (int64_t)tokens, e->stream, path, e->sm_count, e->err_flag, scratch,
                       &e->ctr.launches);
  e->path = saved;
  return ce;
}

}  // namespace

namespace {

// Shapes and residency of a routed-expert layer, checked once per call.
struct MoeShape {
  size_t n_embd = 0, n_ff = 0, n_exp = 0, n_used = 0;
  std::vector<unsigned char> local;  // expert resident on this executor
  bool any_remote = false;
};

int moe_check_layer(llr_exec* e, const llr_moe_layer* L, bool need_router, MoeShape* S) {
  if (!L || (need_router && !L->router) || !L->gate || !L->up || !L->down || L->n_expert == 0 || L->n_used == 0 ||
      L->n_used > L->n_expert || L->n_expert > 4096)
    return fail(e, LLR_ERR_INVALID, "expert_used_count");
  int rc;
  S->n_exp = L->n_expert;
  S->n_used = L->n_used;
  if (need_router) {
    if ((rc = check_matrix(e, L->router))) return rc;
    S->n_embd = (size_t)L->router->cols;
    if ((size_t)L->router->rows != S->n_exp || S->n_embd % 4 != 0) return fail(e, LLR_ERR_INVALID, "ffn_gate_inp shape");
  }
  // An expert whose three matrices are all null lives on another rank (experts striped over GPUs):
  // it takes part in the routing, its rows are not computed here and contribute zero to `out`.
  S->local.assign(S->n_exp, 1);
  for (size_t i = 0; i < S->n_exp; ++i) {
    if (!L->gate[i] && !L->up[i] && !L->down[i]) { S->local[i] = 0; S->any_remote = true; continue; }
    if ((rc = check_matrix(e, L->gate[i])) || (rc = check_matrix(e, L->up[i])) || (rc = check_matrix(e, L->down[i]))) return rc;
    if (S->n_ff == 0) S->n_ff = (size_t)L->gate[i]->rows;
    if (S->n_embd == 0) S->n_embd = (size_t)L->gate[i]->cols;
    if ((size_t)L->gate[i]->rows != S->n_ff || (size_t)L->gate[i]->cols != S->n_embd || (size_t)L->up[i]->rows != S->n_ff ||
        (size_t)L->up[i]->cols != S->n_embd || (size_t)L->down[i]->rows != S->n_embd || (size_t)L->down[i]->cols != S->n_ff)
      return fail(e, LLR_ERR_INVALID, "expert matrix shapes do not match the layer");
  }
  if (S->n_ff == 0) return fail(e, LLR_ERR_INVALID, "no expert of the layer is resident on this executor");
  return LLR_OK;
}

// Device workspace of the expert products for n_rows packed rows, carved from one block.
struct MoeBuffers {
  float *g, *u, *y;        // gate / up results (n_rows x n_ff), down results (n_rows x n_embd)
  float* pack;             // packed f32 rows (n_rows x n_embd) when the rows have to be gathered first
  char *x16a, *x16b;       // 16-bit operand copies for the grouped tensor-core launches
  float *sa, *sb;          // their per-row scales
  void* desc;              // descriptors of a grouped launch
};
size_t moe_buffer_floats(const MoeShape& S, size_t n_rows) {
  const size_t f_pack = n_rows * S.n_embd, f_g = n_rows * S.n_ff;
  return f_pack + 2 * f_g + f_pack + (f_pack + f_g) / 2 + 2 * n_rows + 1024 + gemm_tc_group_desc_bytes((int)(2 * S.n_exp)) / 4 + 64;
}
MoeBuffers moe_carve(float* base, const MoeShape& S, size_t n_rows) {
  auto align256 = [](void* p) { return (char*)(((uintptr_t)p + 255) & ~(uintptr_t)255); };
  MoeBuffers B;
  B.pack = base;
  B.g = B.pack + n_rows * S.n_embd;
  B.u = B.g + n_rows * S.n_ff;
  B.y = B.u + n_rows * S.n_ff;
  B.x16a = align256(B.y + n_rows * S.n_embd);
  B.x16b = align256(B.x16a + n_rows * S.n_embd * 2);
  B.sa = (float*)align256(B.x16b + n_rows * S.n_ff * 2);
  B.sb = B.sa + n_rows;
  B.desc = align256(B.sb + n_rows);
  return B;
}

// The expert products over packed rows (grouped_routed_ffn decode.rs:10006-10290 without the scatter): rows
// [first_row[ex], first_row[ex+1]) belong to expert ex.  The rows are x[tok_of_row[r]] when tok_of_row is given
// (device), else x itself is the packed matrix.  Results: B.y, packed the same way; rows of experts that are not
// resident here are zero.
cudaError_t moe_run_experts(llr_exec* e, const llr_moe_layer* L, const MoeShape& S, const std::vector<int>& first_row,
                            const float* d_x, const int* d_tok_of_row, const MoeBuffers& B) {
  const size_t n_exp = S.n_exp, n_embd = S.n_embd, n_ff = S.n_ff;
  const size_t n_rows = (size_t)first_row[n_exp];
  cudaError_t ce = cudaSuccess;
  if (n_rows == 0) return ce;
  if (S.any_remote && (ce = cudaMemsetAsync(B.y, 0, n_rows * n_embd * 4, e->stream)) != cudaSuccess) return ce;  // rows nobody computes here
  {  // size the GEMM staging buffer once, for the busiest expert's widest product: growing it between
     // launches would free and reallocate, which synchronizes the device
    size_t busiest = 0, most = 0;
    for (size_t ex = 0; ex < n_exp; ++ex)
      if (S.local[ex] && (size_t)(first_row[ex + 1] - first_row[ex]) > most) { most = (size_t)(first_row[ex + 1] - first_row[ex]); busiest = ex; }
    void* unused = nullptr;
    if (most > 0 && ((ce = ensure_scratch(e, L->down[busiest], most, &unused)) != cudaSuccess ||
                     (ce = ensure_scratch(e, L->gate[busiest], most, &unused)) != cudaSuccess))
      return ce;
    if (most == 0) return cudaSuccess;  // nothing routed to a resident expert
  }
  // Grouped tensor-core path (automatic choice, 64 routed rows or more, formats the GEMM takes): the tiles of
  // all experts' gate and up products in one launch, silu(g)*u, all down products in one launch.
  bool grouped = e->path == PATH_AUTO && n_rows >= 64;
  int f16a = 1, f16b = 1;
  size_t first_local = 0;
  while (!S.local[first_local]) ++first_local;
  for (size_t ex = 0; ex < n_exp && grouped; ++ex) {
    if (!S.local[ex]) continue;
    const MatView vg = view_of(L->gate[ex]), vu = view_of(L->up[ex]), vd = view_of(L->down[ex]);
    grouped = gemm_tc_supported(vg, 16) && gemm_tc_supported(vu, 16) && gemm_tc_supported(vd, 16) &&
              vg.dtype == view_of(L->gate[first_local]).dtype && vu.dtype == vg.dtype &&
              vd.dtype == view_of(L->down[first_local]).dtype;
    if (vg.f16_ok != 1 || vu.f16_ok != 1) f16a = 0;
    if (vd.f16_ok != 1) f16b = 0;
  }
  const float* rows_f32 = d_x;  // packed f32 rows for the per-expert path
  if (!grouped && d_tok_of_row) {
    if ((ce = launch_gather_rows(d_x, d_tok_of_row, B.pack, (int)n_rows, (int)n_embd, e->stream, &e->ctr.launches)) != cudaSuccess) return ce;
    rows_f32 = B.pack;
  }
  if (grouped) {
    std::vector<GemmGroupSpec> specs;
    for (size_t ex = 0; ex < n_exp; ++ex) {
      const size_t r0 = (size_t)first_row[ex], n = (size_t)first_row[ex + 1] - r0;
      if (n == 0 || !S.local[ex]) continue;
      specs.push_back(GemmGroupSpec{view_of(L->gate[ex]), B.x16a + r0 * n_embd * 2, B.sa + r0, B.g + r0 * n_ff, (int)n});
      specs.push_back(GemmGroupSpec{view_of(L->up[ex]), B.x16a + r0 * n_embd * 2, B.sa + r0, B.u + r0 * n_ff, (int)n});
    }
    // the gather of the routed rows is part of the 16-bit conversion
    if (d_tok_of_row) ce = tc_convert_expert_rows(d_x, d_tok_of_row, (int64_t)n_rows, (int)n_embd, f16a != 0, B.x16a, B.sa, e->stream, &e->ctr.launches);
    else ce = tc_convert_activations(d_x, (int64_t)n_rows, (int)n_embd, f16a != 0, B.x16a, B.sa, e->stream, &e->ctr.launches);
    if (ce != cudaSuccess ||
        (ce = launch_gemm_tc_grouped(specs.data(), (int)specs.size(), f16a != 0, B.desc, e->stream, e->err_flag, &e->ctr.launches)) != cudaSuccess ||
        (ce = launch_silu_mul(B.g, B.u, (int64_t)(n_rows * n_ff), e->stream, &e->ctr.launches)) != cudaSuccess)
      return ce;
    specs.clear();
    for (size_t ex = 0; ex < n_exp; ++ex) {
      const size_t r0 = (size_t)first_row[ex], n = (size_t)first_row[ex + 1] - r0;
      if (n == 0 || !S.local[ex]) continue;
      specs.push_back(GemmGroupSpec{view_of(L->down[ex]), B.x16b + r0 * n_ff * 2, B.sb + r0, B.y + r0 * n_embd, (int)n});
    }
    // the descriptor buffer is reused: stream order puts this copy after the first grouped launch
    if ((ce = tc_convert_activations(B.g, (int64_t)n_rows, (int)n_ff, f16b != 0, B.x16b, B.sb, e->stream, &e->ctr.launches)) != cudaSuccess ||
        (ce = launch_gemm_tc_grouped(specs.data(), (int)specs.size(), f16b != 0, B.desc, e->stream, e->err_flag, &e->ctr.launches)) != cudaSuccess)
      return ce;
    return cudaSuccess;
  }
  for (size_t ex = 0; ex < n_exp; ++ex) {
    const size_t r0 = (size_t)first_row[ex], n = (size_t)first_row[ex + 1] - r0;
    if (n == 0 || !S.local[ex]) continue;
    if ((ce = matmul_dev(e, L->gate[ex], n, rows_f32 + r0 * n_embd, B.g + r0 * n_ff, expert_path(e, n))) != cudaSuccess ||
        (ce = matmul_dev(e, L->up[ex], n, rows_f32 + r0 * n_embd, B.u + r0 * n_ff, expert_path(e, n))) != cudaSuccess)
      return ce;
  }
  if ((ce = launch_silu_mul(B.g, B.u, (int64_t)(n_rows * n_ff), e->stream, &e->ctr.launches)) != cudaSuccess) return ce;
  for (size_t ex = 0; ex < n_exp; ++ex) {
    const size_t r0 = (size_t)first_row[ex], n = (size_t)first_row[ex + 1] - r0;
    if (n == 0 || !S.local[ex]) continue;
    if ((ce = matmul_dev(e, L->down[ex], n, B.g + r0 * n_ff, B.y + r0 * n_embd, expert_path(e, n))) != cudaSuccess) return ce;
  }
  return cudaSuccess;
}

// Router product and routing on the device: ids / wts (tokens x n_used, top-k order) in device memory.
cudaError_t moe_route(llr_exec* e, const llr_moe_layer* L, const MoeShape& S, size_t tokens, const float* d_x, float* d_logits,
                      int* d_ids, float* d_wts) {
  cudaError_t ce;
  // router product (decode.rs:9977)
  if (L->router->dtype == DT_F32 && ((uintptr_t)L->router->dev & 15) == 0)
    ce = launch_router_logits((const float*)L->router->dev, d_x, d_logits, (int)tokens, (int)S.n_exp, (int)S.n_embd, e->stream,
                              &e->ctr.launches);
  else
    ce = matmul_dev(e, L->router, tokens, d_x, d_logits, PATH_MMA);
  if (ce != cudaSuccess) return ce;
  return launch_route(d_logits, (int)tokens, (int)S.n_exp, (int)S.n_used, (int)L->norm_w, d_ids, d_wts, e->stream, &e->ctr.launches);
}

}  // namespace

int llr_moe_ffn(llr_exec* e, const llr_moe_layer* L, size_t tokens, const float* x, size_t x_len, float* out,
                size_t out_len, int32_t* sel_ids, float* sel_w) {
  if (!e) return LLR_ERR_INVALID;
  MoeShape S;
  int rc = moe_check_layer(e, L, true, &S);
  if (rc) return rc;
  const size_t n_embd = S.n_embd, n_exp = S.n_exp, n_used = S.n_used;
  size_t nx = 0;
  if (tokens == 0 || !mul_ok(tokens, n_embd, &nx) || x_len != nx || out_len != nx || !x || !out || tokens > (1u << 24))
    return fail(e, LLR_ERR_INVALID, "matrix dimensions must be positive and token-aligned");
  DeviceGuard guard(e->device);
  const size_t n_rows = tokens * n_used;
  // device workspace, one block: x | logits | out | routing tables | expert buffers
  const size_t f_logits = (tokens * n_exp + 3) & ~(size_t)3;
  const size_t f_tables = 6 * n_rows + tokens + n_exp + 64;  // ids, wts, tok_of_row, rows_of_tok, w_of_tok, fill, first_row, local
  const size_t floats = nx + f_logits + nx + f_tables + moe_buffer_floats(S, n_rows) + 256;
  cudaError_t ce;
  if ((ce = grow_device(&e->dev_moe, &e->dev_moe_cap, floats)) != cudaSuccess) return fail_cuda(e, ce, "expert workspace");
  float* d_x = e->dev_moe;
  float* d_logits = d_x + nx;
  float* d_out = d_logits + f_logits;
  int* d_ids = (int*)(d_out + nx);
  float* d_wts = (float*)(d_ids + n_rows);
  int* d_tok_of_row = (int*)(d_wts + n_rows);
  int* d_rows_of_tok = d_tok_of_row + n_rows;
  float* d_w = (float*)(d_rows_of_tok + n_rows);
  int* d_fill = (int*)(d_w + n_rows);
  int* d_first_row = d_fill + tokens;
  unsigned char* d_local = (unsigned char*)(d_first_row + n_exp + 1);
  float* d_expert = (float*)(((uintptr_t)(d_local + n_exp) + 255) & ~(uintptr_t)255);
  const MoeBuffers B = moe_carve(d_expert, S, n_rows);
  if ((ce = cudaMemcpyAsync(d_x, x, nx * 4, cudaMemcpyHostToDevice, e->stream)) != cudaSuccess ||
      (ce = cudaMemcpyAsync(d_local, S.local.data(), n_exp, cudaMemcpyHostToDevice, e->stream)) != cudaSuccess)
    return fail_cuda(e, ce, "activation upload");
  // Routing stays on the device: softmax, top-k and the router weights per token, then the packed row order of the
  // grouped products.  Only the per-expert row counts come back to the host, which needs them to size the launches.
  if ((ce = moe_route(e, L, S, tokens, d_x, d_logits, d_ids, d_wts)) != cudaSuccess ||
      (ce = launch_bucket(d_ids, d_wts, d_local, (int)tokens, (int)n_exp, (int)n_used, d_first_row, d_tok_of_row, d_rows_of_tok, d_w,
                          d_fill, e->stream, &e->ctr.launches)) != cudaSuccess)
    return fail_cuda(e, ce, "kernel launch");
  std::vector<int> first_row(n_exp + 1, 0);
  if ((ce = cudaMemcpyAsync(first_row.data(), d_first_row, (n_exp + 1) * sizeof(int), cudaMemcpyDeviceToHost, e->stream)) != cudaSuccess ||
      (ce = cudaStreamSynchronize(e->stream)) != cudaSuccess)
    return fail_cuda(e, ce, "routing counts");
  if ((ce = moe_run_experts(e, L, S, first_row, d_x, d_tok_of_row, B)) != cudaSuccess) return fail_cuda(e, ce, "kernel launch");
  if ((ce = launch_scatter_combine(B.y, d_rows_of_tok, d_w, d_out, (int)tokens, (int)n_used, (int)n_embd, e->stream,
                                   &e->ctr.launches)) != cudaSuccess)
    return fail_cuda(e, ce, "kernel launch");
  const bool out_pinned = is_pinned_host(e, out);  // a pinned result buffer is written directly
  float* dst = out;
  if (!out_pinned) {
    if ((ce = grow_pinned(&e->pin_y, &e->pin_y_cap, nx)) != cudaSuccess) return fail_cuda(e, ce, "pinned result staging");
    dst = e->pin_y;
  }
  std::vector<int32_t> ids(sel_ids ? n_rows : 0);
  std::vector<float> wts(sel_w ? n_rows : 0);
  if ((ce = cudaMemcpyAsync(dst, d_out, nx * 4, cudaMemcpyDeviceToHost, e->stream)) != cudaSuccess ||
      (sel_ids && (ce = cudaMemcpyAsync(ids.data(), d_ids, n_rows * 4, cudaMemcpyDeviceToHost, e->stream)) != cudaSuccess) ||
      (sel_w && (ce = cudaMemcpyAsync(wts.data(), d_wts, n_rows * 4, cudaMemcpyDeviceToHost, e->stream)) != cudaSuccess) ||
      (ce = cudaStreamSynchronize(e->stream)) != cudaSuccess)
    return fail_cuda(e, ce, "result download");
  if (take_device_error(e) != 0) {
    return fail(e, LLR_ERR_CUDA, "a device-side wait ran out of iterations");
  }
  if (!out_pinned) std::memcpy(out, e->pin_y, nx * 4);
  if (sel_ids) std::memcpy(sel_ids, ids.data(), n_rows * 4);
  if (sel_w) std::memcpy(sel_w, wts.data(), n_rows * 4);
  e->ctr.h2d_bytes += nx * 4 + n_exp;
  e->ctr.d2h_bytes += nx * 4 + (n_exp + 1) * 4 + (sel_ids ? n_rows * 4 : 0) + (sel_w ? n_rows * 4 : 0);
  return LLR_OK;
}

// Device-pointer pieces of the layer, for callers that keep tokens on the device and exchange routed rows between
// ranks themselves (experts striped over GPUs).
int llr_moe_route_device(llr_exec* e, const llr_moe_layer* L, size_t tokens, const float* x_dev, int32_t* ids_dev, float* w_dev) {
  if (!e) return LLR_ERR_INVALID;
  if (!L || !L->router || L->n_expert == 0 || L->n_used == 0 || L->n_used > L->n_expert || L->n_expert > 4096)
    return fail(e, LLR_ERR_INVALID, "expert_used_count");
  int rc = check_matrix(e, L->router);
  if (rc) return rc;
  MoeShape S;
  S.n_exp = L->n_expert; S.n_used = L->n_used; S.n_embd = (size_t)L->router->cols;
  if ((size_t)L->router->rows != S.n_exp || S.n_embd % 4 != 0) return fail(e, LLR_ERR_INVALID, "ffn_gate_inp shape");
  if (tokens == 0 || tokens > (1u << 24) || !x_dev || !ids_dev || !w_dev || ((uintptr_t)x_dev & 15) != 0)
    return fail(e, LLR_ERR_INVALID, "matrix dimensions must be positive and token-aligned");
  DeviceGuard guard(e->device);
  cudaError_t ce;
  const size_t f_logits = tokens * S.n_exp;
  if ((ce = grow_device(&e->dev_y, &e->dev_y_cap, f_logits)) != cudaSuccess) return fail_cuda(e, ce, "router scratch");
  if ((ce = moe_route(e, L, S, tokens, x_dev, e->dev_y, (int*)ids_dev, w_dev)) != cudaSuccess) return fail_cuda(e, ce, "kernel launch");
  return LLR_OK;
}

int llr_moe_experts_device(llr_exec* e, const llr_moe_layer* L, const uint32_t* counts, const float* rows_dev, float* y_dev) {
  if (!e) return LLR_ERR_INVALID;
  MoeShape S;
  int rc = moe_check_layer(e, L, false, &S);
  if (rc) return rc;
  if (!counts || !rows_dev || !y_dev || ((uintptr_t)rows_dev & 15) != 0 || ((uintptr_t)y_dev & 15) != 0)
    return fail(e, LLR_ERR_INVALID, "null or unaligned buffer");
  std::vector<int> first_row(S.n_exp + 1, 0);
  size_t total = 0;
  for (size_t ex = 0; ex < S.n_exp; ++ex) {
    if (counts[ex] != 0 && !S.local[ex]) return fail(e, LLR_ERR_INVALID, "rows for expert " + std::to_string(ex) + ", which is not resident on this executor");
    total += counts[ex];
    if (total > (1u << 24)) return fail(e, LLR_ERR_INVALID, "too many routed rows");
    first_row[ex + 1] = (int)total;
  }
  if (total == 0) return LLR_OK;
  DeviceGuard guard(e->device);
  cudaError_t ce;
  if ((ce = grow_device(&e->dev_moe, &e->dev_moe_cap, moe_buffer_floats(S, total) + 256)) != cudaSuccess) return fail_cuda(e, ce, "expert workspace");
  const MoeBuffers B = moe_carve((float*)(((uintptr_t)e->dev_moe + 255) & ~(uintptr_t)255), S, total);
  S.any_remote = false;  // every row given here belongs to a resident expert
  if ((ce = moe_run_experts(e, L, S, first_row, rows_dev, nullptr, B)) != cudaSuccess) return fail_cuda(e, ce, "kernel launch");
  if ((ce = cudaMemcpyAsync(y_dev, B.y, total * S.n_embd * 4, cudaMemcpyDeviceToDevice, e->stream)) != cudaSuccess)
    return fail_cuda(e, ce, "result copy");
  return LLR_OK;
}

// ---- expert parallelism over peer stores (kernels: llr_moe_ep.cu) ----------------------------------------
struct llr_moe_ep {
  llr_exec* owner = nullptr;
  MoeShape S;
  llr_moe_layer layer{};
  std::vector<const llr_matrix*> gate, up, down;
  EpLayout L{};
  EpPeers peers{};
  unsigned long long epoch = 0, dispatch_total = 0, return_total = 0;
  size_t tokens = 0;  // of the run in flight
  int stage = 0;      // 0 idle, 1 dispatched, 2 served
  char* tables = nullptr;  // one device block: everything below except rows
  float* d_logits = nullptr; int* d_ids = nullptr; float* d_wts = nullptr; int* d_tok_of_row = nullptr;
  int* d_rows_of_tok = nullptr; float* d_w = nullptr; int* d_fill = nullptr; int* d_first_row = nullptr;
  unsigned char* d_local = nullptr; int* d_seg_first = nullptr; int* d_ret_src = nullptr; int* d_ret_tag = nullptr;
  float* d_rows = nullptr; size_t rows_cap = 0;  // gathered rows of this rank's experts
  int* h_cnt = nullptr;  // pinned: counts [local expert][sender], then the segment starts
};

size_t llr_moe_ep_arena_bytes(uint32_t n_expert, uint32_t n_used, size_t n_embd, uint32_t world, size_t max_tokens) {
  if (n_expert == 0 || n_used == 0 || n_used > n_expert || n_expert > 4096 || n_embd == 0 || n_embd % 4 != 0 || n_embd > (1u << 20) ||
      world == 0 || world > (uint32_t)EP_MAX_WORLD || max_tokens == 0 || max_tokens > (1u << 20))
    return 0;
  return ep_layout((int)n_expert, (int)n_used, (int)n_embd, (int)world, 0, (int)max_tokens).total;
}

int llr_moe_ep_free(llr_moe_ep* ep) {
  if (!ep) return LLR_OK;
  DeviceGuard guard(ep->owner->device);
  cudaStreamSynchronize(ep->owner->stream);
  if (ep->tables) cudaFree(ep->tables);
  if (ep->d_rows) cudaFree(ep->d_rows);
  if (ep->h_cnt) cudaFreeHost(ep->h_cnt);
  delete ep;
  return LLR_OK;
}

int llr_moe_ep_create(llr_exec* e, const llr_moe_layer* L, uint32_t world, uint32_t rank, size_t max_tokens, void* arena,
                      size_t arena_bytes, void* const* peer_arenas, llr_moe_ep** out) {
  if (!e) return LLR_ERR_INVALID;
  if (!out) return fail(e, LLR_ERR_INVALID, "null output");
  *out = nullptr;
  MoeShape S;
  int rc = moe_check_layer(e, L, true, &S);
  if (rc) return rc;
  if (world == 0 || world > (uint32_t)EP_MAX_WORLD || rank >= world || max_tokens == 0 || max_tokens > (1u << 20) || !arena ||
      ((uintptr_t)arena & 255) != 0 || (world > 1 && !peer_arenas))
    return fail(e, LLR_ERR_INVALID, "expert-parallel layer: world 1..8, rank < world, max_tokens 1..2^20, a 256-byte aligned arena");
  for (size_t ex = 0; ex < S.n_exp; ++ex)
    if ((S.local[ex] != 0) != (ex % world == rank))
      return fail(e, LLR_ERR_INVALID, "expert " + std::to_string(ex) + ": rank e % world holds an expert's matrices and every other rank passes NULL for it");
  const EpLayout lay = ep_layout((int)S.n_exp, (int)S.n_used, (int)S.n_embd, (int)world, (int)rank, (int)max_tokens);
  if (arena_bytes < lay.total)
    return fail(e, LLR_ERR_INVALID, "the arena holds " + std::to_string(arena_bytes) + " bytes, llr_moe_ep_arena_bytes asks for " + std::to_string(lay.total));
  DeviceGuard guard(e->device);
  {
    // Runs are counted from zero in this object and in the arena alike.  The words below are written by this rank's own
    // kernels only, so they tell (without racing against peers that already run) whether this arena served a layer
    // before: its flags would then pass for runs that have not happened yet.
    EpHeader h;
    cudaError_t ce = cudaMemcpy(&h, arena, sizeof(h), cudaMemcpyDeviceToHost);
    if (ce != cudaSuccess) return fail_cuda(e, ce, "expert-parallel arena");
    if (h.done_dispatch != 0 || h.done_return != 0 || h.flag_in[rank] != 0 || h.flag_back[rank] != 0)
      return fail(e, LLR_ERR_INVALID, "the arena has served an expert-parallel layer before: free the layer on every rank, zero every arena "
                                      "(or allocate new ones), and only then create the next layer");
  }
  std::unique_ptr<llr_moe_ep> ep(new llr_moe_ep);
  ep->owner = e;
  ep->S = S;
  ep->S.any_remote = false;  // the rows this rank computes all belong to its own experts
  ep->gate.assign(L->gate, L->gate + S.n_exp);
  ep->up.assign(L->up, L->up + S.n_exp);
  ep->down.assign(L->down, L->down + S.n_exp);
  ep->layer = *L;
  ep->layer.gate = ep->gate.data(); ep->layer.up = ep->up.data(); ep->layer.down = ep->down.data();
  ep->L = lay;
  for (uint32_t g = 0; g < world; ++g) {
    ep->peers.arena[g] = g == rank ? (char*)arena : (char*)peer_arenas[g];
    if (!ep->peers.arena[g] || ((uintptr_t)ep->peers.arena[g] & 255) != 0) return fail(e, LLR_ERR_INVALID, "peer arena " + std::to_string(g));
  }
  const size_t T = max_tokens, n_rows = T * S.n_used, n_seg = (size_t)lay.e_loc * world, max_gather = n_seg * T;
  auto up256 = [](size_t v) { return (v + 255) & ~(size_t)255; };
  size_t at = 0;
  auto take = [&](size_t bytes) { const size_t o = at; at = up256(at + bytes); return o; };
  const size_t o_logits = take(T * S.n_exp * 4), o_ids = take(n_rows * 4), o_wts = take(n_rows * 4), o_tor = take(n_rows * 4),
               o_rot = take(n_rows * 4), o_w = take(n_rows * 4), o_fill = take(T * 4), o_first = take((S.n_exp + 1) * 4),
               o_local = take(S.n_exp), o_seg = take((n_seg + 1) * 4), o_rsrc = take(max_gather * 4), o_rtag = take(max_gather * 4);
  cudaError_t ce;
  if ((ce = cudaMalloc((void**)&ep->tables, at)) != cudaSuccess) return fail_cuda(e, ce, "expert-parallel tables");
  char* tb = ep->tables;
  ep->d_logits = (float*)(tb + o_logits); ep->d_ids = (int*)(tb + o_ids); ep->d_wts = (float*)(tb + o_wts);
  ep->d_tok_of_row = (int*)(tb + o_tor); ep->d_rows_of_tok = (int*)(tb + o_rot); ep->d_w = (float*)(tb + o_w);
  ep->d_fill = (int*)(tb + o_fill); ep->d_first_row = (int*)(tb + o_first); ep->d_local = (unsigned char*)(tb + o_local);
  ep->d_seg_first = (int*)(tb + o_seg); ep->d_ret_src = (int*)(tb + o_rsrc); ep->d_ret_tag = (int*)(tb + o_rtag);
  if ((ce = cudaMallocHost((void**)&ep->h_cnt, (2 * n_seg + 2) * sizeof(int))) != cudaSuccess) {
    llr_moe_ep_free(ep.release());
    return fail_cuda(e, ce, "expert-parallel tables");
  }
  // every selected expert's weight counts: the rows of experts that live elsewhere come back from their owners
  if ((ce = cudaMemsetAsync(ep->d_local, 1, S.n_exp, e->stream)) != cudaSuccess || (ce = cudaStreamSynchronize(e->stream)) != cudaSuccess) {
    llr_moe_ep_free(ep.release());
    return fail_cuda(e, ce, "expert-parallel tables");
  }
  *out = ep.release();
  return LLR_OK;
}

int llr_moe_ep_dispatch(llr_moe_ep* ep, size_t tokens, const float* x_dev) {
  if (!ep) return LLR_ERR_INVALID;
  llr_exec* e = ep->owner;
  if (ep->stage != 0) return fail(e, LLR_ERR_INVALID, "expert-parallel layer: the previous run has not been combined");
  if (tokens == 0 || tokens > (size_t)ep->L.t_max || !x_dev || ((uintptr_t)x_dev & 15) != 0)
    return fail(e, LLR_ERR_INVALID, "expert-parallel layer: 1..max_tokens rows at a 16-byte aligned device address");
  DeviceGuard guard(e->device);
  const MoeShape& S = ep->S;
  cudaError_t ce;
  if ((ce = moe_route(e, &ep->layer, S, tokens, x_dev, ep->d_logits, ep->d_ids, ep->d_wts)) != cudaSuccess ||
      (ce = launch_bucket(ep->d_ids, ep->d_wts, ep->d_local, (int)tokens, (int)S.n_exp, (int)S.n_used, ep->d_first_row, ep->d_tok_of_row,
                          ep->d_rows_of_tok, ep->d_w, ep->d_fill, e->stream, &e->ctr.launches)) != cudaSuccess)
    return fail_cuda(e, ce, "kernel launch");
  const size_t n_rows = tokens * S.n_used;
  ++ep->epoch;
  ep->dispatch_total += n_rows;
  if ((ce = launch_ep_dispatch(x_dev, ep->d_tok_of_row, ep->d_first_row, (int)n_rows, ep->peers, ep->L, (int)(ep->epoch & 1), ep->epoch,
                               ep->dispatch_total, e->stream, &e->ctr.launches)) != cudaSuccess)
    return fail_cuda(e, ce, "kernel launch");
  ep->tokens = tokens;
  ep->stage = 1;
  return LLR_OK;
}

int llr_moe_ep_serve(llr_moe_ep* ep) {
  if (!ep) return LLR_ERR_INVALID;
  llr_exec* e = ep->owner;
  if (ep->stage != 1) return fail(e, LLR_ERR_INVALID, "expert-parallel layer: serve follows dispatch");
  DeviceGuard guard(e->device);
  const EpLayout& L = ep->L;
  const MoeShape& S = ep->S;
  const int p = (int)(ep->epoch & 1);
  const size_t n_seg = (size_t)L.e_loc * L.world;
  char* mine = ep->peers.arena[L.rank];
  ep->stage = 0;  // a failure below ends the run
  cudaError_t ce;
  if ((ce = launch_ep_wait(((EpHeader*)mine)->flag_in, L.world, ep->epoch, e->poll_limit, e->err_flag, e->stream, &e->ctr.launches)) != cudaSuccess ||
      (ce = cudaMemcpyAsync(ep->h_cnt, mine + L.cnt_off[p], n_seg * sizeof(int), cudaMemcpyDeviceToHost, e->stream)) != cudaSuccess ||
      (ce = cudaStreamSynchronize(e->stream)) != cudaSuccess)
    return fail_cuda(e, ce, "routed-row counts");
  if (take_device_error(e) != 0)
    return fail(e, LLR_ERR_CUDA, "a device-side wait ran out of iterations (a rank did not deliver its routed rows); re-create the expert-parallel layer on every rank");
  e->ctr.d2h_bytes += n_seg * sizeof(int);
  // packed order of this rank's experts: expert ascending, sender ascending, arrival position ascending
  int* seg = ep->h_cnt + n_seg;
  std::vector<int> first_row(S.n_exp + 1, 0);
  int total = 0;
  for (size_t k = 0; k < n_seg; ++k) {
    const int c = ep->h_cnt[k];
    if (c < 0 || c > L.t_max) return fail(e, LLR_ERR_CUDA, "expert-parallel layer: a sender's row count is out of range");
    seg[k] = total;
    total += c;
  }
  seg[n_seg] = total;
  for (size_t ex = 0; ex < S.n_exp; ++ex) {
    const size_t le = ex / L.world;
    first_row[ex + 1] = first_row[ex] + (S.local[ex] ? seg[(le + 1) * L.world] - seg[le * L.world] : 0);
  }
  if ((ce = cudaMemcpyAsync(ep->d_seg_first, seg, (n_seg + 1) * sizeof(int), cudaMemcpyHostToDevice, e->stream)) != cudaSuccess)
    return fail_cuda(e, ce, "segment table");
  const float* y = nullptr;
  if (total > 0) {
    if ((ce = grow_device(&ep->d_rows, &ep->rows_cap, (size_t)total * S.n_embd)) != cudaSuccess ||
        (ce = grow_device(&e->dev_moe, &e->dev_moe_cap, moe_buffer_floats(S, (size_t)total) + 256)) != cudaSuccess)
      return fail_cuda(e, ce, "expert workspace");
    const MoeBuffers B = moe_carve((float*)(((uintptr_t)e->dev_moe + 255) & ~(uintptr_t)255), S, (size_t)total);
    if ((ce = launch_ep_gather(mine, L, p, ep->d_seg_first, (int)n_seg, total, ep->d_rows, ep->d_ret_src, ep->d_ret_tag, e->stream,
                               &e->ctr.launches)) != cudaSuccess ||
        (ce = moe_run_experts(e, &ep->layer, S, first_row, ep->d_rows, nullptr, B)) != cudaSuccess)
      return fail_cuda(e, ce, "kernel launch");
    y = B.y;
  }
  ep->return_total += (unsigned long long)total;
  if ((ce = launch_ep_return(y, ep->d_ret_src, ep->d_ret_tag, total, ep->peers, L, p, ep->epoch, ep->return_total, e->stream,
                             &e->ctr.launches)) != cudaSuccess)
    return fail_cuda(e, ce, "kernel launch");
  ep->stage = 2;
  return LLR_OK;
}

int llr_moe_ep_combine(llr_moe_ep* ep, float* out_dev, int32_t* ids_dev, float* w_dev) {
  if (!ep) return LLR_ERR_INVALID;
  llr_exec* e = ep->owner;
  if (ep->stage != 2) return fail(e, LLR_ERR_INVALID, "expert-parallel layer: combine follows serve");
  if (!out_dev || ((uintptr_t)out_dev & 15) != 0) return fail(e, LLR_ERR_INVALID, "null or unaligned buffer");
  DeviceGuard guard(e->device);
  const EpLayout& L = ep->L;
  const int p = (int)(ep->epoch & 1);
  char* mine = ep->peers.arena[L.rank];
  const size_t n_rows = ep->tokens * ep->S.n_used;
  ep->stage = 0;
  cudaError_t ce;
  if ((ce = launch_ep_wait(((EpHeader*)mine)->flag_back, L.world, ep->epoch, e->poll_limit, e->err_flag, e->stream, &e->ctr.launches)) != cudaSuccess ||
      (ce = launch_scatter_combine((const float*)(mine + L.back_off[p]), ep->d_rows_of_tok, ep->d_w, out_dev, (int)ep->tokens, (int)ep->S.n_used,
                                   (int)ep->S.n_embd, e->stream, &e->ctr.launches)) != cudaSuccess ||
      (ids_dev && (ce = cudaMemcpyAsync(ids_dev, ep->d_ids, n_rows * 4, cudaMemcpyDeviceToDevice, e->stream)) != cudaSuccess) ||
      (w_dev && (ce = cudaMemcpyAsync(w_dev, ep->d_wts, n_rows * 4, cudaMemcpyDeviceToDevice, e->stream)) != cudaSuccess))
    return fail_cuda(e, ce, "kernel launch");
  return LLR_OK;
}

int llr_moe_ep_run(llr_moe_ep* ep, size_t tokens, const float* x_dev, float* out_dev, int32_t* ids_dev, float* w_dev) {
  int rc = llr_moe_ep_dispatch(ep, tokens, x_dev);
  if (rc == LLR_OK) rc = llr_moe_ep_serve(ep);
  if (rc == LLR_OK) rc = llr_moe_ep_combine(ep, out_dev, ids_dev, w_dev);
  return rc;
}

struct llr_program {
  llr_exec* owner;
  llr::Program* prog;
};

namespace {
// validation shared by the ways of creating a program; ops may carry an operation on the input and a residual
int program_entries(llr_exec* e, const llr_program_op* ops, size_t n, std::vector<ProgEntry>* pe, std::vector<int>* phase) {
  if (!ops || n == 0 || n > (1u << 20)) return fail(e, LLR_ERR_INVALID, "a program needs 1..2^20 entries");
  pe->resize(n);
  phase->resize(n);
  for (size_t i = 0; i < n; ++i) {
    const llr_program_op& in = ops[i];
    const std::string which = "program entry " + std::to_string(i);
    int rc = check_matrix(e, in.matrix);
    if (rc) return rc;
    if (in.tokens == 0 || in.tokens > 8 || !in.x_dev || !in.y_dev || ((uintptr_t)in.x_dev & 15) != 0)
      return fail(e, LLR_ERR_INVALID, which + ": tokens must be 1..8 and buffers 16-byte aligned");
    if (i > 0 && in.phase < ops[i - 1].phase) return fail(e, LLR_ERR_INVALID, which + ": phase must be non-decreasing");
    const MatView v = view_of(in.matrix);
    if (!prog_entry_supported(v))
      return fail(e, LLR_ERR_INVALID, which + ": only Q4_K, Q6_K (cols % 2048 == 0) and Q8_0 with cols % 256 == 0 run in programs");
    const int64_t ld = in.y_ld ? (int64_t)in.y_ld : v.rows;
    if (ld < v.rows) return fail(e, LLR_ERR_INVALID, which + ": y_ld is smaller than the row count");
    if (in.x_op > LLR_XOP_SWIGLU) return fail(e, LLR_ERR_INVALID, which + ": unknown input operation");
    if (in.x_op == LLR_XOP_SWIGLU && (!in.x2_dev || ((uintptr_t)in.x2_dev & 15) != 0))
      return fail(e, LLR_ERR_INVALID, which + ": SwiGLU needs its second input, 16-byte aligned");
    if (in.x_op == LLR_XOP_RMSNORM && (((uintptr_t)in.x2_dev & 15) != 0 || !(in.eps >= 0.0f)))
      return fail(e, LLR_ERR_INVALID, which + ": RMSNorm weights must be 16-byte aligned and eps non-negative");
    if (((uintptr_t)in.resid_dev & 3) != 0 || ((uintptr_t)in.y_dev & 3) != 0)
      return fail(e, LLR_ERR_INVALID, which + ": result and residual must be 4-byte aligned");
    ProgEntry E{};
    E.w = v.w; E.x = in.x_dev; E.y = in.y_dev; E.row_bytes = v.row_bytes;
    E.rows = (int)v.rows; E.cols = (int)v.cols; E.dtype = v.dtype; E.tokens = (int)in.tokens;
    E.y_ld = ld;
    E.x2 = in.x_op == LLR_XOP_NONE ? nullptr : in.x2_dev;
    E.resid = in.resid_dev;
    E.x_op = (int)in.x_op; E.eps = in.eps;
    E.x_phase = E.x2_phase = E.resid_phase = -1;
    (*pe)[i] = E;
    (*phase)[i] = (int)in.phase;
  }
  return LLR_OK;
}

int program_from(llr_exec* e, const llr_program_op* ops, size_t n, bool strict, const llr_program_shard* sh, llr_program** out) {
  if (!e) return LLR_ERR_INVALID;
  if (!out) return fail(e, LLR_ERR_INVALID, "null output pointer");
  *out = nullptr;
  if (sh && (sh->world < 2 || sh->world > 8 || sh->rank >= sh->world || !sh->arena || !sh->peer_arenas ||
             sh->arena_bytes <= LLR_ARENA_HEADER_BYTES))
    return fail(e, LLR_ERR_INVALID, "a sharded program needs 2..8 ranks, an arena larger than its header and the peers' arenas");
  std::vector<ProgEntry> pe;
  std::vector<int> phase;
  int rc = program_entries(e, ops, n, &pe, &phase);
  if (rc) return rc;
  ShardInfo si{};
  if (sh) {
    // header | results | tagged copies of the results (twice as large)
    const size_t result_bytes = ((sh->arena_bytes - LLR_ARENA_HEADER_BYTES) / 3) & ~(size_t)255;
    const char* lo = (const char*)sh->arena + LLR_ARENA_HEADER_BYTES;
    const char* hi = lo + result_bytes;
    int n_phases = 0;
    for (size_t i = 0; i < n; ++i) {
      const char* y0 = (const char*)pe[i].y;
      const char* y1 = y0 + ((size_t)(pe[i].tokens - 1) * (size_t)pe[i].y_ld + (size_t)pe[i].rows) * sizeof(float);
      if (y0 < lo || y1 > hi)
        return fail(e, LLR_ERR_INVALID, "program entry " + std::to_string(i) + ": the result slice is outside the arena's result area");
      if (i == 0 || phase[i] != phase[i - 1]) ++n_phases;
    }
    if (n_phases > 4095) return fail(e, LLR_ERR_INVALID, "a sharded program has at most 4095 phases");
    for (uint32_t g = 0; g < sh->world; ++g) {
      if (g == sh->rank) continue;
      if (!sh->peer_arenas[g]) return fail(e, LLR_ERR_INVALID, "missing arena of rank " + std::to_string(g));
      si.peers.counters[si.peers.n_peers] = (unsigned long long*)sh->peer_arenas[g];
      si.peers.y_delta[si.peers.n_peers] = (long long)((const char*)sh->peer_arenas[g] - (const char*)sh->arena);
      ++si.peers.n_peers;
    }
    si.counters = (unsigned long long*)sh->arena;
    si.arena = (char*)sh->arena;
    si.result_bytes = result_bytes;
    si.world = (int)sh->world;
    si.rank = (int)sh->rank;
  }
  DeviceGuard guard(e->device);
  llr::Program* prog = nullptr;
  std::string msg;
  cudaError_t ce = program_create(pe, phase, e->sm_count, strict, sh ? &si : nullptr, &prog, &msg);
  if (ce != cudaSuccess) return fail_cuda(e, ce, msg.empty() ? "program creation" : msg.c_str());
  llr_program* p = new (std::nothrow) llr_program{e, prog};
  if (!p) { program_destroy(prog); return fail(e, LLR_ERR_OOM, "host allocation failed"); }
  *out = p;
  return LLR_OK;
}

std::vector<llr_program_op> ops_of(const llr_program_entry* entries, const uint64_t* y_ld, size_t n) {
  std::vector<llr_program_op> ops(entries ? n : 0);
  for (size_t i = 0; i < ops.size(); ++i) {
    ops[i] = llr_program_op{};
    ops[i].matrix = entries[i].matrix;
    ops[i].x_dev = entries[i].x_dev;
    ops[i].y_dev = entries[i].y_dev;
    ops[i].y_ld = y_ld ? y_ld[i] : 0;
    ops[i].tokens = entries[i].tokens;
    ops[i].phase = entries[i].phase;
  }
  return ops;
}
}  // namespace

int llr_program_create(llr_exec* e, const llr_program_entry* entries, size_t n, llr_program** out) {
  if (!e) return LLR_ERR_INVALID;
  if (n > (1u << 20)) return fail(e, LLR_ERR_INVALID, "a program needs 1..2^20 entries");
  const std::vector<llr_program_op> ops = ops_of(entries, nullptr, n);
  return program_from(e, ops.empty() ? nullptr : ops.data(), n, true, nullptr, out);
}

int llr_program_create_ops(llr_exec* e, const llr_program_op* ops, size_t n, const llr_program_shard* shard,
                           llr_program** out) {
  return program_from(e, ops, n, false, shard, out);
}

int llr_program_info(const llr_program* p, uint32_t* entries, uint32_t* phases, uint32_t* counter_phases, uint32_t* ctas) {
  if (!p || !p->prog) return LLR_ERR_INVALID;
  if (entries) *entries = (uint32_t)llr::program_entries(p->prog);
  if (phases) *phases = (uint32_t)llr::program_phases(p->prog);
  if (counter_phases) *counter_phases = (uint32_t)llr::program_counter_phases(p->prog);
  if (ctas) *ctas = (uint32_t)llr::program_grid(p->prog);
  return LLR_OK;
}

int llr_exec_set_wait_limit(llr_exec* e, uint32_t polls) {
  if (!e) return LLR_ERR_INVALID;
  if (polls == 0 || polls > (1u << 30)) return fail(e, LLR_ERR_INVALID, "the wait limit must be 1..2^30 polls");
  e->poll_limit = (int)polls;
  return LLR_OK;
}

// ---------------------------------------------------------------- row-sharded programs
int llr_shared_alloc(llr_exec* e, size_t bytes, void** dev, llr_ipc_handle* handle) {
  if (!e) return LLR_ERR_INVALID;
  if (!dev || !handle || bytes == 0) return fail(e, LLR_ERR_INVALID, "shared allocation needs a size, an address slot and a handle slot");
  static_assert(sizeof(cudaIpcMemHandle_t) == sizeof(llr_ipc_handle), "handle size");
  DeviceGuard guard(e->device);
  void* p = nullptr;
  cudaError_t ce = cudaMalloc(&p, bytes);
  if (ce == cudaSuccess) ce = cudaMemset(p, 0, bytes);
  cudaIpcMemHandle_t h;
  if (ce == cudaSuccess) ce = cudaIpcGetMemHandle(&h, p);
  if (ce != cudaSuccess) {
    if (p) cudaFree(p);
    return fail_cuda(e, ce, "shared allocation");
  }
  std::memcpy(handle->bytes, &h, sizeof(h));
  *dev = p;
  return LLR_OK;
}

int llr_shared_open(llr_exec* e, const llr_ipc_handle* handle, void** dev) {
  if (!e) return LLR_ERR_INVALID;
  if (!dev || !handle) return fail(e, LLR_ERR_INVALID, "null handle or address slot");
  DeviceGuard guard(e->device);
  cudaIpcMemHandle_t h;
  std::memcpy(&h, handle->bytes, sizeof(h));
  void* p = nullptr;
  cudaError_t ce = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
  if (ce != cudaSuccess) return fail_cuda(e, ce, "opening a peer's shared allocation");
  *dev = p;
  return LLR_OK;
}

int llr_shared_close(llr_exec* e, void* dev) {
  if (!e) return LLR_ERR_INVALID;
  if (!dev) return LLR_OK;
  DeviceGuard guard(e->device);
  cudaError_t ce = cudaIpcCloseMemHandle(dev);
  if (ce != cudaSuccess) return fail_cuda(e, ce, "closing a peer's shared allocation");
  return LLR_OK;
}

int llr_shared_free(llr_exec* e, void* dev) {
  if (!e) return LLR_ERR_INVALID;
  if (!dev) return LLR_OK;
  DeviceGuard guard(e->device);
  cudaError_t ce = cudaFree(dev);
  if (ce != cudaSuccess) return fail_cuda(e, ce, "freeing a shared allocation");
  return LLR_OK;
}

int llr_program_create_sharded(llr_exec* e, const llr_program_entry* entries, const uint64_t* y_ld, size_t n,
                               void* arena, size_t arena_bytes, uint32_t world, uint32_t rank,
                               void* const* peer_arenas, llr_program** out) {
  if (!e) return LLR_ERR_INVALID;
  if (n > (1u << 20)) return fail(e, LLR_ERR_INVALID, "a program needs 1..2^20 entries");
  const std::vector<llr_program_op> ops = ops_of(entries, y_ld, n);
  const llr_program_shard sh{arena, arena_bytes, world, rank, peer_arenas};
  return program_from(e, ops.empty() ? nullptr : ops.data(), n, true, &sh, out);
}

int llr_program_run(llr_exec* e, llr_program* p, void* stream) {
  if (!e) return LLR_ERR_INVALID;
  if (!p || p->owner != e) return fail(e, LLR_ERR_FOREIGN, "program belongs to a different executor");
  DeviceGuard guard(e->device);
  cudaStream_t s = stream ? (cudaStream_t)stream : e->stream;
  cudaError_t ce = program_run(p->prog, s, e->err_flag, e->poll_limit, &e->ctr.launches);
  if (ce != cudaSuccess) return fail_cuda(e, ce, "program launch");
  return LLR_OK;
}

int llr_program_free(llr_program* p) {
  if (!p) return LLR_OK;
  if (p->owner) {
    DeviceGuard guard(p->owner->device);
    cudaDeviceSynchronize();
    program_destroy(p->prog);
  }
  delete p;
  return LLR_OK;
}

// ---------------------------------------------------------------- device-resident Llama walk
struct llr_session {
  llr_exec* owner = nullptr;
  llr_llama_config cfg{};
  WalkShape shape{};
  const llr_matrix* embd = nullptr;
  const llr_matrix* output = nullptr;
  std::vector<llr_llama_layer> layers;
  std::vector<float*> attn_norm, ffn_norm;  // device copies (null: all ones)
  float* out_norm = nullptr;
  size_t max_batch = 0;
  // sequences and their paged KV (kv_page.rs): blocks of block_tokens positions, a table of block ids per sequence
  size_t n_seq = 1, block_tokens = 16, max_blocks = 0, n_blocks = 0;
  std::vector<size_t> position;             // tokens appended per sequence
  std::vector<std::vector<int>> seq_blocks; // block ids per sequence, in order
  std::vector<int> free_blocks;
  std::vector<char> have_logits;            // sequence 0: logits in `logits` belong to it
  // device buffers
  float *x = nullptr, *xn = nullptr, *q = nullptr, *k = nullptr, *v = nullptr, *attn = nullptr, *proj = nullptr,
        *gate = nullptr, *up = nullptr, *logits = nullptr, *cache_k = nullptr, *cache_v = nullptr, *att_scratch = nullptr,
        *margins = nullptr, *last_x = nullptr, *arg_part = nullptr;
  size_t logits_rows = 1;
  int *ids = nullptr, *pos_dev = nullptr;  // ids[0]: the token the next step reads; ids[1..]: prompt chunk or generated tokens
  size_t ids_cap = 0;
  int* count_dev = nullptr;  // tokens generated by the current llr_session_decode call
  int *table_dev = nullptr, *row_pos = nullptr, *row_seq = nullptr, *last_rows = nullptr;
  // decode steps (one row): the independent products of a layer as one launch each -- {q, k, v} and {gate, up}
  std::vector<llr::Program*> qkv_prog, gateup_prog;
  // routed layers, one token: the chosen experts' {gate, up} products as one launch and their down products as another
  // (select programs over Moe::maps and moe_sel); null where a format is outside the programs' and the products run one by one
  std::vector<llr::Program*> moe_gateup_prog, moe_down_prog;
  // layers whose FFN is a routed-expert layer (architecture=llama with n_expert > 0): own copies of the matrix arrays
  struct Moe {
    std::vector<const llr_matrix*> gate, up, down;
    llr_moe_layer layer{};
    MoeShape S;
    char* maps = nullptr;  // device: tensor maps of the experts' gate | up | down matrices (n_expert each), for one-token steps
  };
  std::vector<std::unique_ptr<Moe>> moe;  // per layer, null: dense FFN
  std::vector<std::pair<size_t, size_t>> batch_groups;  // llr_session_batch: (first row, rows) of each group of the batch in flight
  bool has_moe = false, moe_select = false;  // moe_select: every routed layer can choose its experts' products on the device
  int* moe_sel = nullptr;     // one token's experts in ascending id (8 ints), then their router weights (8 floats)
  float* moe_y = nullptr;     // the selected experts' down results (8 x n_embd)
  char* moe_tables = nullptr;             // routing tables for max_batch rows, one device block
  float *moe_logits = nullptr, *moe_wts = nullptr, *moe_w = nullptr;
  int *moe_ids = nullptr, *moe_tok_of_row = nullptr, *moe_rows_of_tok = nullptr, *moe_fill = nullptr, *moe_first_row = nullptr;
  unsigned char* moe_local = nullptr;
  cudaGraphExec_t step_graph = nullptr;  // one decode step, captured once per kernel path
  int step_graph_path = -1, step_kernels = 0;
  bool use_graph = true;
};

namespace {

void session_release(llr_session* s) {
  for (float* p : s->attn_norm) if (p) cudaFree(p);
  for (float* p : s->ffn_norm) if (p) cudaFree(p);
  float* bufs[] = {s->out_norm, s->x, s->xn, s->q, s->k, s->v, s->attn, s->proj, s->gate, s->up, s->logits,
                   s->cache_k, s->cache_v, s->att_scratch, s->margins, s->last_x, s->arg_part};
  for (float* p : bufs) if (p) cudaFree(p);
  int* ibufs[] = {s->ids, s->pos_dev, s->count_dev, s->table_dev, s->row_pos, s->row_seq, s->last_rows};
  for (int* p : ibufs) if (p) cudaFree(p);
  if (s->step_graph) cudaGraphExecDestroy(s->step_graph);
  if (s->moe_tables) cudaFree(s->moe_tables);
  if (s->moe_sel) cudaFree(s->moe_sel);
  if (s->moe_y) cudaFree(s->moe_y);
  for (auto& M : s->moe) if (M && M->maps) cudaFree(M->maps);
  for (llr::Program* p : s->qkv_prog) program_destroy(p);
  for (llr::Program* p : s->gateup_prog) program_destroy(p);
  for (llr::Program* p : s->moe_gateup_prog) program_destroy(p);
  for (llr::Program* p : s->moe_down_prog) program_destroy(p);
  cudaGetLastError();
}

cudaError_t session_matmul(llr_exec* e, const llr_matrix* m, size_t tokens, const float* x, float* y) {
  void* scratch = nullptr;
  cudaError_t ce = ensure_scratch(e, m, tokens, &scratch);
  if (ce != cudaSuccess) return ce;
  return launch_matmul(view_of(m), x, y, (int64_t)tokens, e->stream, e->path, e->sm_count, e->err_flag, scratch, &e->ctr.launches);
}

KvView session_kv(const llr_session* s) {
  return KvView{s->cache_k, s->cache_v, s->table_dev, (int)s->block_tokens, (int)s->max_blocks, (int)s->cfg.n_layer};
}

// Blocks for positions [0, upto) of a sequence; new table entries go to the device on the executor's stream.
int session_reserve(llr_session* s, size_t seq, size_t upto) {
  llr_exec* e = s->owner;
  const size_t need = (upto + s->block_tokens - 1) / s->block_tokens;
  std::vector<int>& mine = s->seq_blocks[seq];
  const size_t had = mine.size();
  if (need <= had) return LLR_OK;
  if (need - had > s->free_blocks.size())
    return fail(e, LLR_ERR_OOM, "the session's KV pool has no free block left (" + std::to_string(s->n_blocks) + " blocks of " +
                                    std::to_string(s->block_tokens) + " positions)");
  while (mine.size() < need) { mine.push_back(s->free_blocks.back()); s->free_blocks.pop_back(); }
  cudaError_t ce = cudaMemcpyAsync(s->table_dev + seq * s->max_blocks + had, mine.data() + had, (need - had) * sizeof(int),
                                   cudaMemcpyHostToDevice, e->stream);
  if (ce != cudaSuccess) return fail_cuda(e, ce, "block table upload");
  // the host vector may grow again before the copy has run: pageable copies of this size are staged by the driver at call time
  return LLR_OK;
}

// The routed-expert layer of layer li over the n normalised rows in s->xn; the result (not yet added to the residual
// stream) goes to s->proj.  The per-expert row counts visit the host, which sizes the expert launches with them.
cudaError_t session_moe_ffn(llr_session* s, size_t li, size_t n) {
  llr_exec* e = s->owner;
  llr_session::Moe& M = *s->moe[li];
  const MoeShape& S = M.S;
  cudaError_t ce;
  if (n == 1 && s->moe_select && (e->path == PATH_AUTO || e->path == PATH_MMA)) {
    // One token: its experts are chosen on the device and their products read the weights through the chosen expert's
    // tensor map, so the step needs no row counts on the host (and can be replayed from a graph).  Same kernels and the
    // same order of additions as below: the result has the same bits.
    const size_t U = S.n_used, FF = S.n_ff, E = S.n_embd, NE = S.n_exp;
    int* sel = s->moe_sel;
    float* selw = (float*)(s->moe_sel + 8);
    const MatView vg = view_of(M.gate[0]), vd = view_of(M.down[0]);
    if ((ce = moe_route(e, &M.layer, S, 1, s->xn, s->moe_logits, s->moe_ids, s->moe_wts)) != cudaSuccess ||
        (ce = launch_select_sorted(s->moe_ids, s->moe_wts, (int)U, sel, selw, e->stream, &e->ctr.launches)) != cudaSuccess)
      return ce;
    llr::Program* pgu = s->moe_gateup_prog[li];
    llr::Program* pdn = s->moe_down_prog[li];
    if (pgu) {
      if ((ce = program_run(pgu, e->stream, e->err_flag, e->poll_limit, &e->ctr.launches)) != cudaSuccess) return ce;
    } else {
      for (size_t j = 0; j < U; ++j)
        if ((ce = launch_gemv_mma_select(vg, M.maps, sel + j, s->xn, s->gate + j * FF, e->stream, e->sm_count, e->err_flag, &e->ctr.launches)) != cudaSuccess ||
            (ce = launch_gemv_mma_select(vg, M.maps + NE * GEMV_MAP_BYTES, sel + j, s->xn, s->up + j * FF, e->stream, e->sm_count, e->err_flag,
                                         &e->ctr.launches)) != cudaSuccess)
          return ce;
    }
    if ((ce = launch_silu_mul(s->gate, s->up, (int64_t)(U * FF), e->stream, &e->ctr.launches)) != cudaSuccess) return ce;
    if (pdn) {
      if ((ce = program_run(pdn, e->stream, e->err_flag, e->poll_limit, &e->ctr.launches)) != cudaSuccess) return ce;
    } else {
      for (size_t j = 0; j < U; ++j)
        if ((ce = launch_gemv_mma_select(vd, M.maps + 2 * NE * GEMV_MAP_BYTES, sel + j, s->gate + j * FF, s->moe_y + j * E, e->stream, e->sm_count,
                                         e->err_flag, &e->ctr.launches)) != cudaSuccess)
          return ce;
    }
    return launch_combine_one(s->moe_y, selw, s->proj, (int)U, (int)E, e->stream, &e->ctr.launches);
  }
  if ((ce = moe_route(e, &M.layer, S, n, s->xn, s->moe_logits, s->moe_ids, s->moe_wts)) != cudaSuccess ||
      (ce = launch_bucket(s->moe_ids, s->moe_wts, s->moe_local, (int)n, (int)S.n_exp, (int)S.n_used, s->moe_first_row, s->moe_tok_of_row,
                          s->moe_rows_of_tok, s->moe_w, s->moe_fill, e->stream, &e->ctr.launches)) != cudaSuccess)
    return ce;
  std::vector<int> first_row(S.n_exp + 1, 0);
  if ((ce = cudaMemcpyAsync(first_row.data(), s->moe_first_row, (S.n_exp + 1) * sizeof(int), cudaMemcpyDeviceToHost, e->stream)) != cudaSuccess ||
      (ce = cudaStreamSynchronize(e->stream)) != cudaSuccess)
    return ce;
  e->ctr.d2h_bytes += (S.n_exp + 1) * sizeof(int);
  const size_t n_rows = n * S.n_used;
  if ((ce = grow_device(&e->dev_moe, &e->dev_moe_cap, moe_buffer_floats(S, n_rows) + 256)) != cudaSuccess) return ce;
  const MoeBuffers B = moe_carve((float*)(((uintptr_t)e->dev_moe + 255) & ~(uintptr_t)255), S, n_rows);
  if ((ce = moe_run_experts(e, &M.layer, S, first_row, s->xn, s->moe_tok_of_row, B)) != cudaSuccess) return ce;
  return launch_scatter_combine(B.y, s->moe_rows_of_tok, s->moe_w, s->proj, (int)n, (int)S.n_used, (int)S.n_embd, e->stream,
                                &e->ctr.launches);
}

// The layers over n rows whose token ids lie at ids_dev; rows stand where `rows` says.  Leaves the residual stream in
// s->x and the last ffn_down result, not yet added, in s->proj (returned through *pending).
cudaError_t session_layers(llr_session* s, const int* ids_dev, size_t n, const RowMap& rows, const float** pending_out) {
  llr_exec* e = s->owner;
  const llr_llama_config& c = s->cfg;
  const size_t E = c.n_embd, FF = c.n_ff;
  cudaStream_t st = e->stream;
  uint64_t* L = &e->ctr.launches;
  const KvView kv = session_kv(s);
  cudaError_t ce = launch_dequant_indexed(view_of(s->embd), ids_dev, (int64_t)n, s->x, st, L);
  const float* pending = nullptr;  // ffn_down result of the previous layer, not yet added to the residual stream
  for (size_t li = 0; li < c.n_layer && ce == cudaSuccess; ++li) {
    const llr_llama_layer& W = s->layers[li];
    if ((ce = launch_rmsnorm(s->x, pending, s->attn_norm[li], s->xn, (int)n, (int)E, c.rms_eps, st, L)) != cudaSuccess) break;
    const bool one_row_programs = n == 1 && (e->path == PATH_AUTO || e->path == PATH_MMA);
    if (one_row_programs && s->qkv_prog[li]) {
      if ((ce = program_run(s->qkv_prog[li], st, e->err_flag, e->poll_limit, L)) != cudaSuccess) break;
    } else {
      if ((ce = session_matmul(e, W.attn_q, n, s->xn, s->q)) != cudaSuccess) break;
      if ((ce = session_matmul(e, W.attn_k, n, s->xn, s->k)) != cudaSuccess) break;
      if ((ce = session_matmul(e, W.attn_v, n, s->xn, s->v)) != cudaSuccess) break;
    }
    if (n == 1) {  // a decode token: rotation and cache store happen inside the attention kernel
      if ((ce = launch_attention(s->q, kv, s->attn, s->att_scratch, rows, 1, (int)li, s->shape, st, L, s->k, s->v)) != cudaSuccess) break;
    } else {
      if ((ce = launch_rope_store(s->q, s->k, s->v, kv, rows, (int)n, (int)li, s->shape, st, L)) != cudaSuccess) break;
      // the automatic path takes the tensor cores for chunks of 64 rows and more of one sequence, as it does for the products
      const bool tc = e->path == PATH_AUTO && n >= TC_MIN_TOKENS;
      bool big_group = false;
      if (tc && rows.row_seq)
        for (const auto& gr : s->batch_groups) big_group = big_group || gr.second >= (size_t)TC_MIN_TOKENS;
      if (big_group) {
        // a ragged batch: every group of 64 rows and more on its own (tensor cores), the runs of smaller groups between them together
        const size_t q_row = (size_t)c.n_head * c.head_dim, rec_row = attention_scratch_floats(1, s->shape);
        auto part = [&](size_t t0, size_t len, bool one) {
          return launch_attention(s->q + t0 * q_row, kv, s->attn + t0 * q_row, s->att_scratch + t0 * rec_row,
                                  RowMap{nullptr, rows.row_pos + t0, rows.row_seq + t0}, (int)len, (int)li, s->shape, st, L, nullptr, nullptr, one, one);
        };
        size_t run0 = 0, at = 0;
        for (const auto& gr : s->batch_groups) {
          if (gr.second >= (size_t)TC_MIN_TOKENS) {
            if (at > run0 && (ce = part(run0, at - run0, false)) != cudaSuccess) break;
            if ((ce = part(gr.first, gr.second, true)) != cudaSuccess) break;
            run0 = gr.first + gr.second;
          }
          at = gr.first + gr.second;
        }
        if (ce == cudaSuccess && at > run0) ce = part(run0, at - run0, false);
        if (ce != cudaSuccess) break;
      } else if ((ce = launch_attention(s->q, kv, s->attn, s->att_scratch, rows, (int)n, (int)li, s->shape, st, L, nullptr, nullptr, tc)) != cudaSuccess) {
        break;
      }
    }
    if ((ce = session_matmul(e, W.attn_output, n, s->attn, s->proj)) != cudaSuccess) break;
    if ((ce = launch_rmsnorm(s->x, s->proj, s->ffn_norm[li], s->xn, (int)n, (int)E, c.rms_eps, st, L)) != cudaSuccess) break;
    if (s->moe[li]) {  // routed experts stand where the dense FFN stands (llama_moe_into decode.rs:10366)
      if ((ce = session_moe_ffn(s, li, n)) != cudaSuccess) break;
      pending = s->proj;
      continue;
    }
    if (one_row_programs && s->gateup_prog[li]) {
      if ((ce = program_run(s->gateup_prog[li], st, e->err_flag, e->poll_limit, L)) != cudaSuccess) break;
    } else {
      if ((ce = session_matmul(e, W.ffn_gate, n, s->xn, s->gate)) != cudaSuccess) break;
      if ((ce = session_matmul(e, W.ffn_up, n, s->xn, s->up)) != cudaSuccess) break;
    }
    if ((ce = launch_swiglu(s->gate, s->up, (int64_t)(n * FF), st, L)) != cudaSuccess) break;
    if ((ce = session_matmul(e, W.ffn_down, n, s->gate, s->proj)) != cudaSuccess) break;
    pending = s->proj;
  }
  *pending_out = pending;
  return ce;
}

// One forward pass of sequence 0 over `n` tokens at its device-side position; with_logits: the last token's logits, then
// (generate) argmax into ids[0] and the history, and the position advanced by n.
cudaError_t session_forward(llr_session* s, const int* ids_dev, size_t n, bool with_logits, bool generate) {
  llr_exec* e = s->owner;
  const llr_llama_config& c = s->cfg;
  const size_t E = c.n_embd;
  cudaStream_t st = e->stream;
  uint64_t* L = &e->ctr.launches;
  const float* pending = nullptr;
  cudaError_t ce = session_layers(s, ids_dev, n, RowMap{s->pos_dev, nullptr, nullptr}, &pending);
  if (ce != cudaSuccess) return ce;
  if (with_logits) {
    // LogitsKind::Last (decode.rs:3058-3079): the last row only
    float* xl = s->x + (n - 1) * E;
    if ((ce = launch_rmsnorm(xl, pending ? pending + (n - 1) * E : nullptr, s->out_norm, s->xn, 1, (int)E, c.rms_eps, st, L)) != cudaSuccess) return ce;
    if ((ce = session_matmul(e, s->output, 1, s->xn, s->logits)) != cudaSuccess) return ce;
    // generation: the winner goes to ids[0] (read by the next step) and to the history
    return launch_argmax_advance(s->logits, generate ? (int)c.n_vocab : 0, s->ids, s->margins, s->pos_dev, (int)n,
                                 generate ? s->count_dev : nullptr, s->arg_part, st, L);
  }
  return launch_argmax_advance(nullptr, 0, nullptr, nullptr, s->pos_dev, (int)n, nullptr, nullptr, st, L);
}

int session_ids(llr_session* s, size_t n) {
  if (n <= s->ids_cap) return LLR_OK;
  cudaStreamSynchronize(s->owner->stream);
  if (s->ids) cudaFree(s->ids);
  if (s->margins) cudaFree(s->margins);
  s->ids = nullptr; s->margins = nullptr; s->ids_cap = 0;
  cudaError_t ce = cudaMalloc((void**)&s->ids, (n + 2) * sizeof(int));
  if (ce == cudaSuccess) ce = cudaMalloc((void**)&s->margins, (n + 2) * sizeof(float));
  if (ce != cudaSuccess) return fail_cuda(s->owner, ce, "token buffer");
  s->ids_cap = n;
  if (s->step_graph) { cudaGraphExecDestroy(s->step_graph); s->step_graph = nullptr; }  // the captured step addresses the old buffers
  return LLR_OK;
}

int session_create(llr_exec* e, const llr_llama_model* m, size_t n_seq, size_t kv_blocks, size_t block_tokens, llr_session** out) {
  if (!e) return LLR_ERR_INVALID;
  if (!out) return fail(e, LLR_ERR_INVALID, "null output pointer");
  *out = nullptr;
  if (!m || !m->layers || !m->token_embd) return fail(e, LLR_ERR_INVALID, "null model");
  const llr_llama_config& c = m->cfg;
  if (c.n_layer == 0 || c.n_embd == 0 || c.n_head == 0 || c.n_head_kv == 0 || c.head_dim == 0 || c.n_ff == 0 || c.n_vocab == 0 ||
      c.n_ctx == 0 || c.n_head % c.n_head_kv != 0 || c.n_head / c.n_head_kv > 8 || c.head_dim % 2 != 0 || c.head_dim > 256 ||
      c.n_embd % 8 != 0 || c.n_ctx > (1u << 20) || !(c.rms_eps >= 0.0f) || !(c.rope_base > 0.0f))
    return fail(e, LLR_ERR_INVALID, "llama configuration out of range (grouped-query ratio at most 8, even head_dim up to 256, n_embd % 8 == 0)");
  if (n_seq == 0 || n_seq > 4096 || block_tokens == 0 || block_tokens > c.n_ctx)
    return fail(e, LLR_ERR_INVALID, "a session holds 1..4096 sequences and KV blocks of 1..n_ctx positions");
  const size_t E = c.n_embd, QW = (size_t)c.n_head * c.head_dim, KVW = (size_t)c.n_head_kv * c.head_dim, FF = c.n_ff, V = c.n_vocab;
  auto shape_ok = [&](const llr_matrix* w, size_t rows, size_t cols) {
    return w && w->owner == e && (size_t)w->rows == rows && (size_t)w->cols == cols;
  };
  size_t max_expert = 0, max_used = 0;  // over the layers with routed experts
  const llr_matrix* output = m->output ? m->output : m->token_embd;
  if (!shape_ok(m->token_embd, V, E) || !shape_ok(output, V, E))
    return fail(e, LLR_ERR_INVALID, "token_embd / output must be n_vocab x n_embd matrices of this executor");
  for (uint32_t li = 0; li < c.n_layer; ++li) {
    const llr_llama_layer& W = m->layers[li];
    bool ffn_ok = shape_ok(W.ffn_gate, FF, E) && shape_ok(W.ffn_up, FF, E) && shape_ok(W.ffn_down, E, FF);
    if (W.n_expert > 0) {
      ffn_ok = W.n_expert_used > 0 && W.n_expert_used <= W.n_expert && W.n_expert <= 4096 && shape_ok(W.ffn_gate_inp, W.n_expert, E) &&
               W.ffn_gate_exps && W.ffn_up_exps && W.ffn_down_exps && E % 4 == 0;
      for (uint32_t ex = 0; ex < W.n_expert && ffn_ok; ++ex)
        ffn_ok = shape_ok(W.ffn_gate_exps[ex], FF, E) && shape_ok(W.ffn_up_exps[ex], FF, E) && shape_ok(W.ffn_down_exps[ex], E, FF);
      if (ffn_ok) { max_expert = std::max(max_expert, (size_t)W.n_expert); max_used = std::max(max_used, (size_t)W.n_expert_used); }
    }
    if (!shape_ok(W.attn_q, QW, E) || !shape_ok(W.attn_k, KVW, E) || !shape_ok(W.attn_v, KVW, E) || !shape_ok(W.attn_output, E, QW) || !ffn_ok)
      return fail(e, LLR_ERR_INVALID, "blk." + std::to_string(li) + ": matrix shapes do not match the configuration (or another executor owns them)");
  }
  DeviceGuard guard(e->device);
  llr_session* s = new (std::nothrow) llr_session();
  if (!s) return fail(e, LLR_ERR_OOM, "host allocation failed");
  s->owner = e;
  s->cfg = c;
  s->embd = m->token_embd;
  s->output = output;
  s->layers.assign(m->layers, m->layers + c.n_layer);
  s->moe.resize(c.n_layer);
  for (uint32_t li = 0; li < c.n_layer; ++li) {
    const llr_llama_layer& W = m->layers[li];
    if (W.n_expert == 0) continue;
    std::unique_ptr<llr_session::Moe> M(new llr_session::Moe);
    M->gate.assign(W.ffn_gate_exps, W.ffn_gate_exps + W.n_expert);
    M->up.assign(W.ffn_up_exps, W.ffn_up_exps + W.n_expert);
    M->down.assign(W.ffn_down_exps, W.ffn_down_exps + W.n_expert);
    M->layer = llr_moe_layer{W.n_expert, W.n_expert_used, 1u, W.ffn_gate_inp, M->gate.data(), M->up.data(), M->down.data()};
    M->S.n_embd = E; M->S.n_ff = FF; M->S.n_exp = W.n_expert; M->S.n_used = W.n_expert_used;
    M->S.local.assign(W.n_expert, 1);
    s->moe[li] = std::move(M);
    s->layers[li].ffn_gate_exps = s->layers[li].ffn_up_exps = s->layers[li].ffn_down_exps = nullptr;  // the copies above are the ones used
    s->has_moe = true;
  }
  const float n_rot = (float)(uint16_t)c.head_dim;
  s->shape = WalkShape{(int)c.n_embd, (int)c.n_head, (int)c.n_head_kv, (int)c.head_dim, (int)c.n_ff, (int)c.n_ctx, c.rms_eps, c.rope_base,
                       std::pow(c.rope_base, -2.0f / n_rot)};  // decode.rs:11578: theta_scale in f32
  s->max_batch = c.n_ctx * n_seq < 512 ? c.n_ctx * n_seq : 512;
  s->n_seq = n_seq;
  s->block_tokens = block_tokens;
  s->max_blocks = (c.n_ctx + block_tokens - 1) / block_tokens;
  s->n_blocks = kv_blocks ? kv_blocks : s->max_blocks * n_seq;
  s->position.assign(n_seq, 0);
  s->seq_blocks.assign(n_seq, {});
  s->have_logits.assign(n_seq, 0);
  for (size_t b = s->n_blocks; b-- > 0;) s->free_blocks.push_back((int)b);
  s->logits_rows = n_seq;
  const size_t B = s->max_batch;
  cudaError_t ce = cudaSuccess;
  auto alloc = [&](float** p, size_t n) { if (ce == cudaSuccess) ce = cudaMalloc((void**)p, n * sizeof(float)); };
  auto ialloc = [&](int** p, size_t n) { if (ce == cudaSuccess) ce = cudaMalloc((void**)p, n * sizeof(int)); };
  auto norm = [&](const float* host, float** dev) {
    *dev = nullptr;
    if (!host || ce != cudaSuccess) return;
    ce = cudaMalloc((void**)dev, E * sizeof(float));
    if (ce == cudaSuccess) ce = cudaMemcpy(*dev, host, E * sizeof(float), cudaMemcpyHostToDevice);
  };
  s->attn_norm.assign(c.n_layer, nullptr);
  s->ffn_norm.assign(c.n_layer, nullptr);
  for (uint32_t li = 0; li < c.n_layer; ++li) { norm(m->layers[li].attn_norm, &s->attn_norm[li]); norm(m->layers[li].ffn_norm, &s->ffn_norm[li]); }
  norm(m->output_norm, &s->out_norm);
  alloc(&s->x, B * E); alloc(&s->xn, B * E); alloc(&s->q, B * QW); alloc(&s->k, B * KVW); alloc(&s->v, B * KVW);
  alloc(&s->attn, B * QW); alloc(&s->proj, B * E); alloc(&s->gate, B * FF); alloc(&s->up, B * FF);
  alloc(&s->logits, s->logits_rows * V); alloc(&s->last_x, n_seq * E); alloc(&s->arg_part, 512);
  const size_t pool = s->n_blocks * c.n_layer * c.n_head_kv * block_tokens * c.head_dim;
  alloc(&s->cache_k, pool); alloc(&s->cache_v, pool);
  alloc(&s->att_scratch, attention_scratch_floats((int)B, s->shape));
  ialloc(&s->pos_dev, 1); ialloc(&s->count_dev, 1);
  ialloc(&s->table_dev, n_seq * s->max_blocks); ialloc(&s->row_pos, B); ialloc(&s->row_seq, B); ialloc(&s->last_rows, n_seq);
  if (ce == cudaSuccess) ce = cudaMemset(s->pos_dev, 0, sizeof(int));
  if (ce == cudaSuccess) ce = cudaMemset(s->table_dev, 0, n_seq * s->max_blocks * sizeof(int));
  if (const char* g = std::getenv("LLR_SESSION_GRAPH")) s->use_graph = s->use_graph && std::strcmp(g, "0") != 0;
  if (max_expert > 0 && ce == cudaSuccess) {
    // One-token steps choose their experts' products on the device when every expert matrix of every routed layer goes
    // through the streaming decode kernel in one format per kind: tensor maps gate | up | down of all experts per layer.
    s->moe_select = max_used <= 8 && B >= max_used;
    for (uint32_t li = 0; li < c.n_layer && s->moe_select; ++li) {
      if (!s->moe[li]) continue;
      const llr_session::Moe& M = *s->moe[li];
      for (size_t ex = 0; ex < M.S.n_exp && s->moe_select; ++ex)
        s->moe_select = gemv_mma_supported(view_of(M.gate[ex])) && gemv_mma_supported(view_of(M.up[ex])) && gemv_mma_supported(view_of(M.down[ex])) &&
                        M.gate[ex]->dtype == M.gate[0]->dtype && M.up[ex]->dtype == M.gate[0]->dtype && M.down[ex]->dtype == M.down[0]->dtype;
    }
    for (uint32_t li = 0; li < c.n_layer && s->moe_select && ce == cudaSuccess; ++li) {
      if (!s->moe[li]) continue;
      llr_session::Moe& M = *s->moe[li];
      const size_t NE = M.S.n_exp;
      std::vector<char> host(3 * NE * GEMV_MAP_BYTES);
      for (size_t ex = 0; ex < NE && ce == cudaSuccess; ++ex) {
        if ((ce = gemv_mma_encode_map(view_of(M.gate[ex]), host.data() + ex * GEMV_MAP_BYTES)) != cudaSuccess ||
            (ce = gemv_mma_encode_map(view_of(M.up[ex]), host.data() + (NE + ex) * GEMV_MAP_BYTES)) != cudaSuccess ||
            (ce = gemv_mma_encode_map(view_of(M.down[ex]), host.data() + (2 * NE + ex) * GEMV_MAP_BYTES)) != cudaSuccess)
          break;
      }
      if (ce == cudaSuccess) ce = cudaMalloc((void**)&M.maps, host.size());
      if (ce == cudaSuccess) ce = cudaMemcpy(M.maps, host.data(), host.size(), cudaMemcpyHostToDevice);
    }
    if (s->moe_select && ce == cudaSuccess) {
      ce = cudaMalloc((void**)&s->moe_sel, 8 * sizeof(int) + 8 * sizeof(float));
      if (ce == cudaSuccess) ce = cudaMalloc((void**)&s->moe_y, 8 * E * sizeof(float));
    }
    const size_t n_rows = B * max_used;
    auto up256 = [](size_t v) { return (v + 255) & ~(size_t)255; };
    size_t at = 0;
    auto take = [&](size_t bytes) { const size_t o = at; at = up256(at + bytes); return o; };
    const size_t o_logits = take(B * max_expert * 4), o_ids = take(n_rows * 4), o_wts = take(n_rows * 4), o_tor = take(n_rows * 4),
                 o_rot = take(n_rows * 4), o_w = take(n_rows * 4), o_fill = take(B * 4), o_first = take((max_expert + 1) * 4),
                 o_local = take(max_expert);
    if (ce == cudaSuccess) ce = cudaMalloc((void**)&s->moe_tables, at);
    if (ce == cudaSuccess) {
      char* tb = s->moe_tables;
      s->moe_logits = (float*)(tb + o_logits); s->moe_ids = (int*)(tb + o_ids); s->moe_wts = (float*)(tb + o_wts);
      s->moe_tok_of_row = (int*)(tb + o_tor); s->moe_rows_of_tok = (int*)(tb + o_rot); s->moe_w = (float*)(tb + o_w);
      s->moe_fill = (int*)(tb + o_fill); s->moe_first_row = (int*)(tb + o_first); s->moe_local = (unsigned char*)(tb + o_local);
      ce = cudaMemset(s->moe_local, 1, max_expert);
    }
  }
  // One launch for the products of a layer that share their input, where the streaming decode kernel takes all of them
  s->qkv_prog.assign(c.n_layer, nullptr);
  s->gateup_prog.assign(c.n_layer, nullptr);
  auto group = [&](std::initializer_list<std::pair<const llr_matrix*, float*>> items, llr::Program** slot) {
    std::vector<ProgEntry> pe;
    std::vector<int> phase;
    for (const auto& it : items) {
      const MatView v = view_of(it.first);
      if (!prog_entry_supported(v)) return;
      ProgEntry E{};
      E.w = v.w; E.x = s->xn; E.y = it.second; E.row_bytes = v.row_bytes;
      E.rows = (int)v.rows; E.cols = (int)v.cols; E.dtype = v.dtype; E.tokens = 1; E.y_ld = v.rows;
      E.x_phase = E.x2_phase = E.resid_phase = -1;
      pe.push_back(E);
      phase.push_back(0);
    }
    std::string msg;
    if (ce == cudaSuccess && program_create(pe, phase, e->sm_count, false, nullptr, slot, &msg) != cudaSuccess) { *slot = nullptr; cudaGetLastError(); }
  };
  for (uint32_t li = 0; li < c.n_layer && ce == cudaSuccess; ++li) {
    const llr_llama_layer& W = s->layers[li];
    group({{W.attn_q, s->q}, {W.attn_k, s->k}, {W.attn_v, s->v}}, &s->qkv_prog[li]);
    if (!s->moe[li]) group({{W.ffn_gate, s->gate}, {W.ffn_up, s->up}}, &s->gateup_prog[li]);
  }
  s->moe_gateup_prog.assign(c.n_layer, nullptr);
  s->moe_down_prog.assign(c.n_layer, nullptr);
  for (uint32_t li = 0; li < c.n_layer && ce == cudaSuccess && s->moe_select; ++li) {
    if (!s->moe[li]) continue;
    const llr_session::Moe& M = *s->moe[li];
    const MatView vg = view_of(M.gate[0]), vd = view_of(M.down[0]);
    // slot j of the step's sorted experts: x, y and the base of its kind's maps
    auto select_group = [&](const MatView& v, std::initializer_list<std::pair<float*, size_t>> kinds, const float* x, size_t x_step,
                            size_t y_step, llr::Program** slot) {
      if (!prog_entry_supported(v)) return;
      std::vector<ProgEntry> pe;
      for (size_t j = 0; j < M.S.n_used; ++j)
        for (const auto& kind : kinds) {
          ProgEntry E{};
          E.w = v.w; E.x = x + j * x_step; E.y = kind.first + j * y_step; E.row_bytes = v.row_bytes;
          E.rows = (int)v.rows; E.cols = (int)v.cols; E.dtype = v.dtype; E.tokens = 1; E.y_ld = v.rows;
          E.x_phase = E.x2_phase = E.resid_phase = -1;
          E.sel_slot = (int)j; E.map_base = (int)kind.second;
          pe.push_back(E);
        }
      std::string msg;
      if (program_create(pe, std::vector<int>(pe.size(), 0), e->sm_count, false, nullptr, slot, &msg) != cudaSuccess ||
          program_set_select(*slot, M.maps, s->moe_sel) != cudaSuccess) {
        if (*slot) program_destroy(*slot);
        *slot = nullptr;
        cudaGetLastError();
      }
    };
    select_group(vg, {{s->gate, 0}, {s->up, M.S.n_exp}}, s->xn, 0, M.S.n_ff, &s->moe_gateup_prog[li]);
    select_group(vd, {{s->moe_y, 2 * M.S.n_exp}}, s->gate, M.S.n_ff, E, &s->moe_down_prog[li]);
  }
  if (ce != cudaSuccess) {
    session_release(s);
    delete s;
    return fail_cuda(e, ce, "session buffers");
  }
  *out = s;
  return LLR_OK;
}

}  // namespace

int llr_session_create(llr_exec* e, const llr_llama_model* m, llr_session** out) { return session_create(e, m, 1, 0, 16, out); }

int llr_session_create_paged(llr_exec* e, const llr_llama_model* m, size_t n_seq, size_t kv_blocks, size_t block_tokens,
                             llr_session** out) {
  return session_create(e, m, n_seq, kv_blocks, block_tokens, out);
}

int llr_session_free(llr_session* s) {
  if (!s) return LLR_OK;
  if (s->owner) {
    DeviceGuard guard(s->owner->device);
    cudaStreamSynchronize(s->owner->stream);
    session_release(s);
  }
  delete s;
  return LLR_OK;
}

int llr_session_seq_reset(llr_session* s, size_t seq) {
  if (!s || !s->owner) return LLR_ERR_INVALID;
  if (seq >= s->n_seq) return fail(s->owner, LLR_ERR_INVALID, "sequence index out of range");
  DeviceGuard guard(s->owner->device);
  if (seq == 0) {
    cudaError_t ce = cudaMemsetAsync(s->pos_dev, 0, sizeof(int), s->owner->stream);
    if (ce != cudaSuccess) return fail_cuda(s->owner, ce, "session reset");
  }
  for (int b : s->seq_blocks[seq]) s->free_blocks.push_back(b);  // its blocks go back to the pool
  s->seq_blocks[seq].clear();
  s->position[seq] = 0;
  s->have_logits[seq] = 0;
  return LLR_OK;
}

int llr_session_seq_truncate(llr_session* s, size_t seq, size_t n_keep) {
  if (!s || !s->owner) return LLR_ERR_INVALID;
  llr_exec* e = s->owner;
  if (seq >= s->n_seq) return fail(e, LLR_ERR_INVALID, "sequence index out of range");
  if (n_keep > s->position[seq]) return fail(e, LLR_ERR_INVALID, "a sequence cannot be truncated beyond its position");
  if (n_keep == s->position[seq]) return LLR_OK;
  DeviceGuard guard(e->device);
  if (seq == 0) {  // sequence 0 keeps its position on the device too (graph replay advances it there)
    const int p = (int)n_keep;
    cudaError_t ce = cudaMemcpyAsync(s->pos_dev, &p, sizeof(int), cudaMemcpyHostToDevice, e->stream);
    if (ce != cudaSuccess) return fail_cuda(e, ce, "session truncate");
  }
  // Blocks wholly behind the kept prefix go back to the pool; work already queued on the stream that reads them
  // runs before anything that could write them again.
  const size_t keep_blocks = (n_keep + s->block_tokens - 1) / s->block_tokens;
  std::vector<int>& mine = s->seq_blocks[seq];
  while (mine.size() > keep_blocks) { s->free_blocks.push_back(mine.back()); mine.pop_back(); }
  s->position[seq] = n_keep;
  s->have_logits[seq] = 0;
  return LLR_OK;
}

int llr_session_reset(llr_session* s) {
  if (!s || !s->owner) return LLR_ERR_INVALID;
  for (size_t q = 0; q < s->n_seq; ++q) {
    int rc = llr_session_seq_reset(s, q);
    if (rc) return rc;
  }
  return LLR_OK;
}

int llr_session_position(const llr_session* s, size_t* position) {
  if (!s || !position) return LLR_ERR_INVALID;
  *position = s->position[0];
  return LLR_OK;
}

int llr_session_seq_position(const llr_session* s, size_t seq, size_t* position) {
  if (!s || !position || seq >= s->n_seq) return LLR_ERR_INVALID;
  *position = s->position[seq];
  return LLR_OK;
}

int llr_session_prefill(llr_session* s, const int32_t* tokens, size_t n, float* last_logits) {
  if (!s || !s->owner) return LLR_ERR_INVALID;
  llr_exec* e = s->owner;
  if (!tokens || n == 0) return fail(e, LLR_ERR_INVALID, "prefill needs at least one token");
  if (s->position[0] + n > s->cfg.n_ctx) return fail(e, LLR_ERR_INVALID, "the sequence would exceed the session's context length");
  for (size_t i = 0; i < n; ++i)
    if (tokens[i] < 0 || (uint32_t)tokens[i] >= s->cfg.n_vocab) return fail(e, LLR_ERR_INVALID, "token id out of range");
  DeviceGuard guard(e->device);
  int rc = session_ids(s, n > 1 ? n : 1);
  if (rc) return rc;
  if ((rc = session_reserve(s, 0, s->position[0] + n))) return rc;
  cudaError_t ce = cudaMemcpyAsync(s->ids + 1, tokens, n * sizeof(int), cudaMemcpyHostToDevice, e->stream);
  for (size_t t0 = 0; t0 < n && ce == cudaSuccess; t0 += s->max_batch) {
    const size_t m = n - t0 < s->max_batch ? n - t0 : s->max_batch;
    ce = session_forward(s, s->ids + 1 + t0, m, t0 + m == n, false);
  }
  if (ce == cudaSuccess && last_logits)
    ce = cudaMemcpyAsync(last_logits, s->logits, s->cfg.n_vocab * sizeof(float), cudaMemcpyDeviceToHost, e->stream);
  if (ce == cudaSuccess) ce = cudaStreamSynchronize(e->stream);
  if (ce != cudaSuccess) return fail_cuda(e, ce, "prefill");
  if (take_device_error(e) != 0) return fail(e, LLR_ERR_CUDA, "a device-side wait ran out of iterations");
  s->position[0] += n;
  s->have_logits[0] = 1;
  return LLR_OK;
}

int llr_session_decode(llr_session* s, size_t n_gen, int32_t* out_ids, float* out_margin) {
  if (!s || !s->owner) return LLR_ERR_INVALID;
  llr_exec* e = s->owner;
  if (!out_ids || n_gen == 0) return fail(e, LLR_ERR_INVALID, "decode needs a token count and an output buffer");
  if (!s->have_logits[0]) return fail(e, LLR_ERR_INVALID, "decode needs logits: prefill at least one token first");
  if (s->position[0] + n_gen > s->cfg.n_ctx) return fail(e, LLR_ERR_INVALID, "the sequence would exceed the session's context length");
  DeviceGuard guard(e->device);
  int rc = session_ids(s, n_gen + 1);
  if (rc) return rc;
  if ((rc = session_reserve(s, 0, s->position[0] + n_gen))) return rc;  // every block the steps below will write
  // Token 0 = argmax of the current logits.  Every step then reads its token from ids[0], runs the walk, and its
  // argmax writes the next token to ids[0] and appends it to the history ids[1..]; the position and the count live on
  // the device too.  So all steps are the same sequence of launches: the second one is captured into a graph, which
  // the remaining steps replay (several hundred launches per token otherwise cost more host time than device time).
  cudaError_t ce = cudaMemsetAsync(s->count_dev, 0, sizeof(int), e->stream);
  if (ce == cudaSuccess)
    ce = launch_argmax_advance(s->logits, (int)s->cfg.n_vocab, s->ids, s->margins, nullptr, 0, s->count_dev, s->arg_part, e->stream, &e->ctr.launches);
  size_t done = 0;
  if (ce == cudaSuccess) { ce = session_forward(s, s->ids, 1, true, true); ++done; }  // also initialises per-kernel launch state before any capture
  // a step with routed layers is the same sequence of launches only when its experts are chosen on the device
  const bool graph_ok = s->use_graph && (!s->has_moe || (s->moe_select && (e->path == PATH_AUTO || e->path == PATH_MMA)));
  if (ce == cudaSuccess && graph_ok && n_gen > 2 && (!s->step_graph || s->step_graph_path != e->path)) {
    if (s->step_graph) { cudaGraphExecDestroy(s->step_graph); s->step_graph = nullptr; }
    cudaGraph_t graph = nullptr;
    const uint64_t launches_before = e->ctr.launches;
    ce = cudaStreamBeginCapture(e->stream, cudaStreamCaptureModeThreadLocal);
    if (ce == cudaSuccess) {
      const cudaError_t fe = session_forward(s, s->ids, 1, true, true);
      ce = cudaStreamEndCapture(e->stream, &graph);
      if (fe != cudaSuccess) ce = fe;
    }
    const uint64_t captured = e->ctr.launches - launches_before;
    e->ctr.launches = launches_before;  // captured, not launched
    if (ce == cudaSuccess) ce = cudaGraphInstantiate(&s->step_graph, graph, 0);
    if (graph) cudaGraphDestroy(graph);
    if (ce != cudaSuccess) {  // fall back to plain launches
      cudaGetLastError();
      if (s->step_graph) { cudaGraphExecDestroy(s->step_graph); s->step_graph = nullptr; }
      s->use_graph = false;
      ce = cudaSuccess;
    } else {
      s->step_graph_path = e->path;
      s->step_kernels = (int)captured;
    }
  }
  for (; done < n_gen && ce == cudaSuccess; ++done) {
    if (graph_ok && s->use_graph && s->step_graph && s->step_graph_path == e->path) {
      ce = cudaGraphLaunch(s->step_graph, e->stream);
      e->ctr.launches += (uint64_t)s->step_kernels;
    } else {
      ce = session_forward(s, s->ids, 1, true, true);
    }
  }
  // the last step's argmax produced one token more than asked for: it is the next call's token 0 again
  if (ce == cudaSuccess) ce = cudaMemcpyAsync(out_ids, s->ids + 1, n_gen * sizeof(int), cudaMemcpyDeviceToHost, e->stream);
  if (ce == cudaSuccess && out_margin) ce = cudaMemcpyAsync(out_margin, s->margins, n_gen * sizeof(float), cudaMemcpyDeviceToHost, e->stream);
  if (ce == cudaSuccess) ce = cudaStreamSynchronize(e->stream);
  if (ce != cudaSuccess) return fail_cuda(e, ce, "decode");
  if (take_device_error(e) != 0) return fail(e, LLR_ERR_CUDA, "a device-side wait ran out of iterations");
  s->position[0] += n_gen;
  e->ctr.d2h_bytes += n_gen * sizeof(int);
  return LLR_OK;
}

int llr_session_logits(llr_session* s, float* logits, size_t n) {
  if (!s || !s->owner) return LLR_ERR_INVALID;
  llr_exec* e = s->owner;
  if (!logits || n != s->cfg.n_vocab || !s->have_logits[0]) return fail(e, LLR_ERR_INVALID, "logits buffer does not match n_vocab, or no token has been run");
  DeviceGuard guard(e->device);
  cudaError_t ce = cudaMemcpyAsync(logits, s->logits, n * sizeof(float), cudaMemcpyDeviceToHost, e->stream);
  if (ce == cudaSuccess) ce = cudaStreamSynchronize(e->stream);
  if (ce != cudaSuccess) return fail_cuda(e, ce, "logits download");
  return LLR_OK;
}

// A ragged batch: group g appends counts[g] tokens to sequence seq_ids[g].  The groups are flattened, in ascending sequence
// id, into one activation matrix of sum(counts) rows, so that every matrix product of the step runs once over all of them
// (Engine::try_compute_batch, engine.rs:1215-1274 -> prefill_batch decode.rs:2579); attention and the KV cache go by
// each row's own sequence and position.  last_logits (optional, n_groups x n_vocab, in the caller's group order) and
// next_ids (optional, n_groups) receive each group's last-row logits and their greedy argmax.
int llr_session_batch(llr_session* s, size_t n_groups, const uint32_t* seq_ids, const uint32_t* counts, const int32_t* tokens,
                      float* last_logits, int32_t* next_ids) {
  if (!s || !s->owner) return LLR_ERR_INVALID;
  llr_exec* e = s->owner;
  if (n_groups == 0 || n_groups > s->n_seq || !seq_ids || !counts || !tokens) return fail(e, LLR_ERR_INVALID, "a batch needs 1..n_seq groups");
  const llr_llama_config& c = s->cfg;
  const size_t E = c.n_embd, V = c.n_vocab;
  size_t total = 0;
  std::vector<size_t> first(n_groups);
  std::vector<char> seen(s->n_seq, 0);
  for (size_t g = 0; g < n_groups; ++g) {
    if (seq_ids[g] >= s->n_seq || seen[seq_ids[g]]) return fail(e, LLR_ERR_INVALID, "sequence index out of range or used twice in one batch");
    seen[seq_ids[g]] = 1;
    if (counts[g] == 0) return fail(e, LLR_ERR_INVALID, "an empty group");
    if (s->position[seq_ids[g]] + counts[g] > c.n_ctx) return fail(e, LLR_ERR_INVALID, "a sequence would exceed the session's context length");
    first[g] = total;
    total += counts[g];
  }
  if (total > s->max_batch) return fail(e, LLR_ERR_INVALID, "the batch has more rows than the session's chunk size (" + std::to_string(s->max_batch) + ")");
  for (size_t i = 0; i < total; ++i)
    if (tokens[i] < 0 || (uint32_t)tokens[i] >= c.n_vocab) return fail(e, LLR_ERR_INVALID, "token id out of range");
  DeviceGuard guard(e->device);
  int rc = session_ids(s, total);
  if (rc) return rc;
  // flatten in ascending sequence id (the engine sorts its jobs by slot)
  std::vector<size_t> order(n_groups);
  for (size_t g = 0; g < n_groups; ++g) order[g] = g;
  std::sort(order.begin(), order.end(), [&](size_t a, size_t b) { return seq_ids[a] < seq_ids[b]; });
  std::vector<int> ids(total), rpos(total), rseq(total), last(n_groups);
  size_t r = 0;
  s->batch_groups.clear();
  for (size_t oi = 0; oi < n_groups; ++oi) {
    const size_t g = order[oi], q = seq_ids[g];
    if ((rc = session_reserve(s, q, s->position[q] + counts[g]))) return rc;
    s->batch_groups.emplace_back(r, (size_t)counts[g]);
    for (size_t i = 0; i < counts[g]; ++i, ++r) {
      ids[r] = tokens[first[g] + i];
      rpos[r] = (int)(s->position[q] + i);
      rseq[r] = (int)q;
    }
    last[oi] = (int)r - 1;
  }
  cudaStream_t st = e->stream;
  uint64_t* L = &e->ctr.launches;
  cudaError_t ce;
  if ((ce = cudaMemcpyAsync(s->ids + 1, ids.data(), total * sizeof(int), cudaMemcpyHostToDevice, st)) != cudaSuccess ||
      (ce = cudaMemcpyAsync(s->row_pos, rpos.data(), total * sizeof(int), cudaMemcpyHostToDevice, st)) != cudaSuccess ||
      (ce = cudaMemcpyAsync(s->row_seq, rseq.data(), total * sizeof(int), cudaMemcpyHostToDevice, st)) != cudaSuccess ||
      (ce = cudaMemcpyAsync(s->last_rows, last.data(), n_groups * sizeof(int), cudaMemcpyHostToDevice, st)) != cudaSuccess)
    return fail_cuda(e, ce, "batch upload");
  const float* pending = nullptr;
  if ((ce = session_layers(s, s->ids + 1, total, RowMap{nullptr, s->row_pos, s->row_seq}, &pending)) != cudaSuccess)
    return fail_cuda(e, ce, "kernel launch");
  // each group's last row: residual add, output norm, logits (LogitsKind::Last per sequence)
  if (pending && (ce = launch_add(s->x, pending, (int64_t)(total * E), st, L)) != cudaSuccess) return fail_cuda(e, ce, "kernel launch");
  if ((ce = launch_gather_rows(s->x, s->last_rows, s->last_x, (int)n_groups, (int)E, st, L)) != cudaSuccess ||
      (ce = launch_rmsnorm(s->last_x, nullptr, s->out_norm, s->last_x, (int)n_groups, (int)E, c.rms_eps, st, L)) != cudaSuccess ||
      (ce = session_matmul(e, s->output, n_groups, s->last_x, s->logits)) != cudaSuccess)
    return fail_cuda(e, ce, "kernel launch");
  std::vector<int> win(n_groups);
  if (next_ids) {
    if ((ce = launch_argmax_rows(s->logits, (int)n_groups, (int)V, s->ids, nullptr, st, L)) != cudaSuccess ||
        (ce = cudaMemcpyAsync(win.data(), s->ids, n_groups * sizeof(int), cudaMemcpyDeviceToHost, st)) != cudaSuccess)
      return fail_cuda(e, ce, "argmax");
  }
  std::vector<float> lg(last_logits ? n_groups * V : 0);
  if (last_logits && (ce = cudaMemcpyAsync(lg.data(), s->logits, n_groups * V * sizeof(float), cudaMemcpyDeviceToHost, st)) != cudaSuccess)
    return fail_cuda(e, ce, "logits download");
  if ((ce = cudaStreamSynchronize(st)) != cudaSuccess) return fail_cuda(e, ce, "batch");
  if (take_device_error(e) != 0) return fail(e, LLR_ERR_CUDA, "a device-side wait ran out of iterations");
  for (size_t oi = 0; oi < n_groups; ++oi) {  // results back in the caller's group order
    const size_t g = order[oi];
    if (next_ids) next_ids[g] = win[oi];
    if (last_logits) std::memcpy(last_logits + g * V, lg.data() + oi * V, V * sizeof(float));
    s->position[seq_ids[g]] += counts[g];
    s->have_logits[seq_ids[g]] = 0;  // the single-sequence decode loop keeps its own logits
  }
  // sequence 0's device-side position follows what was appended to it here
  if (seen[0]) {
    const int p0 = (int)s->position[0];
    if ((ce = cudaMemcpyAsync(s->pos_dev, &p0, sizeof(int), cudaMemcpyHostToDevice, st)) != cudaSuccess ||
        (ce = cudaStreamSynchronize(st)) != cudaSuccess)
      return fail_cuda(e, ce, "position upload");
  }
  return LLR_OK;
}

int llr_dequant_rows(llr_exec* e, const llr_matrix* m, size_t row0, size_t n_rows, float* out,
                     size_t out_len) {
  if (!e) return LLR_ERR_INVALID;
  int rc = check_matrix(e, m);
  if (rc) return rc;
  size_t n = 0;
  if (row0 > (size_t)m->rows || n_rows > (size_t)m->rows - row0 ||
      !mul_ok(n_rows, (size_t)m->cols, &n) || out_len != n || (!out && n))
    return fail(e, LLR_ERR_INVALID, "dequant row range or output length does not match the matrix");
  if (n == 0) return LLR_OK;
  DeviceGuard guard(e->device);
  cudaError_t ce;
  if ((ce = grow_device(&e->dev_y, &e->dev_y_cap, n)) != cudaSuccess) return fail_cuda(e, ce, "result scratch");
  if ((ce = launch_dequant(view_of(m), (int64_t)row0, (int64_t)n_rows, e->dev_y, e->stream,
                           &e->ctr.launches)) != cudaSuccess)
    return fail_cuda(e, ce, "kernel launch");
  if ((ce = grow_pinned(&e->pin_y, &e->pin_y_cap, n)) != cudaSuccess) return fail_cuda(e, ce, "pinned result staging");
  if ((ce = cudaMemcpyAsync(e->pin_y, e->dev_y, n * sizeof(float), cudaMemcpyDeviceToHost, e->stream)) != cudaSuccess ||
      (ce = cudaStreamSynchronize(e->stream)) != cudaSuccess)
    return fail_cuda(e, ce, "result download");
  std::memcpy(out, e->pin_y, n * sizeof(float));
  e->ctr.d2h_bytes += n * sizeof(float);
  return LLR_OK;
}

int llr_matrix_synth(llr_exec* e, uint8_t dtype, size_t rows, size_t cols, uint64_t seed,
                     llr_matrix** out) {
  if (!e) return LLR_ERR_INVALID;
  if (!out) return fail(e, LLR_ERR_INVALID, "null output pointer");
  *out = nullptr;
  if (rows == 0 || cols == 0) return fail(e, LLR_ERR_INVALID, "GEMV dimensions must be positive");
  size_t rb = 0, expect = 0;
  std::string msg;
  int rc = row_bytes_checked(dtype, cols, &rb, &msg);
  if (rc) return fail(e, rc, msg);
  if (!mul_ok(rb, rows, &expect)) return fail(e, LLR_ERR_OVERFLOW, "GEMV shape overflow");
  DeviceGuard guard(e->device);
  llr_matrix* m = nullptr;
  if ((rc = alloc_matrix(e, dtype, rows, cols, rb, expect, &m)) != LLR_OK) return rc;
  cudaError_t ce = launch_synth(dtype, (int64_t)rows, (int64_t)cols, seed, m->dev, e->stream,
                                &e->ctr.launches);
  unsigned int bound = 0;
  const bool examine = gemm_tc_supported(view_of(m), 64) && e->bound_dev != nullptr;
  if (ce == cudaSuccess) ce = begin_range_check(e, m, &bound);
  if (ce == cudaSuccess) ce = cudaStreamSynchronize(e->stream);
  if (ce != cudaSuccess) { release_matrix(e, m); return fail_cuda(e, ce, "synthetic fill"); }
  finish_range_check(m, bound, examine);
  *out = m;
  return LLR_OK;
}

int llr_matrix_download(llr_exec* e, const llr_matrix* m, void* out, size_t out_len) {
  if (!e) return LLR_ERR_INVALID;
  int rc = check_matrix(e, m);
  if (rc) return rc;
  if (!out || out_len != m->bytes) return fail(e, LLR_ERR_INVALID, "output length does not match the matrix");
  DeviceGuard guard(e->device);
  cudaError_t ce = cudaMemcpyAsync(out, m->dev, m->bytes, cudaMemcpyDeviceToHost, e->stream);
  if (ce == cudaSuccess) ce = cudaStreamSynchronize(e->stream);
  if (ce != cudaSuccess) return fail_cuda(e, ce, "weight download");
  return LLR_OK;
}

}  // extern "C"
