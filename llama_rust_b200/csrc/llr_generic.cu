// Shape-agnostic kernels: the fallback GEMV (any alignment, any column count
// the format allows) and the bit-exact row dequantizer.
//
// The GEMV computes what gemv_<t>_f32 / gemm_<t>_f32 compute
// (langtax/src/quant.rs:6144-6478, 7176-7221): each weight is dequantized with
// the reference's own roundings (decode8) and multiplied into an f32
// accumulator; only the order of the additions differs from the CPU kernels.
#include "llr_formats.cuh"
#include "llr_kernels.cuh"

namespace llr {
namespace {

constexpr int GEN_WARPS = 8;
constexpr int GEN_TOK = 8;  // tokens per pass

template <int DT>
__global__ void __launch_bounds__(GEN_WARPS * 32)
gemv_generic_kernel(const uint8_t* __restrict__ W, int64_t row_bytes, int64_t rows, int64_t cols,
                    const float* __restrict__ X, float* __restrict__ Y, int64_t tokens) {
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * GEN_WARPS + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int64_t tok0 = (int64_t)blockIdx.y * GEN_TOK;
  const int ntok = (int)min((int64_t)GEN_TOK, tokens - tok0);
  const uint8_t* wrow = W + row * row_bytes;
  const float* x0 = X + tok0 * cols;
  constexpr int UPB = units_per_block(DT);
  constexpr int BE = block_elems(DT);
  const int64_t n_units = (cols + 7) / 8;

  float acc[GEN_TOK];
#pragma unroll
  for (int t = 0; t < GEN_TOK; ++t) acc[t] = 0.0f;

  for (int64_t u = lane; u < n_units; u += 32) {
    float w[8];
    int valid = 8;
    if constexpr (BE == 1) {
      valid = (int)min((int64_t)8, cols - 8 * u);
      decode8<DT>(wrow + u * unit_bytes_elem(DT), 0, valid, w);
    } else {
      decode8<DT>(wrow + (u / UPB) * block_bytes(DT), (int)(u % UPB), 8, w);
    }
#pragma unroll
    for (int t = 0; t < GEN_TOK; ++t) {
      if (t < ntok) {
        const float* xp = x0 + (int64_t)t * cols + 8 * u;
#pragma unroll
        for (int j = 0; j < 8; ++j)
          if (j < valid) acc[t] = fmaf(w[j], xp[j], acc[t]);
      }
    }
  }
#pragma unroll
  for (int t = 0; t < GEN_TOK; ++t) {
    float v = acc[t];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    if (lane == 0 && t < ntok) Y[(tok0 + t) * rows + row] = v;
  }
}

template <int DT>
__global__ void __launch_bounds__(256)
dequant_kernel(const uint8_t* __restrict__ W, int64_t row_bytes, int64_t cols, int64_t row0,
               int64_t n_rows, float* __restrict__ out) {
  constexpr int UPB = units_per_block(DT);
  constexpr int BE = block_elems(DT);
  const int64_t n_units = (cols + 7) / 8;
  const int64_t total = n_units * n_rows;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = i / n_units, u = i % n_units;
    const uint8_t* wrow = W + (row0 + r) * row_bytes;
    float w[8];
    int valid = 8;
    if constexpr (BE == 1) {
      valid = (int)min((int64_t)8, cols - 8 * u);
      decode8<DT>(wrow + u * unit_bytes_elem(DT), 0, valid, w);
    } else {
      decode8<DT>(wrow + (u / UPB) * block_bytes(DT), (int)(u % UPB), 8, w);
    }
    float* o = out + r * cols + 8 * u;
#pragma unroll
    for (int j = 0; j < 8; ++j)
      if (j < valid) o[j] = w[j];
  }
}

// Rows picked by an index list in device memory (token embeddings): out[i] = dequantized row ids[i];
// an index outside the matrix yields zeros.
template <int DT>
__global__ void __launch_bounds__(256)
dequant_indexed_kernel(const uint8_t* __restrict__ W, int64_t row_bytes, int64_t rows, int64_t cols,
                       const int* __restrict__ ids, int64_t n, float* __restrict__ out) {
  constexpr int UPB = units_per_block(DT);
  constexpr int BE = block_elems(DT);
  const int64_t n_units = (cols + 7) / 8;
  const int64_t total = n_units * n;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = i / n_units, u = i % n_units;
    const int64_t src = ids[r];
    float w[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    int valid = BE == 1 ? (int)min((int64_t)8, cols - 8 * u) : 8;
    if (src >= 0 && src < rows) {
      const uint8_t* wrow = W + src * row_bytes;
      if constexpr (BE == 1) decode8<DT>(wrow + u * unit_bytes_elem(DT), 0, valid, w);
      else decode8<DT>(wrow + (u / UPB) * block_bytes(DT), (int)(u % UPB), 8, w);
    }
    float* o = out + r * cols + 8 * u;
#pragma unroll
    for (int j = 0; j < 8; ++j)
      if (j < valid) o[j] = w[j];
  }
}

// *flag = 1 when the two byte ranges differ anywhere (both 16-byte aligned; n bytes), else 0
__global__ void bytes_differ_kernel(const uint8_t* __restrict__ a, const uint8_t* __restrict__ b, size_t n, int* __restrict__ flag) {
  const size_t n16 = n / 16;
  bool diff = false;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n16; i += (size_t)gridDim.x * blockDim.x) {
    const uint4 x = ((const uint4*)a)[i], y = ((const uint4*)b)[i];
    diff = diff || x.x != y.x || x.y != y.y || x.z != y.z || x.w != y.w;
  }
  if (blockIdx.x == 0 && threadIdx.x == 0)
    for (size_t i = n16 * 16; i < n; ++i) diff = diff || a[i] != b[i];
  if (diff) *flag = 1;
}

}  // namespace

cudaError_t launch_bytes_differ(const void* a, const void* b, size_t n, int* flag_dev, cudaStream_t stream, uint64_t* launches) {
  cudaError_t e = cudaMemsetAsync(flag_dev, 0, sizeof(int), stream);
  if (e != cudaSuccess) return e;
  size_t blocks = (n / 16 + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  if (blocks == 0) blocks = 1;
  bytes_differ_kernel<<<(unsigned)blocks, 256, 0, stream>>>((const uint8_t*)a, (const uint8_t*)b, n, flag_dev);
  if (launches) ++*launches;
  return cudaGetLastError();
}

#define LLR_DISPATCH_DTYPE(dt, CALL)                         \
  switch (dt) {                                              \
    case DT_F16: { constexpr int DT = DT_F16; CALL; } break;   \
    case DT_BF16: { constexpr int DT = DT_BF16; CALL; } break; \
    case DT_F32: { constexpr int DT = DT_F32; CALL; } break;   \
    case DT_Q4_1: { constexpr int DT = DT_Q4_1; CALL; } break; \
    case DT_Q5_K: { constexpr int DT = DT_Q5_K; CALL; } break; \
    case DT_Q5_0: { constexpr int DT = DT_Q5_0; CALL; } break; \
    case DT_Q5_1: { constexpr int DT = DT_Q5_1; CALL; } break; \
    case DT_Q4_0: { constexpr int DT = DT_Q4_0; CALL; } break; \
    case DT_Q8_0: { constexpr int DT = DT_Q8_0; CALL; } break; \
    case DT_Q4_K: { constexpr int DT = DT_Q4_K; CALL; } break; \
    case DT_Q6_K: { constexpr int DT = DT_Q6_K; CALL; } break; \
    default: return cudaErrorInvalidValue;                   \
  }

cudaError_t launch_gemv_generic(const MatView& m, const float* x, float* y, int64_t tokens,
                                cudaStream_t stream, uint64_t* launches) {
  if (m.rows <= 0 || tokens <= 0) return cudaSuccess;
  const int64_t gx = (m.rows + GEN_WARPS - 1) / GEN_WARPS;
  // grid.y is limited to 65535: cover very wide batches in slabs of tokens
  const int64_t slab = (int64_t)GEN_TOK * 65535;
  for (int64_t t0 = 0; t0 < tokens; t0 += slab) {
    const int64_t nt = tokens - t0 < slab ? tokens - t0 : slab;
    dim3 grid((unsigned)gx, (unsigned)((nt + GEN_TOK - 1) / GEN_TOK));
    LLR_DISPATCH_DTYPE(m.dtype, (gemv_generic_kernel<DT><<<grid, GEN_WARPS * 32, 0, stream>>>(
                                    m.w, m.row_bytes, m.rows, m.cols, x + t0 * m.cols,
                                    y + t0 * m.rows, nt)));
    if (launches) ++*launches;
  }
  return cudaGetLastError();
}

cudaError_t launch_dequant_indexed(const MatView& m, const int* ids_dev, int64_t n, float* out,
                                   cudaStream_t stream, uint64_t* launches) {
  if (n <= 0) return cudaSuccess;
  const int64_t total = ((m.cols + 7) / 8) * n;
  int64_t blocks = (total + 255) / 256;
  if (blocks > 148 * 32) blocks = 148 * 32;
  LLR_DISPATCH_DTYPE(m.dtype, (dequant_indexed_kernel<DT><<<(unsigned)blocks, 256, 0, stream>>>(
                                  m.w, m.row_bytes, m.rows, m.cols, ids_dev, n, out)));
  if (launches) ++*launches;
  return cudaGetLastError();
}

cudaError_t launch_dequant(const MatView& m, int64_t row0, int64_t n_rows, float* out,
                           cudaStream_t stream, uint64_t* launches) {
  if (n_rows <= 0) return cudaSuccess;
  const int64_t total = ((m.cols + 7) / 8) * n_rows;
  int64_t blocks = (total + 255) / 256;
  if (blocks > 148 * 32) blocks = 148 * 32;
  LLR_DISPATCH_DTYPE(m.dtype, (dequant_kernel<DT><<<(unsigned)blocks, 256, 0, stream>>>(
                                  m.w, m.row_bytes, m.cols, row0, n_rows, out)));
  if (launches) ++*launches;
  return cudaGetLastError();
}

}  // namespace llr
