// Decode GEMV (1..8 activation rows) for the element formats F32, F16 and BF16: gemv_f32 / gemv_f16 of
// langtax/src/quant.rs (:6191, :6144) and their gemm twins for a handful of rows.
//
// These formats need no unpacking, so the kernel is a plain stream: one warp per weight row, every lane pulls
// 16-byte pieces of the row straight from HBM with streaming loads (several pieces in flight per lane, no shared
// memory in between), multiplies them into f32 accumulators against activations that stay in L1, and the warp
// finishes with shuffles.  Bound: HBM.  Algorithmic bytes per weight: 4 (F32), 2 (F16, BF16).
// Rows must start 16-byte aligned and hold a multiple of eight columns; other shapes take the shape-agnostic kernel.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "llr_formats.cuh"
#include "llr_kernels.cuh"

namespace llr {
namespace {

constexpr int ROW_WARPS = 8;
// 16-byte pieces in flight per lane: 8 for the 2-byte formats, 4 pairs for F32 (128 bytes per lane either way)
template <int DT> struct Unroll { static constexpr int N = DT == DT_F32 ? 4 : 8; };

__device__ __forceinline__ uint4 ld_stream16(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}

// The raw 16-byte pieces that hold eight consecutive weights starting at element index c of the row: kept as they
// come (32 bytes for F32, 16 for the 2-byte formats) and widened only when they are used, so that the pieces in
// flight cost a quarter of the registers their f32 values would and four CTAs fit an SM.
template <int DT> struct Raw8 { uint4 a, b; };
template <int DT> __device__ __forceinline__ void fetch8(const uint8_t* row, int64_t c, Raw8<DT>& r) {
  if constexpr (DT == DT_F32) {
    r.a = ld_stream16(row + 4 * c);
    r.b = ld_stream16(row + 4 * c + 16);
  } else {
    r.a = ld_stream16(row + 2 * c);
  }
}
template <int DT> __device__ __forceinline__ void widen8(const Raw8<DT>& r, float (&w)[8]) {
  if constexpr (DT == DT_F32) {
    w[0] = __uint_as_float(r.a.x); w[1] = __uint_as_float(r.a.y); w[2] = __uint_as_float(r.a.z); w[3] = __uint_as_float(r.a.w);
    w[4] = __uint_as_float(r.b.x); w[5] = __uint_as_float(r.b.y); w[6] = __uint_as_float(r.b.z); w[7] = __uint_as_float(r.b.w);
  } else {
    const uint32_t u[4] = {r.a.x, r.a.y, r.a.z, r.a.w};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      if constexpr (DT == DT_F16) {
        // exact for every finite value, infinities included; NaN payloads are a matter of the dequantizer, not of a dot product
        const float2 f = __half22float2(*(const __half2*)&u[k]);
        w[2 * k] = f.x; w[2 * k + 1] = f.y;
      } else {
        w[2 * k] = __uint_as_float(u[k] << 16);
        w[2 * k + 1] = __uint_as_float(u[k] & 0xffff0000u);
      }
    }
  }
}

template <int DT, int MT>
__global__ void __launch_bounds__(ROW_WARPS * 32, (DT == DT_F32 || MT > 2) ? 2 : 4)
gemv_rows_kernel(const uint8_t* __restrict__ W, int64_t row_bytes, int64_t rows, int64_t cols,
                 const float* __restrict__ X, float* __restrict__ Y, int tokens) {
  const int lane = threadIdx.x & 31;
  const int64_t warp = (int64_t)blockIdx.x * ROW_WARPS + (threadIdx.x >> 5);
  const int64_t n_warps = (int64_t)gridDim.x * ROW_WARPS;
  for (int64_t row = warp; row < rows; row += n_warps) {
    const uint8_t* wr = W + row * row_bytes;
    float acc[MT];
#pragma unroll
    for (int t = 0; t < MT; ++t) acc[t] = 0.f;
    constexpr int UNROLL = Unroll<DT>::N;
    for (int64_t c0 = 8 * lane; c0 < cols; c0 += 256 * UNROLL) {
      Raw8<DT> raw[UNROLL];
#pragma unroll
      for (int i = 0; i < UNROLL; ++i)
        if (c0 + 256 * i < cols) fetch8<DT>(wr, c0 + 256 * i, raw[i]);
#pragma unroll
      for (int i = 0; i < UNROLL; ++i) {
        const int64_t c = c0 + 256 * i;
        if (c < cols) {
          float w[8];
          widen8<DT>(raw[i], w);
#pragma unroll
          for (int t = 0; t < MT; ++t)
            if (t < tokens) {
              const float4* xp = (const float4*)(X + (int64_t)t * cols + c);
              const float4 a = __ldg(xp), b = __ldg(xp + 1);
              float s = acc[t];
              s = fmaf(w[0], a.x, s); s = fmaf(w[1], a.y, s); s = fmaf(w[2], a.z, s); s = fmaf(w[3], a.w, s);
              s = fmaf(w[4], b.x, s); s = fmaf(w[5], b.y, s); s = fmaf(w[6], b.z, s); s = fmaf(w[7], b.w, s);
              acc[t] = s;
            }
        }
      }
    }
#pragma unroll
    for (int t = 0; t < MT; ++t) {
      float v = acc[t];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(~0u, v, o);
      if (lane == 0 && t < tokens) Y[(int64_t)t * rows + row] = v;
    }
  }
}

template <int DT, int MT>
cudaError_t launch_rows(const MatView& m, const float* x, float* y, int tokens, cudaStream_t stream, int sm_count) {
  int64_t grid = (m.rows + ROW_WARPS - 1) / ROW_WARPS;
  const int64_t cap = (int64_t)sm_count * 8;  // two waves of the four CTAs of 256 threads an SM holds
  if (grid > cap) grid = cap;
  gemv_rows_kernel<DT, MT><<<(unsigned)grid, ROW_WARPS * 32, 0, stream>>>(m.w, m.row_bytes, m.rows, m.cols, x, y, tokens);
  return cudaGetLastError();
}

template <int DT>
cudaError_t launch_rows_mt(const MatView& m, const float* x, float* y, int tokens, cudaStream_t stream, int sm_count) {
  if (tokens == 1) return launch_rows<DT, 1>(m, x, y, tokens, stream, sm_count);
  if (tokens == 2) return launch_rows<DT, 2>(m, x, y, tokens, stream, sm_count);
  if (tokens <= 4) return launch_rows<DT, 4>(m, x, y, tokens, stream, sm_count);
  return launch_rows<DT, 8>(m, x, y, tokens, stream, sm_count);
}

}  // namespace

bool gemv_rows_supported(const MatView& m) {
  if (m.dtype != DT_F32 && m.dtype != DT_F16 && m.dtype != DT_BF16) return false;
  return m.rows > 0 && m.cols > 0 && m.cols % 8 == 0 && m.row_bytes % 16 == 0 && ((uintptr_t)m.w & 15) == 0;
}

cudaError_t launch_gemv_rows(const MatView& m, const float* x, float* y, int64_t tokens, cudaStream_t stream, int sm_count,
                             uint64_t* launches) {
  for (int64_t t0 = 0; t0 < tokens; t0 += 8) {
    const int nt = (int)(tokens - t0 < 8 ? tokens - t0 : 8);
    const float* xp = x + t0 * m.cols;
    float* yp = y + t0 * m.rows;
    cudaError_t e;
    if (m.dtype == DT_F32) e = launch_rows_mt<DT_F32>(m, xp, yp, nt, stream, sm_count);
    else if (m.dtype == DT_F16) e = launch_rows_mt<DT_F16>(m, xp, yp, nt, stream, sm_count);
    else e = launch_rows_mt<DT_BF16>(m, xp, yp, nt, stream, sm_count);
    if (e != cudaSuccess) return e;
    if (launches) ++*launches;
  }
  return cudaSuccess;
}

}  // namespace llr
