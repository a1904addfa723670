// Decode GEMV (1..8 activation rows) over packed GGUF blocks, staged through
// shared memory.
//
// Computes what gemv_<t>_f32 / gemm_<t>_f32 compute (langtax/src/quant.rs:
// 6144-6478, 7176-7221) without ever expanding the weights: every warp streams
// its rows' packed bytes from HBM into a private shared-memory ring with 16-byte
// asynchronous copies (three stages in flight per warp), decodes scales, mins
// and quants in registers, keeps F32 accumulators and finishes with warp
// shuffles.  Rows are treated as byte streams: a copy starts at the 16-byte
// boundary below the row segment and the decoder indexes from the remainder,
// because only Q4_K blocks (144 B) are 16-byte aligned inside a row; Q5_1 is
// 8-byte, the others 2-byte aligned.
//
// Numerics: the affine terms are factored out of the inner sum (Q4_K:
// a*sum(q*x) - b*sum(x); Q6_K/Q8_0/Q4_0/Q5_0: scale*sum(q*x); Q5_1:
// d*sum(q*x) + m*sum(x)), so one FMA per weight remains.  The result differs
// from the CPU row kernels (langtax/src/simd/x86.rs:208-775) by rounding order
// only; the parity tests hold it to |gpu-cpu| <= 1e-5*(1+|cpu|).
#include "llr_formats.cuh"
#include "llr_kernels.cuh"

namespace llr {
namespace {

constexpr int NW = 8;      // warps per CTA
constexpr int STAGES = 3;  // per-warp ring depth

template <int DT> struct Seg {
  static constexpr int COLS = block_elems(DT) > 1 ? 2048 : (DT == DT_F32 ? 512 : 1024);
  static constexpr int BYTES = COLS / block_elems(DT) * block_bytes(DT);
  static constexpr int SROW = ((BYTES + 15) & ~15) + 32;  // window slack + bank skew
};

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gsrc) {
  const uint32_t d = (uint32_t)__cvta_generic_to_shared(smem_dst);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(d), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory");
}

__device__ __forceinline__ uint32_t lds16(const uint8_t* p) { return *(const uint16_t*)p; }
// eight bytes from a 2-byte aligned address as two little-endian words
__device__ __forceinline__ uint2 lds8_a2(const uint8_t* p) {
  return make_uint2(lds16(p) | (lds16(p + 2) << 16), lds16(p + 4) | (lds16(p + 6) << 16));
}
__device__ __forceinline__ float byte_f32(uint32_t w, int k) { return (float)((w >> (8 * k)) & 255u); }
__device__ __forceinline__ float sbyte_f32(uint32_t w, int k) {
  return (float)(int)(int8_t)((w >> (8 * k)) & 255u);
}

// acc[t] += scale * sum_j q[j]*x[t][j] (+ offs * sum_j x[t][j])
template <int MT, bool WITH_SUM>
__device__ __forceinline__ void fold(const float q[8], const float (&x)[MT][8], float scale,
                                     float offs, float (&acc)[MT]) {
#pragma unroll
  for (int t = 0; t < MT; ++t) {
    float s1 = 0.0f, s0 = 0.0f;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      s1 = fmaf(q[j], x[t][j], s1);
      if (WITH_SUM) s0 += x[t][j];
    }
    acc[t] = fmaf(scale, s1, acc[t]);
    if (WITH_SUM) acc[t] = fmaf(offs, s0, acc[t]);
  }
}

// One unit (eight consecutive columns) of a staged block against MT activation rows.
template <int DT, int MT>
__device__ __forceinline__ void unit_dot(const uint8_t* blk, int u, const float (&x)[MT][8],
                                         float (&acc)[MT]) {
  float q[8];
  if constexpr (DT == DT_F32) {
    const float4 a = *(const float4*)blk, b = *(const float4*)(blk + 16);
    q[0] = a.x; q[1] = a.y; q[2] = a.z; q[3] = a.w; q[4] = b.x; q[5] = b.y; q[6] = b.z; q[7] = b.w;
    fold<MT, false>(q, x, 1.0f, 0.0f, acc);
  } else if constexpr (DT == DT_F16) {
    const uint4 v = *(const uint4*)blk;
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 f = __half22float2(*(const __half2*)&w[k]);
      q[2 * k] = f.x; q[2 * k + 1] = f.y;
    }
    fold<MT, false>(q, x, 1.0f, 0.0f, acc);
  } else if constexpr (DT == DT_BF16) {
    const uint4 v = *(const uint4*)blk;
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      q[2 * k] = __uint_as_float(w[k] << 16);
      q[2 * k + 1] = __uint_as_float(w[k] & 0xffff0000u);
    }
    fold<MT, false>(q, x, 1.0f, 0.0f, acc);
  } else if constexpr (DT == DT_Q8_0) {
    const float d = f16_bits_to_f32(lds16(blk));
    const uint2 v = lds8_a2(blk + 2 + 8 * u);
#pragma unroll
    for (int k = 0; k < 4; ++k) { q[k] = sbyte_f32(v.x, k); q[4 + k] = sbyte_f32(v.y, k); }
    fold<MT, false>(q, x, d, 0.0f, acc);
  } else if constexpr (DT == DT_Q4_0) {
    const float d = f16_bits_to_f32(lds16(blk));
    uint2 v = lds8_a2(blk + 2 + 8 * (u & 1));
    if (u >= 2) { v.x >>= 4; v.y >>= 4; }
    v.x &= 0x0f0f0f0fu; v.y &= 0x0f0f0f0fu;
#pragma unroll
    for (int k = 0; k < 4; ++k) { q[k] = byte_f32(v.x, k) - 8.0f; q[4 + k] = byte_f32(v.y, k) - 8.0f; }
    fold<MT, false>(q, x, d, 0.0f, acc);
  } else if constexpr (DT == DT_Q4_1) {
    const float d = f16_bits_to_f32(lds16(blk));
    const float m = f16_bits_to_f32(lds16(blk + 2));
    uint2 v = lds8_a2(blk + 4 + 8 * (u & 1));
    if (u >= 2) { v.x >>= 4; v.y >>= 4; }
    v.x &= 0x0f0f0f0fu; v.y &= 0x0f0f0f0fu;
#pragma unroll
    for (int k = 0; k < 4; ++k) { q[k] = byte_f32(v.x, k); q[4 + k] = byte_f32(v.y, k); }
    fold<MT, true>(q, x, d, m, acc);
  } else if constexpr (DT == DT_Q5_K) {
    // blocks are 16-byte aligned in the row (176 = 11 x 16) and the window keeps that alignment
    const uint4 h = *(const uint4*)blk;  // d | dmin<<16, then the 12 scale bytes
    const float d = f16_bits_to_f32(h.x & 0xffffu);
    const float dmin = f16_bits_to_f32(h.x >> 16);
    const int g = u >> 3, v8 = u & 7, hi = v8 >= 4, sub = 2 * g + hi, l0 = 8 * (v8 & 3);
    uint32_t sc, mn;
    if (sub < 4) {
      sc = (h.y >> (8 * sub)) & 63u;
      mn = (h.z >> (8 * sub)) & 63u;
    } else {
      const int jj = sub - 4;
      const uint32_t hb = (h.w >> (8 * jj)) & 255u;
      sc = (hb & 15u) | (((h.y >> (8 * jj + 6)) & 3u) << 4);
      mn = (hb >> 4) | (((h.z >> (8 * jj + 6)) & 3u) << 4);
    }
    uint2 v = *(const uint2*)(blk + 48 + g * 32 + l0);
    const uint2 hbits = *(const uint2*)(blk + 16 + l0);
    if (hi) { v.x >>= 4; v.y >>= 4; }
    v.x = (v.x & 0x0f0f0f0fu) | (((hbits.x >> sub) & 0x01010101u) << 4);
    v.y = (v.y & 0x0f0f0f0fu) | (((hbits.y >> sub) & 0x01010101u) << 4);
#pragma unroll
    for (int k = 0; k < 4; ++k) { q[k] = byte_f32(v.x, k); q[4 + k] = byte_f32(v.y, k); }
    fold<MT, true>(q, x, d * (float)sc, -(dmin * (float)mn), acc);
  } else if constexpr (DT == DT_Q5_0 || DT == DT_Q5_1) {
    constexpr int HDR = DT == DT_Q5_0 ? 2 : 4;
    const float d = f16_bits_to_f32(lds16(blk));
    const uint32_t qh = lds16(blk + HDR) | (lds16(blk + HDR + 2) << 16);
    const int hi = u >= 2, j0 = 8 * (u & 1);
    uint2 v = lds8_a2(blk + HDR + 4 + j0);
    if (hi) { v.x >>= 4; v.y >>= 4; }
    v.x &= 0x0f0f0f0fu; v.y &= 0x0f0f0f0fu;
    const uint32_t bits = (qh >> (j0 + 16 * hi)) & 255u;  // fifth bits of the eight codes
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const uint32_t code = (((k < 4 ? v.x : v.y) >> (8 * (k & 3))) & 255u) | (((bits >> k) & 1u) << 4);
      q[k] = DT == DT_Q5_0 ? (float)((int)code - 16) : (float)code;
    }
    if constexpr (DT == DT_Q5_0) {
      fold<MT, false>(q, x, d, 0.0f, acc);
    } else {
      const float m = f16_bits_to_f32(lds16(blk + 2));
      fold<MT, true>(q, x, d, m, acc);
    }
  } else if constexpr (DT == DT_Q4_K) {
    // blocks are 16-byte aligned in the row and the window keeps that alignment
    const uint4 h = *(const uint4*)blk;  // d | dmin<<16, then the 12 scale bytes
    const float d = f16_bits_to_f32(h.x & 0xffffu);
    const float dmin = f16_bits_to_f32(h.x >> 16);
    const int g = u >> 3, v8 = u & 7, hi = v8 >= 4, sub = 2 * g + hi;
    uint32_t sc, mn;
    if (sub < 4) {
      sc = (h.y >> (8 * sub)) & 63u;
      mn = (h.z >> (8 * sub)) & 63u;
    } else {
      const int jj = sub - 4;
      const uint32_t hb = (h.w >> (8 * jj)) & 255u;
      sc = (hb & 15u) | (((h.y >> (8 * jj + 6)) & 3u) << 4);
      mn = (hb >> 4) | (((h.z >> (8 * jj + 6)) & 3u) << 4);
    }
    uint2 v = *(const uint2*)(blk + 16 + g * 32 + 8 * (v8 & 3));
    if (hi) { v.x >>= 4; v.y >>= 4; }
    v.x &= 0x0f0f0f0fu; v.y &= 0x0f0f0f0fu;
#pragma unroll
    for (int k = 0; k < 4; ++k) { q[k] = byte_f32(v.x, k); q[4 + k] = byte_f32(v.y, k); }
    fold<MT, true>(q, x, d * (float)sc, -(dmin * (float)mn), acc);
  } else if constexpr (DT == DT_Q6_K) {
    const float d = f16_bits_to_f32(lds16(blk + 208));
    const int g = u >> 4, r = u & 15, qtr = r >> 2, l0 = (r & 3) * 8;
    uint2 lo = lds8_a2(blk + g * 64 + l0 + ((qtr & 1) ? 32 : 0));
    const uint2 hb = lds8_a2(blk + 128 + g * 32 + l0);
    if (qtr >= 2) { lo.x >>= 4; lo.y >>= 4; }
    const uint32_t c0 = (lo.x & 0x0f0f0f0fu) | (((hb.x >> (2 * qtr)) & 0x03030303u) << 4);
    const uint32_t c1 = (lo.y & 0x0f0f0f0fu) | (((hb.y >> (2 * qtr)) & 0x03030303u) << 4);
    const int s = (int)(int8_t)blk[192 + g * 8 + (l0 >> 4) + 2 * qtr];
#pragma unroll
    for (int k = 0; k < 4; ++k) { q[k] = byte_f32(c0, k) - 32.0f; q[4 + k] = byte_f32(c1, k) - 32.0f; }
    fold<MT, false>(q, x, d * (float)s, 0.0f, acc);
  }
}

template <int DT, int MT, int R>
__global__ void __launch_bounds__(NW * 32)
gemv_staged_kernel(const uint8_t* __restrict__ W, int64_t row_bytes, int64_t rows, int64_t cols,
                   const float* __restrict__ X, float* __restrict__ Y, int tokens) {
  extern __shared__ __align__(16) uint8_t smem[];
  constexpr int COLS = Seg<DT>::COLS, SEGB = Seg<DT>::BYTES, SROW = Seg<DT>::SROW;
  constexpr int UPB = units_per_block(DT), BB = block_bytes(DT), BE = block_elems(DT);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  uint8_t* ring = smem + (size_t)warp * (STAGES * R * SROW);

  const int64_t n_groups = (rows + R - 1) / R;
  const int nseg = (int)((cols + COLS - 1) / COLS);
  const int64_t gstride = (int64_t)gridDim.x * NW;
  const int64_t g_first = (int64_t)blockIdx.x * NW + warp;
  const int64_t my_groups = g_first < n_groups ? (n_groups - g_first + gstride - 1) / gstride : 0;
  const int64_t total = my_groups * nseg;

  auto seg_src = [&](int64_t g, int s, int r) -> const uint8_t* {
    int64_t row = g * R + r;
    if (row >= rows) row = rows - 1;  // tail group: stage a valid row, never written back
    return W + row * row_bytes + (int64_t)s * SEGB;
  };
  auto issue = [&](int64_t item) {
    const int64_t g = g_first + (item / nseg) * gstride;
    const int s = (int)(item % nseg);
    const int stage = (int)(item % STAGES);
    const int64_t left = row_bytes - (int64_t)s * SEGB;
    const int nbytes = (int)(left < SEGB ? left : SEGB);
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const uint8_t* src = seg_src(g, s, r);
      const int off = (int)((uintptr_t)src & 15);
      const uint8_t* a0 = src - off;
      const int nch = (off + nbytes + 15) >> 4;
      uint8_t* dst = ring + (size_t)(stage * R + r) * SROW;
      for (int c = lane; c < nch; c += 32) cp_async16(dst + 16 * c, a0 + 16 * c);
    }
  };

  for (int i = 0; i < STAGES - 1; ++i) {
    if (i < total) issue(i);
    cp_async_commit();
  }

  float acc[R][MT];
#pragma unroll
  for (int r = 0; r < R; ++r)
#pragma unroll
    for (int t = 0; t < MT; ++t) acc[r][t] = 0.0f;

  for (int64_t item = 0; item < total; ++item) {
    if (item + STAGES - 1 < total) issue(item + STAGES - 1);
    cp_async_commit();
    cp_async_wait<STAGES - 1>();
    __syncwarp();

    const int64_t g = g_first + (item / nseg) * gstride;
    const int s = (int)(item % nseg);
    const int stage = (int)(item % STAGES);
    const int64_t col0 = (int64_t)s * COLS;
    const int seg_cols = (int)(cols - col0 < COLS ? cols - col0 : COLS);
    const int n_units = seg_cols >> 3;
    const uint8_t* rowp[R];
#pragma unroll
    for (int r = 0; r < R; ++r)
      rowp[r] = ring + (size_t)(stage * R + r) * SROW + ((uintptr_t)seg_src(g, s, r) & 15);

    for (int u = lane; u < n_units; u += 32) {
      float x[MT][8];
#pragma unroll
      for (int t = 0; t < MT; ++t) {
        if (t < tokens) {
          const float4* xp = (const float4*)(X + (int64_t)t * cols + col0 + 8 * u);
          const float4 a = __ldg(xp), b = __ldg(xp + 1);
          x[t][0] = a.x; x[t][1] = a.y; x[t][2] = a.z; x[t][3] = a.w;
          x[t][4] = b.x; x[t][5] = b.y; x[t][6] = b.z; x[t][7] = b.w;
        } else {
#pragma unroll
          for (int j = 0; j < 8; ++j) x[t][j] = 0.0f;
        }
      }
#pragma unroll
      for (int r = 0; r < R; ++r) {
        const uint8_t* blk = BE > 1 ? rowp[r] + (u / UPB) * BB : rowp[r] + u * unit_bytes_elem(DT);
        unit_dot<DT, MT>(blk, BE > 1 ? u % UPB : 0, x, acc[r]);
      }
    }
    __syncwarp();  // every lane is done with this stage before it is refilled

    if (s == nseg - 1) {
#pragma unroll
      for (int r = 0; r < R; ++r) {
        const int64_t row = g * R + r;
#pragma unroll
        for (int t = 0; t < MT; ++t) {
          float v = acc[r][t];
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
          if (lane == 0 && row < rows && t < tokens) Y[(int64_t)t * rows + row] = v;
          acc[r][t] = 0.0f;
        }
      }
    }
  }
  cp_async_wait<0>();
}

template <int DT, int MT, int R>
cudaError_t launch_one(const MatView& m, const float* x, float* y, int tokens, cudaStream_t stream,
                       int sm_count) {
  auto kern = gemv_staged_kernel<DT, MT, R>;
  constexpr size_t smem = (size_t)NW * STAGES * R * Seg<DT>::SROW;
  static PerDevice cache;  // per instantiation
  std::atomic<int>& slot = cache.here();
  int blocks_per_sm = slot.load(std::memory_order_relaxed);
  if (blocks_per_sm == 0) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    int n = 0;
    e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kern, NW * 32, smem);
    if (e != cudaSuccess) return e;
    blocks_per_sm = n > 0 ? n : 1;
    slot.store(blocks_per_sm, std::memory_order_relaxed);
  }
  const int64_t n_groups = (m.rows + R - 1) / R;
  int64_t grid = (n_groups + NW - 1) / NW;
  const int64_t cap = (int64_t)sm_count * blocks_per_sm;
  if (grid > cap) grid = cap;
  kern<<<(unsigned)grid, NW * 32, smem, stream>>>(m.w, m.row_bytes, m.rows, m.cols, x, y, tokens);
  return cudaGetLastError();
}

template <int DT, int MT>
cudaError_t launch_r(const MatView& m, const float* x, float* y, int tokens, cudaStream_t stream,
                     int sm_count) {
  // two rows per warp share the activation registers; fall back to one row per
  // warp when the matrix has too few rows to give every SM a full CTA
  if (m.rows >= (int64_t)2 * NW * sm_count * 2)
    return launch_one<DT, MT, 2>(m, x, y, tokens, stream, sm_count);
  return launch_one<DT, MT, 1>(m, x, y, tokens, stream, sm_count);
}

template <int DT>
cudaError_t launch_mt(const MatView& m, const float* x, float* y, int tokens, cudaStream_t stream,
                      int sm_count) {
  if (tokens == 1) return launch_r<DT, 1>(m, x, y, tokens, stream, sm_count);
  if (tokens == 2) return launch_r<DT, 2>(m, x, y, tokens, stream, sm_count);
  if (tokens <= 4) return launch_r<DT, 4>(m, x, y, tokens, stream, sm_count);
  return launch_r<DT, 8>(m, x, y, tokens, stream, sm_count);
}

}  // namespace

bool gemv_staged_supported(const MatView& m) {
  if (m.rows <= 0 || m.cols <= 0) return false;
  if (((uintptr_t)m.w & 15) != 0) return false;
  return m.cols % 8 == 0;  // block formats always are; element formats need whole units
}

cudaError_t launch_gemv_staged(const MatView& m, const float* x, float* y, int64_t tokens,
                               cudaStream_t stream, int sm_count, uint64_t* launches) {
  for (int64_t t0 = 0; t0 < tokens; t0 += 8) {
    const int nt = (int)(tokens - t0 < 8 ? tokens - t0 : 8);
    const float* xp = x + t0 * m.cols;
    float* yp = y + t0 * m.rows;
    cudaError_t e;
    switch (m.dtype) {
      case DT_F16: e = launch_mt<DT_F16>(m, xp, yp, nt, stream, sm_count); break;
      case DT_BF16: e = launch_mt<DT_BF16>(m, xp, yp, nt, stream, sm_count); break;
      case DT_F32: e = launch_mt<DT_F32>(m, xp, yp, nt, stream, sm_count); break;
      case DT_Q5_0: e = launch_mt<DT_Q5_0>(m, xp, yp, nt, stream, sm_count); break;
      case DT_Q4_1: e = launch_mt<DT_Q4_1>(m, xp, yp, nt, stream, sm_count); break;
      case DT_Q5_K: e = launch_mt<DT_Q5_K>(m, xp, yp, nt, stream, sm_count); break;
      case DT_Q5_1: e = launch_mt<DT_Q5_1>(m, xp, yp, nt, stream, sm_count); break;
      case DT_Q4_0: e = launch_mt<DT_Q4_0>(m, xp, yp, nt, stream, sm_count); break;
      case DT_Q8_0: e = launch_mt<DT_Q8_0>(m, xp, yp, nt, stream, sm_count); break;
      case DT_Q4_K: e = launch_mt<DT_Q4_K>(m, xp, yp, nt, stream, sm_count); break;
      case DT_Q6_K: e = launch_mt<DT_Q6_K>(m, xp, yp, nt, stream, sm_count); break;
      default: return cudaErrorInvalidValue;
    }
    if (e != cudaSuccess) return e;
    if (launches) ++*launches;
  }
  return cudaSuccess;
}

}  // namespace llr
