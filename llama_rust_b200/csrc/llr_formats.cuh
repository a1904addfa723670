// GGUF block formats of the matrix-executor path and their exact decoding.
//
// Layouts follow langtax/src/quant.rs:86-163 (constants) and the packers at
// :4342 (Q8_0), :4581 (Q4_0), :4639 (Q5_0), :4680 (Q5_1), :4977 (Q4_K),
// :5712 (Q6_K), :4611 (Q4_1), :5019 (Q5_K).  `decode8` yields eight consecutive weights of a row with the
// reference's arithmetic, rounding by rounding (dequant_<t>_row,
// quant.rs:7511-8853): products and sums are issued with __fmul_rn / __fsub_rn
// / __fadd_rn so the compiler can never contract them into an FMA.
#pragma once
#include <cuda_fp16.h>
#include <stdint.h>

namespace llr {

enum : int {
  DT_F16 = 0, DT_BF16 = 1, DT_F32 = 2, DT_Q4_1 = 5, DT_Q5_0 = 6, DT_Q5_1 = 7,
  DT_Q4_0 = 12, DT_Q8_0 = 13, DT_Q4_K = 17, DT_Q5_K = 18, DT_Q6_K = 19
};

__host__ __device__ constexpr int block_elems(int dt) {
  return (dt == DT_F16 || dt == DT_BF16 || dt == DT_F32) ? 1
         : (dt == DT_Q5_0 || dt == DT_Q5_1 || dt == DT_Q4_0 || dt == DT_Q4_1 || dt == DT_Q8_0) ? 32
         : (dt == DT_Q4_K || dt == DT_Q5_K || dt == DT_Q6_K) ? 256 : 0;
}

__host__ __device__ constexpr int block_bytes(int dt) {
  return (dt == DT_F16 || dt == DT_BF16) ? 2
         : dt == DT_F32 ? 4
         : dt == DT_Q5_0 ? 22
         : dt == DT_Q5_1 ? 24
         : dt == DT_Q4_0 ? 18
         : dt == DT_Q4_1 ? 20
         : dt == DT_Q8_0 ? 34
         : dt == DT_Q4_K ? 144
         : dt == DT_Q5_K ? 176
         : dt == DT_Q6_K ? 210 : 0;
}

// Units of eight consecutive columns per block (element formats: one unit is
// eight elements of the row).
__host__ __device__ constexpr int units_per_block(int dt) {
  return block_elems(dt) >= 8 ? block_elems(dt) / 8 : 1;
}
// Bytes a unit index advances in the row for the element formats.
__host__ __device__ constexpr int unit_bytes_elem(int dt) { return 8 * block_bytes(dt); }

// binary16 -> binary32, exact for every input (langtax/src/fp16.rs:4-33).  The
// hardware conversion is exact for zero, subnormal, normal and infinite
// inputs; NaN keeps its payload the way the reference's bit shuffle does.
__device__ __forceinline__ float f16_bits_to_f32(uint32_t h) {
  if (((h >> 10) & 31u) == 31u)
    return __uint_as_float(((h & 0x8000u) << 16) | 0x7f800000u | ((h & 0x3ffu) << 13));
  return __half2float(__ushort_as_half((unsigned short)h));
}

__device__ __forceinline__ uint32_t ld16(const uint8_t* p) {
  return (uint32_t)p[0] | ((uint32_t)p[1] << 8);
}
__device__ __forceinline__ uint32_t ld32(const uint8_t* p) {
  return (uint32_t)p[0] | ((uint32_t)p[1] << 8) | ((uint32_t)p[2] << 16) | ((uint32_t)p[3] << 24);
}

// ggml get_scale_min_k4 (quant.rs:8901-8912): 6-bit scale and min of sub-block j.
__device__ __forceinline__ void scale_min_k4(const uint8_t* s, int j, int* sc, int* mn) {
  if (j < 4) {
    *sc = s[j] & 63;
    *mn = s[j + 4] & 63;
  } else {
    const int hi = s[j + 4];
    *sc = (hi & 0x0f) | ((s[j - 4] >> 6) << 4);
    *mn = (hi >> 4) | ((s[j] >> 6) << 4);
  }
}

// Eight consecutive weights.  For block formats `blk` points at the block and
// `u` (0 .. units_per_block-1) selects columns 8u .. 8u+7 of that block.  For
// the element formats `blk` points at the first of the eight elements and
// `valid` (1..8) says how many exist; the rest are returned as zero.
template <int DT>
__device__ __forceinline__ void decode8(const uint8_t* __restrict__ blk, int u, int valid,
                                        float w[8]) {
  if constexpr (DT == DT_F32) {
#pragma unroll
    for (int j = 0; j < 8; ++j) w[j] = j < valid ? __uint_as_float(ld32(blk + 4 * j)) : 0.0f;
  } else if constexpr (DT == DT_F16) {
#pragma unroll
    for (int j = 0; j < 8; ++j) w[j] = j < valid ? f16_bits_to_f32(ld16(blk + 2 * j)) : 0.0f;
  } else if constexpr (DT == DT_BF16) {
#pragma unroll
    for (int j = 0; j < 8; ++j) w[j] = j < valid ? __uint_as_float(ld16(blk + 2 * j) << 16) : 0.0f;
  } else if constexpr (DT == DT_Q8_0) {
    const float d = f16_bits_to_f32(ld16(blk));
#pragma unroll
    for (int j = 0; j < 8; ++j) w[j] = __fmul_rn((float)(int)(int8_t)blk[2 + 8 * u + j], d);
  } else if constexpr (DT == DT_Q4_0) {
    const float d = f16_bits_to_f32(ld16(blk));
    const int hi = u >= 2;
    const uint8_t* q = blk + 2 + 8 * (u & 1);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int nib = hi ? (q[j] >> 4) : (q[j] & 15);
      w[j] = __fmul_rn((float)(nib - 8), d);
    }
  } else if constexpr (DT == DT_Q4_1) {  // dequant_q4_1_row, quant.rs:7703: q*d rounded, then + m
    const float d = f16_bits_to_f32(ld16(blk));
    const float m = f16_bits_to_f32(ld16(blk + 2));
    const int hi = u >= 2;
    const uint8_t* q = blk + 4 + 8 * (u & 1);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int nib = hi ? (q[j] >> 4) : (q[j] & 15);
      w[j] = __fadd_rn(__fmul_rn((float)nib, d), m);
    }
  } else if constexpr (DT == DT_Q5_K) {  // dequant_q5_k_row, quant.rs:8133: a = d*sc, b = dmin*m, a*q - b
    const float d = f16_bits_to_f32(ld16(blk));
    const float dmin = f16_bits_to_f32(ld16(blk + 2));
    const int g = u >> 3, v = u & 7, hi = v >= 4, l0 = 8 * (v & 3);
    int sc, mn;
    scale_min_k4(blk + 4, 2 * g + hi, &sc, &mn);
    const float a = __fmul_rn(d, (float)sc);
    const float b = __fmul_rn(dmin, (float)mn);
    const uint8_t* q = blk + 48 + g * 32 + l0;
    const uint8_t* qh = blk + 16 + l0;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int nib = hi ? (q[j] >> 4) : (q[j] & 15);
      const int code = nib + (((qh[j] >> (2 * g + hi)) & 1) << 4);
      w[j] = __fsub_rn(__fmul_rn(a, (float)code), b);
    }
  } else if constexpr (DT == DT_Q5_0 || DT == DT_Q5_1) {
    constexpr int HDR = DT == DT_Q5_0 ? 2 : 4;
    const float d = f16_bits_to_f32(ld16(blk));
    const float m = DT == DT_Q5_1 ? f16_bits_to_f32(ld16(blk + 2)) : 0.0f;
    const uint32_t qh = ld32(blk + HDR);
    const int hi = u >= 2;
    const int j0 = 8 * (u & 1);
    const uint8_t* q = blk + HDR + 4 + j0;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int nib = hi ? (q[j] >> 4) : (q[j] & 15);
      const int code = nib | (int)(((qh >> (j0 + j + 16 * hi)) & 1u) << 4);
      if constexpr (DT == DT_Q5_0) w[j] = __fmul_rn((float)(code - 16), d);
      else w[j] = __fadd_rn(__fmul_rn((float)code, d), m);
    }
  } else if constexpr (DT == DT_Q4_K) {
    const float d = f16_bits_to_f32(ld16(blk));
    const float dmin = f16_bits_to_f32(ld16(blk + 2));
    const int g = u >> 3, v = u & 7, hi = v >= 4;
    int sc, mn;
    scale_min_k4(blk + 4, 2 * g + hi, &sc, &mn);
    const float a = __fmul_rn(d, (float)sc);
    const float b = __fmul_rn(dmin, (float)mn);
    const uint8_t* q = blk + 16 + g * 32 + 8 * (v & 3);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int nib = hi ? (q[j] >> 4) : (q[j] & 15);
      w[j] = __fsub_rn(__fmul_rn(a, (float)nib), b);
    }
  } else if constexpr (DT == DT_Q6_K) {
    const float d = f16_bits_to_f32(ld16(blk + 208));
    const int g = u >> 4, r = u & 15, qtr = r >> 2, l0 = (r & 3) * 8;
    const uint8_t* ql = blk + g * 64 + l0 + ((qtr & 1) ? 32 : 0);
    const uint8_t* qh = blk + 128 + g * 32 + l0;
    const int s = (int)(int8_t)blk[192 + g * 8 + (l0 >> 4) + 2 * qtr];
    const float ds = __fmul_rn(d, (float)s);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int nib = (qtr >= 2) ? (ql[j] >> 4) : (ql[j] & 15);
      const int q = (nib | (((qh[j] >> (2 * qtr)) & 3) << 4)) - 32;
      w[j] = __fmul_rn(ds, (float)q);
    }
  }
}

}  // namespace llr
