// CPU oracle, scalar part.  TEST INFRASTRUCTURE ONLY (see oracle.h).
//
// Restates, in the reference's exact operation order, the scalar side of
// langtax/src/quant.rs and langtax/src/fp16.rs for the nine dtypes of the
// matrix-executor path.  Must be compiled with -ffp-contract=off and without
// -ffast-math: the reference is Rust, which never contracts a*b+c into an FMA,
// and bit-exactness of the dequantized weights depends on the two roundings.
#include "oracle.h"

#include <cmath>
#include <cstring>
#include <vector>

namespace {

inline uint16_t ld16(const uint8_t* p) { return (uint16_t)(p[0] | (p[1] << 8)); }
inline uint32_t ld32(const uint8_t* p) {
  return (uint32_t)p[0] | ((uint32_t)p[1] << 8) | ((uint32_t)p[2] << 16) | ((uint32_t)p[3] << 24);
}
inline float bits_f32(uint32_t b) { float f; std::memcpy(&f, &b, 4); return f; }
inline uint32_t f32_bits(float f) { uint32_t b; std::memcpy(&b, &f, 4); return b; }
inline void st16(uint8_t* p, uint16_t v) { p[0] = (uint8_t)v; p[1] = (uint8_t)(v >> 8); }

}  // namespace

extern "C" {

// fp16.rs:4-33.  Subnormals are normalised by shifting; Inf/NaN keep payload.
float orc_f16_to_f32(uint16_t h) {
  const uint32_t sign = ((uint32_t)h & 0x8000u) << 16;
  const int exp = (h >> 10) & 0x1f;
  uint32_t man = h & 0x3ffu;
  uint32_t bits;
  if (exp == 0) {
    if (man == 0) {
      bits = sign;
    } else {
      int e = -1;
      while ((man & 0x400u) == 0) { man <<= 1; --e; }
      man &= 0x3ffu;
      bits = sign | ((uint32_t)(e + 114) << 23) | (man << 13);
    }
  } else if (exp == 31) {
    bits = sign | 0x7f800000u | (man << 13);
  } else {
    bits = sign | ((uint32_t)(exp + 112) << 23) | (man << 13);
  }
  return bits_f32(bits);
}

// fp16.rs:36-62.  Round toward zero; binary16 subnormals are produced, f32
// subnormals and anything below 2^-25 flush to signed zero.
uint16_t orc_f32_to_f16(float f) {
  const uint32_t b = f32_bits(f);
  const uint16_t sign = (uint16_t)((b >> 16) & 0x8000u);
  const int biased = (int)((b >> 23) & 0xffu);
  const int exp = biased - 127 + 15;
  const uint32_t man = (b >> 13) & 0x3ffu;
  if (exp >= 31) return (uint16_t)(sign | 0x7c00u);
  if (exp > 0) return (uint16_t)(sign | (exp << 10) | man);
  if (biased == 0) return sign;
  const int shift = 1 - exp;
  if (shift > 11) return sign;
  const uint32_t full = 0x400u | man;
  return (uint16_t)(sign | ((full >> shift) & 0x3ffu));
}

float orc_bf16_to_f32(uint16_t h) { return bits_f32((uint32_t)h << 16); }  // fp16.rs:137

// fp16.rs:142-151
uint16_t orc_f32_to_bf16(float f) {
  const uint32_t u = f32_bits(f);
  if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 64);
  const uint32_t lsb = (u >> 16) & 1u;
  return (uint16_t)((u + 0x7fffu + lsb) >> 16);
}

int orc_block_elems(int kind) {
  switch (kind) {
    case ORC_F16: case ORC_BF16: case ORC_F32: return 1;
    case ORC_Q5_0: case ORC_Q5_1: case ORC_Q4_0: case ORC_Q4_1: case ORC_Q8_0: return 32;
    case ORC_Q4_K: case ORC_Q5_K: case ORC_Q6_K: return 256;
    default: return 0;
  }
}

// quant.rs:86-163
int orc_block_bytes(int kind) {
  switch (kind) {
    case ORC_F16: case ORC_BF16: return 2;
    case ORC_F32: return 4;
    case ORC_Q5_0: return 22;
    case ORC_Q5_1: return 24;
    case ORC_Q4_0: return 18;
    case ORC_Q4_1: return 20;
    case ORC_Q8_0: return 34;
    case ORC_Q4_K: return 144;
    case ORC_Q5_K: return 176;
    case ORC_Q6_K: return 210;
    default: return 0;
  }
}

// <t>_row_bytes, e.g. quant.rs:4210-4218
int64_t orc_row_bytes(int kind, int64_t n_cols) {
  const int be = orc_block_elems(kind);
  if (be == 0) return -ORC_ERR_DTYPE;
  if (n_cols < 0) return -ORC_ERR_SIZE;
  if (n_cols % be != 0) return -ORC_ERR_UNALIGNED_COLS;
  const int64_t nb = n_cols / be;
  const int64_t bb = orc_block_bytes(kind);
  if (nb != 0 && bb > INT64_MAX / nb) return -ORC_ERR_OVERFLOW;
  return nb * bb;
}

// ---- packers ------------------------------------------------------------

void orc_pack_q8_0_block(float d, const int8_t qs[32], uint8_t out[34]) {  // quant.rs:4342
  st16(out, orc_f32_to_f16(d));
  for (int j = 0; j < 32; ++j) out[2 + j] = (uint8_t)qs[j];
}

void orc_pack_q4_0_from_i4(float d, const int8_t v[32], uint8_t out[18]) {  // quant.rs:4594
  st16(out, orc_f32_to_f16(d));
  for (int j = 0; j < 16; ++j) {
    const uint8_t lo = (uint8_t)(v[j] + 8) & 0x0f;
    const uint8_t hi = (uint8_t)(v[j + 16] + 8) & 0x0f;
    out[2 + j] = (uint8_t)(lo | (hi << 4));
  }
}

static void pack_q5_bits(const uint8_t q5[32], uint8_t* qh_dst, uint8_t* qs_dst) {
  uint32_t qh = 0;
  for (int j = 0; j < 16; ++j) {
    const uint8_t l = q5[j], h = q5[j + 16];
    qs_dst[j] = (uint8_t)((l & 0x0f) | ((h & 0x0f) << 4));
    if (l & 0x10) qh |= 1u << j;
    if (h & 0x10) qh |= 1u << (j + 16);
  }
  qh_dst[0] = (uint8_t)qh; qh_dst[1] = (uint8_t)(qh >> 8);
  qh_dst[2] = (uint8_t)(qh >> 16); qh_dst[3] = (uint8_t)(qh >> 24);
}

void orc_pack_q5_0_block(float d, const uint8_t q5[32], uint8_t out[22]) {  // quant.rs:4639
  st16(out, orc_f32_to_f16(d));
  pack_q5_bits(q5, out + 2, out + 6);
}

void orc_pack_q5_1_block(float d, float m, const uint8_t q5[32], uint8_t out[24]) {  // :4680
  st16(out, orc_f32_to_f16(d));
  st16(out + 2, orc_f32_to_f16(m));
  pack_q5_bits(q5, out + 4, out + 8);
}

// quant.rs:4852-4877 (scale bytes) and :4977-5011
void orc_pack_q4_k_block(float d, float dmin, const uint8_t sc[8], const uint8_t mn[8],
                         const uint8_t q4[256], uint8_t out[144]) {
  std::memset(out, 0, 144);
  st16(out, orc_f32_to_f16(d));
  st16(out + 2, orc_f32_to_f16(dmin));
  uint8_t* s = out + 4;
  for (int j = 0; j < 4; ++j) {
    s[j] = sc[j] & 63;
    s[j + 4] = mn[j] & 63;
  }
  for (int j = 4; j < 8; ++j) {
    const uint8_t ls = sc[j] & 63, lm = mn[j] & 63;
    s[j + 4] = (uint8_t)((ls & 0x0f) | ((lm & 0x0f) << 4));
    s[j - 4] |= (uint8_t)((ls >> 4) << 6);
    s[j] |= (uint8_t)((lm >> 4) << 6);
  }
  for (int g = 0; g < 4; ++g)
    for (int l = 0; l < 32; ++l)
      out[16 + g * 32 + l] =
          (uint8_t)((q4[g * 64 + l] & 0x0f) | ((q4[g * 64 + 32 + l] & 0x0f) << 4));
}

// quant.rs:4611-4634: lo nibble is element j, hi nibble element j+16
void orc_pack_q4_1_block(float d, float m, const uint8_t q4[32], uint8_t out[20]) {
  st16(out, orc_f32_to_f16(d));
  st16(out + 2, orc_f32_to_f16(m));
  for (int j = 0; j < 16; ++j) out[4 + j] = (uint8_t)((q4[j] & 0x0f) | ((q4[j + 16] & 0x0f) << 4));
}

// quant.rs:5019-5072: the Q4_K header, then qh (bit 2g / 2g+1 of byte l: fifth bit of elements 64g+l / 64g+32+l),
// then the nibbles
void orc_pack_q5_k_block(float d, float dmin, const uint8_t sc[8], const uint8_t mn[8],
                         const uint8_t q5[256], uint8_t out[176]) {
  uint8_t head[144];
  uint8_t zero[256] = {0};
  orc_pack_q4_k_block(d, dmin, sc, mn, zero, head);
  std::memset(out, 0, 176);
  std::memcpy(out, head, 16);
  for (int g = 0; g < 4; ++g)
    for (int l = 0; l < 32; ++l) {
      const uint8_t l5 = q5[g * 64 + l] & 31, h5 = q5[g * 64 + 32 + l] & 31;
      out[48 + g * 32 + l] = (uint8_t)((l5 & 0x0f) | ((h5 & 0x0f) << 4));
      if (l5 > 15) out[16 + l] |= (uint8_t)(1u << (2 * g));
      if (h5 > 15) out[16 + l] |= (uint8_t)(2u << (2 * g));
    }
}

// quant.rs:5712-5748
void orc_pack_q6_k_block(float d, const int8_t sc[16], const int8_t q[256], uint8_t out[210]) {
  std::memset(out, 0, 210);
  for (int g = 0; g < 2; ++g) {
    for (int l = 0; l < 32; ++l) {
      const int j = g * 128;
      const uint8_t q1 = (uint8_t)(q[j + l] + 32) & 63;
      const uint8_t q2 = (uint8_t)(q[j + l + 32] + 32) & 63;
      const uint8_t q3 = (uint8_t)(q[j + l + 64] + 32) & 63;
      const uint8_t q4 = (uint8_t)(q[j + l + 96] + 32) & 63;
      out[g * 64 + l] = (uint8_t)((q1 & 0x0f) | ((q3 & 0x0f) << 4));
      out[g * 64 + l + 32] = (uint8_t)((q2 & 0x0f) | ((q4 & 0x0f) << 4));
      out[128 + g * 32 + l] =
          (uint8_t)((q1 >> 4) | ((q2 >> 4) << 2) | ((q3 >> 4) << 4) | ((q4 >> 4) << 6));
    }
  }
  for (int i = 0; i < 16; ++i) out[192 + i] = (uint8_t)sc[i];
  st16(out + 208, orc_f32_to_f16(d));
}

void orc_pack_f16(const float* v, int64_t n, uint8_t* out) {
  for (int64_t i = 0; i < n; ++i) st16(out + 2 * i, orc_f32_to_f16(v[i]));
}
void orc_pack_bf16(const float* v, int64_t n, uint8_t* out) {
  for (int64_t i = 0; i < n; ++i) st16(out + 2 * i, orc_f32_to_bf16(v[i]));
}

}  // extern "C"

namespace {

// quant.rs:8901-8912 (ggml get_scale_min_k4)
inline void scale_min_k4(const uint8_t* s, int j, uint8_t* sc, uint8_t* mn) {
  if (j < 4) {
    *sc = s[j] & 63;
    *mn = s[j + 4] & 63;
  } else {
    const uint8_t hi = s[j + 4];
    *sc = (uint8_t)((hi & 0x0f) | ((s[j - 4] >> 6) << 4));
    *mn = (uint8_t)((hi >> 4) | ((s[j] >> 6) << 4));
  }
}

inline int q6_from_bits(uint8_t b) { return (int)(b & 63) - 32; }  // quant.rs:5751

// Q5 code of element j (low half) and j+16 (high half), quant.rs:7752-7757
inline void q5_codes(uint32_t qh, uint8_t p, int j, uint8_t* c0, uint8_t* c1) {
  const uint8_t xh0 = (uint8_t)(((qh >> j) << 4) & 0x10);
  const uint8_t xh1 = (uint8_t)((qh >> (j + 12)) & 0x10);
  *c0 = (uint8_t)((p & 0x0f) | xh0);
  *c1 = (uint8_t)((p >> 4) | xh1);
}

// One dequantized block -> out[block elems].  The arithmetic (which product is
// rounded first, mul-then-sub, mul-then-add) is the reference's.
void dequant_block(int kind, const uint8_t* wb, float* out) {
  switch (kind) {
    case ORC_F16: out[0] = orc_f16_to_f32(ld16(wb)); break;    // quant.rs:7511
    case ORC_BF16: out[0] = orc_bf16_to_f32(ld16(wb)); break;  // :7522
    case ORC_F32: out[0] = bits_f32(ld32(wb)); break;          // :7533
    case ORC_Q8_0: {                                           // :7884
      const float d = orc_f16_to_f32(ld16(wb));
      for (int j = 0; j < 32; ++j) out[j] = (float)(int8_t)wb[2 + j] * d;
      break;
    }
    case ORC_Q4_0: {  // :7918
      const float d = orc_f16_to_f32(ld16(wb));
      for (int j = 0; j < 16; ++j) {
        const uint8_t p = wb[2 + j];
        out[j] = (float)((int)(p & 0x0f) - 8) * d;
        out[j + 16] = (float)((int)(p >> 4) - 8) * d;
      }
      break;
    }
    case ORC_Q5_0: {  // :7734
      const float d = orc_f16_to_f32(ld16(wb));
      const uint32_t qh = ld32(wb + 2);
      for (int j = 0; j < 16; ++j) {
        uint8_t c0, c1;
        q5_codes(qh, wb[6 + j], j, &c0, &c1);
        out[j] = (float)((int)c0 - 16) * d;
        out[j + 16] = (float)((int)c1 - 16) * d;
      }
      break;
    }
    case ORC_Q5_1: {  // :8046  (q*d rounded, then + m rounded)
      const float d = orc_f16_to_f32(ld16(wb));
      const float m = orc_f16_to_f32(ld16(wb + 2));
      const uint32_t qh = ld32(wb + 4);
      for (int j = 0; j < 16; ++j) {
        uint8_t c0, c1;
        q5_codes(qh, wb[8 + j], j, &c0, &c1);
        const float p0 = (float)c0 * d;
        const float p1 = (float)c1 * d;
        out[j] = p0 + m;
        out[j + 16] = p1 + m;
      }
      break;
    }
    case ORC_Q4_1: {  // :7703  q*d rounded, then + m rounded
      const float d = orc_f16_to_f32(ld16(wb));
      const float m = orc_f16_to_f32(ld16(wb + 2));
      for (int j = 0; j < 16; ++j) {
        const uint8_t p = wb[4 + j];
        const float p0 = (float)(p & 0x0f) * d;
        const float p1 = (float)(p >> 4) * d;
        out[j] = p0 + m;
        out[j + 16] = p1 + m;
      }
      break;
    }
    case ORC_Q5_K: {  // :8133  a=d*sc, b=dmin*m, w = a*q5 - b
      const float d = orc_f16_to_f32(ld16(wb));
      const float dmin = orc_f16_to_f32(ld16(wb + 2));
      const uint8_t* scales = wb + 4;
      const uint8_t* qh = wb + 16;
      const uint8_t* qs = wb + 48;
      for (int g = 0; g < 4; ++g) {
        uint8_t sc0, m0, sc1, m1;
        scale_min_k4(scales, 2 * g, &sc0, &m0);
        scale_min_k4(scales, 2 * g + 1, &sc1, &m1);
        const float a0 = d * (float)sc0, b0 = dmin * (float)m0;
        const float a1 = d * (float)sc1, b1 = dmin * (float)m1;
        const uint8_t u1 = (uint8_t)(1u << (2 * g)), u2 = (uint8_t)(2u << (2 * g));
        for (int l = 0; l < 32; ++l) {
          const uint8_t p = qs[g * 32 + l];
          const float q0 = (float)((p & 0x0f) + ((qh[l] & u1) ? 16 : 0));  // q5_from_nibble, :5756
          const float q1 = (float)((p >> 4) + ((qh[l] & u2) ? 16 : 0));
          const float t0 = a0 * q0;
          const float t1 = a1 * q1;
          out[g * 64 + l] = t0 - b0;
          out[g * 64 + 32 + l] = t1 - b1;
        }
      }
      break;
    }
    case ORC_Q4_K: {  // :8083  a=d*sc, b=dmin*m, w = a*q - b
      const float d = orc_f16_to_f32(ld16(wb));
      const float dmin = orc_f16_to_f32(ld16(wb + 2));
      const uint8_t* scales = wb + 4;
      const uint8_t* qs = wb + 16;
      for (int g = 0; g < 4; ++g) {
        uint8_t sc0, m0, sc1, m1;
        scale_min_k4(scales, 2 * g, &sc0, &m0);
        scale_min_k4(scales, 2 * g + 1, &sc1, &m1);
        const float a0 = d * (float)sc0, b0 = dmin * (float)m0;
        const float a1 = d * (float)sc1, b1 = dmin * (float)m1;
        for (int l = 0; l < 32; ++l) {
          const uint8_t p = qs[g * 32 + l];
          const float t0 = a0 * (float)(p & 0x0f);
          const float t1 = a1 * (float)(p >> 4);
          out[g * 64 + l] = t0 - b0;
          out[g * 64 + 32 + l] = t1 - b1;
        }
      }
      break;
    }
    case ORC_Q6_K: {  // :8783  w = (d*s)*q, left to right
      const float d = orc_f16_to_f32(ld16(wb + 208));
      const uint8_t* ql = wb;
      const uint8_t* qh = wb + 128;
      const uint8_t* scb = wb + 192;
      for (int g = 0; g < 2; ++g) {
        for (int l = 0; l < 32; ++l) {
          const int is = l / 16;
          const uint8_t ql0 = ql[g * 64 + l], ql1 = ql[g * 64 + l + 32], h = qh[g * 32 + l];
          const int q1 = q6_from_bits((uint8_t)((ql0 & 0x0f) | ((h & 3) << 4)));
          const int q2 = q6_from_bits((uint8_t)((ql1 & 0x0f) | (((h >> 2) & 3) << 4)));
          const int q3 = q6_from_bits((uint8_t)((ql0 >> 4) | (((h >> 4) & 3) << 4)));
          const int q4 = q6_from_bits((uint8_t)((ql1 >> 4) | (((h >> 6) & 3) << 4)));
          const float ds0 = d * (float)(int8_t)scb[g * 8 + is];
          const float ds2 = d * (float)(int8_t)scb[g * 8 + is + 2];
          const float ds4 = d * (float)(int8_t)scb[g * 8 + is + 4];
          const float ds6 = d * (float)(int8_t)scb[g * 8 + is + 6];
          out[g * 128 + l] = ds0 * (float)q1;
          out[g * 128 + l + 32] = ds2 * (float)q2;
          out[g * 128 + l + 64] = ds4 * (float)q3;
          out[g * 128 + l + 96] = ds6 * (float)q4;
        }
      }
      break;
    }
    default: break;
  }
}

// vec_dot_<t>_f32_row for one block: `sum` is the row's single running f32
// accumulator, updated in the reference's element order.
void dot_block(int kind, const uint8_t* wb, const float* x, float& sum) {
  switch (kind) {
    case ORC_F16: sum += orc_f16_to_f32(ld16(wb)) * x[0]; break;    // quant.rs:8963
    case ORC_BF16: sum += orc_bf16_to_f32(ld16(wb)) * x[0]; break;  // :8971
    case ORC_F32: sum += bits_f32(ld32(wb)) * x[0]; break;          // :8979
    case ORC_Q8_0: {                                                // :9326  (q*d)*x
      const float d = orc_f16_to_f32(ld16(wb));
      for (int j = 0; j < 32; ++j) {
        const float w = (float)(int8_t)wb[2 + j] * d;
        sum += w * x[j];
      }
      break;
    }
    case ORC_Q4_0: {  // :9301  element j then j+16, per nibble byte
      const float d = orc_f16_to_f32(ld16(wb));
      for (int j = 0; j < 16; ++j) {
        const uint8_t p = wb[2 + j];
        const float w0 = (float)((int)(p & 0x0f) - 8) * d;
        const float w1 = (float)((int)(p >> 4) - 8) * d;
        sum += w0 * x[j];
        sum += w1 * x[j + 16];
      }
      break;
    }
    case ORC_Q5_0: {  // :9150
      const float d = orc_f16_to_f32(ld16(wb));
      const uint32_t qh = ld32(wb + 2);
      for (int j = 0; j < 16; ++j) {
        uint8_t c0, c1;
        q5_codes(qh, wb[6 + j], j, &c0, &c1);
        const float w0 = (float)((int)c0 - 16) * d;
        const float w1 = (float)((int)c1 - 16) * d;
        sum += w0 * x[j];
        sum += w1 * x[j + 16];
      }
      break;
    }
    case ORC_Q5_1: {  // :9178
      const float d = orc_f16_to_f32(ld16(wb));
      const float m = orc_f16_to_f32(ld16(wb + 2));
      const uint32_t qh = ld32(wb + 4);
      for (int j = 0; j < 16; ++j) {
        uint8_t c0, c1;
        q5_codes(qh, wb[8 + j], j, &c0, &c1);
        const float p0 = (float)c0 * d;
        const float p1 = (float)c1 * d;
        const float w0 = p0 + m;
        const float w1 = p1 + m;
        sum += w0 * x[j];
        sum += w1 * x[j + 16];
      }
      break;
    }
    case ORC_Q4_1: {  // :9125  element j then j+16, per nibble byte
      const float d = orc_f16_to_f32(ld16(wb));
      const float m = orc_f16_to_f32(ld16(wb + 2));
      for (int j = 0; j < 16; ++j) {
        const uint8_t p = wb[4 + j];
        const float p0 = (float)(p & 0x0f) * d;
        const float w0 = p0 + m;
        sum += w0 * x[j];
        const float p1 = (float)(p >> 4) * d;
        const float w1 = p1 + m;
        sum += w1 * x[j + 16];
      }
      break;
    }
    case ORC_Q5_K: {  // :9469  per l: element l of the low half, then of the high half
      const float d = orc_f16_to_f32(ld16(wb));
      const float dmin = orc_f16_to_f32(ld16(wb + 2));
      const uint8_t* scales = wb + 4;
      const uint8_t* qh = wb + 16;
      const uint8_t* qs = wb + 48;
      for (int g = 0; g < 4; ++g) {
        uint8_t sc0, m0, sc1, m1;
        scale_min_k4(scales, 2 * g, &sc0, &m0);
        scale_min_k4(scales, 2 * g + 1, &sc1, &m1);
        const float a0 = d * (float)sc0, b0 = dmin * (float)m0;
        const float a1 = d * (float)sc1, b1 = dmin * (float)m1;
        const uint8_t u1 = (uint8_t)(1u << (2 * g)), u2 = (uint8_t)(2u << (2 * g));
        const float* xlo = x + g * 64;
        const float* xhi = xlo + 32;
        for (int l = 0; l < 32; ++l) {
          const uint8_t p = qs[g * 32 + l];
          const float q0 = (float)((p & 0x0f) + ((qh[l] & u1) ? 16 : 0));
          const float q1 = (float)((p >> 4) + ((qh[l] & u2) ? 16 : 0));
          const float t0 = a0 * q0;
          const float w0 = t0 - b0;
          sum += w0 * xlo[l];
          const float t1 = a1 * q1;
          const float w1 = t1 - b1;
          sum += w1 * xhi[l];
        }
      }
      break;
    }
    case ORC_Q4_K: {  // :9414  all 32 low nibbles of a group, then all 32 high
      const float d = orc_f16_to_f32(ld16(wb));
      const float dmin = orc_f16_to_f32(ld16(wb + 2));
      const uint8_t* scales = wb + 4;
      const uint8_t* qs = wb + 16;
      for (int g = 0; g < 4; ++g) {
        uint8_t sc0, m0, sc1, m1;
        scale_min_k4(scales, 2 * g, &sc0, &m0);
        scale_min_k4(scales, 2 * g + 1, &sc1, &m1);
        const float a0 = d * (float)sc0, b0 = dmin * (float)m0;
        const float a1 = d * (float)sc1, b1 = dmin * (float)m1;
        const float* xlo = x + g * 64;
        const float* xhi = xlo + 32;
        for (int l = 0; l < 32; ++l) {
          const float t = a0 * (float)(qs[g * 32 + l] & 0x0f);
          const float w = t - b0;
          sum += w * xlo[l];
        }
        for (int l = 0; l < 32; ++l) {
          const float t = a1 * (float)(qs[g * 32 + l] >> 4);
          const float w = t - b1;
          sum += w * xhi[l];
        }
      }
      break;
    }
    case ORC_Q6_K: {  // :10095  per l: l, l+32, l+64, l+96
      const float d = orc_f16_to_f32(ld16(wb + 208));
      const uint8_t* ql = wb;
      const uint8_t* qh = wb + 128;
      const uint8_t* scb = wb + 192;
      for (int g = 0; g < 2; ++g) {
        const float* xg = x + g * 128;
        for (int l = 0; l < 32; ++l) {
          const int is = l / 16;
          const uint8_t ql0 = ql[g * 64 + l], ql1 = ql[g * 64 + l + 32], h = qh[g * 32 + l];
          const int q1 = q6_from_bits((uint8_t)((ql0 & 0x0f) | ((h & 3) << 4)));
          const int q2 = q6_from_bits((uint8_t)((ql1 & 0x0f) | (((h >> 2) & 3) << 4)));
          const int q3 = q6_from_bits((uint8_t)((ql0 >> 4) | (((h >> 4) & 3) << 4)));
          const int q4 = q6_from_bits((uint8_t)((ql1 >> 4) | (((h >> 6) & 3) << 4)));
          // `d * s * q * x` parses left to right: ((d*s)*q)*x
          const float w1 = d * (float)(int8_t)scb[g * 8 + is] * (float)q1;
          const float w2 = d * (float)(int8_t)scb[g * 8 + is + 2] * (float)q2;
          const float w3 = d * (float)(int8_t)scb[g * 8 + is + 4] * (float)q3;
          const float w4 = d * (float)(int8_t)scb[g * 8 + is + 6] * (float)q4;
          sum += w1 * xg[l];
          sum += w2 * xg[l + 32];
          sum += w3 * xg[l + 64];
          sum += w4 * xg[l + 96];
        }
      }
      break;
    }
    default: break;
  }
}

}  // namespace

extern "C" {

int orc_dequant_row(int kind, int64_t n_cols, const uint8_t* row, int64_t row_len, float* y,
                    int64_t y_len) {
  const int64_t rb = orc_row_bytes(kind, n_cols);
  if (rb < 0) return (int)-rb;
  if (row_len != rb || y_len != n_cols) return ORC_ERR_SIZE;
  const int be = orc_block_elems(kind), bb = orc_block_bytes(kind);
  for (int64_t b = 0; b < n_cols / be; ++b) dequant_block(kind, row + b * bb, y + b * be);
  return ORC_OK;
}

int orc_dequant_matrix(int kind, int64_t n_rows, int64_t n_cols, const uint8_t* w, int64_t w_len,
                       float* y) {
  const int64_t rb = orc_row_bytes(kind, n_cols);
  if (rb < 0) return (int)-rb;
  if (w_len != rb * n_rows) return ORC_ERR_SIZE;
  for (int64_t r = 0; r < n_rows; ++r) {
    const int rc = orc_dequant_row(kind, n_cols, w + r * rb, rb, y + r * n_cols, n_cols);
    if (rc) return rc;
  }
  return ORC_OK;
}

// The row kernels ignore a truncated trailing block or a short activation
// slice (simd/tests.rs:510-547): only whole blocks with a full x slice count.
float orc_dot_row_scalar(int kind, const uint8_t* row, int64_t row_len, const float* x,
                         int64_t x_len) {
  const int be = orc_block_elems(kind), bb = orc_block_bytes(kind);
  if (be == 0) return 0.0f;
  float sum = 0.0f;
  const int64_t nb = row_len / bb;
  for (int64_t b = 0; b < nb; ++b) {
    if ((b + 1) * be > x_len) {
      if (be == 1) break;  // element formats zip to the shorter side
      continue;
    }
    dot_block(kind, row + b * bb, x + b * be, sum);
  }
  return sum;
}

// Q8_0 x Q8_0 row dot, quant.rs:8860-8876: int32 block dot, then
// sum = sum + (acc as f32) * (dw * dx).
static float dot_q8_0_q8_0_row(const uint8_t* row, const uint8_t* xq, int64_t nb) {
  float sum = 0.0f;
  for (int64_t b = 0; b < nb; ++b) {
    const uint8_t* wb = row + b * 34;
    const uint8_t* xb = xq + b * 34;
    const float dw = orc_f16_to_f32(ld16(wb));
    const float dx = orc_f16_to_f32(ld16(xb));
    int32_t acc = 0;
    for (int j = 0; j < 32; ++j) acc += (int32_t)(int8_t)wb[2 + j] * (int32_t)(int8_t)xb[2 + j];
    const float scale = dw * dx;
    const float term = (float)acc * scale;
    sum = sum + term;
  }
  return sum;
}

float orc_dot_q8_0_q8_0_row_scalar(const uint8_t* row, const uint8_t* xq, int64_t nb) {
  return dot_q8_0_q8_0_row(row, xq, nb);
}

// main.rs:40-48 / q8_gemv.c:58-67: 64-bit LCG, top 31 bits; centred byte.
void orc_demo_q8_0(int64_t n_cols, int64_t n_rows, uint8_t* w, uint8_t* xq) {
  uint64_t seed = 1;
  auto rnd = [&seed]() -> uint32_t {
    seed = seed * 6364136223846793005ull + 1ull;
    return (uint32_t)(seed >> 33);
  };
  auto centred = [](uint32_t u) -> int8_t { return (int8_t)((int32_t)(u % 255u) - 128); };
  const int64_t nb = n_cols / 32;
  int8_t qs[32];
  for (int64_t r = 0; r < n_rows; ++r) {
    for (int64_t b = 0; b < nb; ++b) {
      for (int j = 0; j < 32; ++j) qs[j] = centred(rnd());
      const uint32_t extra = rnd() % 80u;
      const float amax = 20.0f / 1000.0f + (float)extra / 1000.0f;
      orc_pack_q8_0_block(amax, qs, w + (r * nb + b) * 34);
    }
  }
  for (int64_t b = 0; b < nb; ++b) {
    for (int j = 0; j < 32; ++j) qs[j] = centred(rnd());
    orc_pack_q8_0_block(1.0f / 127.0f, qs, xq + b * 34);
  }
}

uint64_t orc_y_checksum(const float* y, int64_t n) {  // q8_gemv.c:103-112
  uint64_t h = 0xcbf29ce484222325ull;
  for (int64_t i = 0; i < n; ++i) {
    h ^= (uint64_t)f32_bits(y[i]);
    h *= 0x100000001b3ull;
  }
  return h;
}

// ---- host-side model walk helpers (langtax/src/decode.rs) ------------------

// decode.rs:11498-11513.  n is cast through u16 in the reference.
void orc_rmsnorm(float* x, const float* w, int64_t n, float eps) {
  float ss = 0.0f;
  for (int64_t i = 0; i < n; ++i) {
    const float sq = x[i] * x[i];
    ss += sq;
  }
  const float nf = (float)(uint16_t)(n <= 65535 ? n : 1);
  const float mean = ss / nf;
  const float rms = std::sqrt(mean + eps);
  const float inv = rms > 0.0f ? 1.0f / rms : 0.0f;
  for (int64_t i = 0; i < n; ++i) {
    const float t = x[i] * inv;
    x[i] = t * w[i];
  }
}

// decode.rs:11578-11602, applied per head: adjacent-pair rotation, theta
// advanced multiplicatively in f32, f32 cos/sin.
void orc_rope_norm(float* v, int64_t n_heads, int64_t head_dim, int64_t n_rot, int64_t pos,
                   float base) {
  const int64_t n = n_rot < head_dim ? n_rot : head_dim;
  if (n < 2) return;
  const float n_rot_f = (float)(uint16_t)n_rot;
  const float theta_scale = std::pow(base, -2.0f / n_rot_f);
  for (int64_t h = 0; h < n_heads; ++h) {
    float* vec = v + h * head_dim;
    float theta = (float)(uint16_t)(pos <= 65535 ? pos : 65535);
    for (int64_t i = 0; i + 1 < n; i += 2) {
      const float c = std::cos(theta), s = std::sin(theta);
      const float a = vec[i], b = vec[i + 1];
      const float ac = a * c, bs = b * s, as = a * s, bc = b * c;
      vec[i] = ac - bs;
      vec[i + 1] = as + bc;
      theta *= theta_scale;
    }
  }
}

void orc_softmax(float* v, int64_t n) {  // decode.rs:12021-12033
  float m = -INFINITY;
  for (int64_t i = 0; i < n; ++i) m = std::fmax(m, v[i]);
  float s = 0.0f;
  for (int64_t i = 0; i < n; ++i) {
    v[i] = std::exp(v[i] - m);
    s += v[i];
  }
  if (s > 0.0f)
    for (int64_t i = 0; i < n; ++i) v[i] /= s;
}

float orc_silu(float v) { return v / (1.0f + std::exp(-v)); }  // decode.rs:11826

int64_t orc_argmax(const float* v, int64_t n) {  // sample.rs:293
  int64_t best_i = 0;
  float best = -INFINITY;
  for (int64_t i = 0; i < n; ++i)
    if (v[i] > best) { best = v[i]; best_i = i; }
  return best_i;
}

// decode.rs:11363-11381: descending by value, ties to the lower index.
void orc_topk(const float* p, int64_t n, int64_t k, int32_t* ids) {
  std::vector<char> used((size_t)n, 0);
  for (int64_t j = 0; j < k; ++j) {
    int64_t best = -1;
    for (int64_t i = 0; i < n; ++i) {
      if (used[(size_t)i]) continue;
      if (best < 0 || p[i] > p[best]) best = i;
    }
    used[(size_t)best] = 1;
    ids[j] = (int32_t)best;
  }
}

}  // extern "C"
