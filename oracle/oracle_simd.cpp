// CPU oracle, AVX2 part + entry points.  TEST INFRASTRUCTURE ONLY (see oracle.h).
//
// Restates langtax/src/simd/x86.rs:208-775 (AVX2+FMA+F16C row dots, the
// `--features simd` CPU reference the GPU results are compared to and timed
// beside), the GEMV/GEMM entry points with their validation
// (langtax/src/quant.rs:6144-6478, 6683-6888, 7176-7221) and the row fan-out of
// langtax/src/pool.rs:43-148 (contiguous row chunks, at most 10 workers).
//
// Compile with -mavx2 -mfma -mf16c -ffp-contract=off: the only fused
// operations are the explicit _mm256_fmadd_ps the reference itself issues.
#include "oracle.h"

#include <immintrin.h>

#include <algorithm>
#include <cstring>
#include <thread>
#include <vector>

extern "C" float orc_dot_q8_0_q8_0_row_scalar(const uint8_t* row, const uint8_t* xq, int64_t nb);

namespace {

inline uint16_t ld16(const uint8_t* p) { return (uint16_t)(p[0] | (p[1] << 8)); }
inline uint32_t ld32(const uint8_t* p) { uint32_t v; std::memcpy(&v, p, 4); return v; }

// x86.rs:186-191: (lo128 + hi128), then (a + movehl), then lane0 + lane1.
inline float hsum_ps(__m256 v) {
  const __m128 quad = _mm_add_ps(_mm256_castps256_ps128(v), _mm256_extractf128_ps(v, 1));
  const __m128 pair = _mm_add_ps(quad, _mm_movehl_ps(quad, quad));
  const __m128 one = _mm_add_ss(pair, _mm_shuffle_ps(pair, pair, 0x55));
  return _mm_cvtss_f32(one);
}

inline int hsum_epi32(__m256i v) {  // x86.rs:196-201
  const __m128i quad = _mm_add_epi32(_mm256_castsi256_si128(v), _mm256_extracti128_si256(v, 1));
  const __m128i pair = _mm_add_epi32(quad, _mm_shuffle_epi32(quad, 0x4e));
  const __m128i one = _mm_add_epi32(pair, _mm_shuffle_epi32(pair, 0xb1));
  return _mm_cvtsi128_si32(one);
}

inline __m128i load8(const uint8_t* p) { return _mm_loadl_epi64((const __m128i*)p); }

// binary16 scale decoded in hardware and broadcast, x86.rs:506-512
inline __m256 f16_scale(const uint8_t* p) {
  return _mm256_broadcastss_ps(_mm_cvtph_ps(_mm_cvtsi32_si128((int)ld16(p))));
}

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

// x86.rs:208-231: two 8-lane FMA accumulators alternating, one hsum, scalar tail
float dot_f32(const uint8_t* row, int64_t row_len, const float* x, int64_t x_len) {
  const int64_t n = std::min<int64_t>(row_len / 4, x_len);
  const int64_t chunks = n / 8;
  __m256 acc0 = _mm256_setzero_ps(), acc1 = _mm256_setzero_ps();
  int64_t c = 0;
  while (c < chunks) {
    acc0 = _mm256_fmadd_ps(_mm256_loadu_ps((const float*)(row + 32 * c)),
                           _mm256_loadu_ps(x + 8 * c), acc0);
    ++c;
    if (c >= chunks) break;
    acc1 = _mm256_fmadd_ps(_mm256_loadu_ps((const float*)(row + 32 * c)),
                           _mm256_loadu_ps(x + 8 * c), acc1);
    ++c;
  }
  float sum = hsum_ps(_mm256_add_ps(acc0, acc1));
  for (int64_t i = chunks * 8; i < n; ++i) {
    float w;
    std::memcpy(&w, row + 4 * i, 4);
    sum += w * x[i];
  }
  return sum;
}

float dot_f16(const uint8_t* row, int64_t row_len, const float* x, int64_t x_len) {  // :237-264
  const int64_t n = std::min<int64_t>(row_len / 2, x_len);
  const int64_t chunks = n / 8;
  __m256 acc0 = _mm256_setzero_ps(), acc1 = _mm256_setzero_ps();
  int64_t c = 0;
  while (c < chunks) {
    acc0 = _mm256_fmadd_ps(_mm256_cvtph_ps(_mm_loadu_si128((const __m128i*)(row + 16 * c))),
                           _mm256_loadu_ps(x + 8 * c), acc0);
    ++c;
    if (c >= chunks) break;
    acc1 = _mm256_fmadd_ps(_mm256_cvtph_ps(_mm_loadu_si128((const __m128i*)(row + 16 * c))),
                           _mm256_loadu_ps(x + 8 * c), acc1);
    ++c;
  }
  float sum = hsum_ps(_mm256_add_ps(acc0, acc1));
  for (int64_t i = chunks * 8; i < n; ++i) sum += orc_f16_to_f32(ld16(row + 2 * i)) * x[i];
  return sum;
}

// x86.rs:270-335: accumulator per super-block; weight = a*q - b by separate
// multiply and subtract; sum += hsum(acc) per block.
float dot_q4_k(const uint8_t* row, int64_t row_len, const float* x, int64_t x_len) {
  float sum = 0.0f;
  const __m128i mask = _mm_set1_epi8(0x0f);
  for (int64_t b = 0; b < row_len / 144; ++b) {
    if ((b + 1) * 256 > x_len) continue;
    const uint8_t* wb = row + b * 144;
    const float d = orc_f16_to_f32(ld16(wb));
    const float dmin = orc_f16_to_f32(ld16(wb + 2));
    const float* xr = x + b * 256;
    __m256 acc = _mm256_setzero_ps();
    for (int g = 0; g < 4; ++g) {
      uint8_t sc0, m0, sc1, m1;
      scale_min_k4(wb + 4, 2 * g, &sc0, &m0);
      scale_min_k4(wb + 4, 2 * g + 1, &sc1, &m1);
      const __m256 a0 = _mm256_set1_ps(d * (float)sc0), b0 = _mm256_set1_ps(dmin * (float)m0);
      const __m256 a1 = _mm256_set1_ps(d * (float)sc1), b1 = _mm256_set1_ps(dmin * (float)m1);
      for (int c = 0; c < 4; ++c) {
        const __m128i nib = load8(wb + 16 + g * 32 + c * 8);
        const __m256 lo = _mm256_cvtepi32_ps(_mm256_cvtepu8_epi32(_mm_and_si128(nib, mask)));
        const __m256 hi = _mm256_cvtepi32_ps(
            _mm256_cvtepu8_epi32(_mm_and_si128(_mm_srli_epi16(nib, 4), mask)));
        const __m256 wlo = _mm256_sub_ps(_mm256_mul_ps(a0, lo), b0);
        const __m256 whi = _mm256_sub_ps(_mm256_mul_ps(a1, hi), b1);
        acc = _mm256_fmadd_ps(wlo, _mm256_loadu_ps(xr + g * 64 + c * 8), acc);
        acc = _mm256_fmadd_ps(whi, _mm256_loadu_ps(xr + g * 64 + 32 + c * 8), acc);
      }
    }
    sum += hsum_ps(acc);
  }
  return sum;
}

// `(low | ((qh >> shift) & 3) << 4) - 32` per lane as f32, x86.rs:424-434
inline __m256 q6_lane(__m256i low, __m256i qh, int shift) {
  const __m256i hi = _mm256_srli_epi32(qh, shift);
  const __m256i bits =
      _mm256_or_si256(low, _mm256_slli_epi32(_mm256_and_si256(hi, _mm256_set1_epi32(3)), 4));
  return _mm256_cvtepi32_ps(_mm256_sub_epi32(bits, _mm256_set1_epi32(32)));
}

// x86.rs:341-417: eight elements per step, weight = (d*s)*q, accumulator per block
float dot_q6_k(const uint8_t* row, int64_t row_len, const float* x, int64_t x_len) {
  float sum = 0.0f;
  const __m256i nib = _mm256_set1_epi32(0x0f);
  for (int64_t b = 0; b < row_len / 210; ++b) {
    if ((b + 1) * 256 > x_len) continue;
    const uint8_t* wb = row + b * 210;
    const float d = orc_f16_to_f32(ld16(wb + 208));
    const uint8_t* ql = wb;
    const uint8_t* qh = wb + 128;
    const uint8_t* scb = wb + 192;
    const float* xr = x + b * 256;
    __m256 acc = _mm256_setzero_ps();
    for (int g = 0; g < 2; ++g) {
      for (int step = 0; step < 4; ++step) {
        const int l = step * 8, is = l / 16;
        const __m256 ds0 = _mm256_set1_ps(d * (float)(int8_t)scb[g * 8 + is]);
        const __m256 ds2 = _mm256_set1_ps(d * (float)(int8_t)scb[g * 8 + is + 2]);
        const __m256 ds4 = _mm256_set1_ps(d * (float)(int8_t)scb[g * 8 + is + 4]);
        const __m256 ds6 = _mm256_set1_ps(d * (float)(int8_t)scb[g * 8 + is + 6]);
        const __m256i lo = _mm256_cvtepu8_epi32(load8(ql + g * 64 + l));
        const __m256i hi = _mm256_cvtepu8_epi32(load8(ql + g * 64 + l + 32));
        const __m256i h = _mm256_cvtepu8_epi32(load8(qh + g * 32 + l));
        const __m256 q1 = q6_lane(_mm256_and_si256(lo, nib), h, 0);
        const __m256 q2 = q6_lane(_mm256_and_si256(hi, nib), h, 2);
        const __m256 q3 = q6_lane(_mm256_srli_epi32(lo, 4), h, 4);
        const __m256 q4 = q6_lane(_mm256_srli_epi32(hi, 4), h, 6);
        const float* xg = xr + g * 128 + l;
        acc = _mm256_fmadd_ps(_mm256_mul_ps(ds0, q1), _mm256_loadu_ps(xg), acc);
        acc = _mm256_fmadd_ps(_mm256_mul_ps(ds2, q2), _mm256_loadu_ps(xg + 32), acc);
        acc = _mm256_fmadd_ps(_mm256_mul_ps(ds4, q3), _mm256_loadu_ps(xg + 64), acc);
        acc = _mm256_fmadd_ps(_mm256_mul_ps(ds6, q4), _mm256_loadu_ps(xg + 96), acc);
      }
    }
    sum += hsum_ps(acc);
  }
  return sum;
}

// low / high nibbles of 8 packed bytes as i32 lanes, x86.rs:568-575
inline void nibbles8(const uint8_t* p, __m256i* low, __m256i* high) {
  const __m256i bytes = _mm256_cvtepu8_epi32(load8(p));
  *low = _mm256_and_si256(bytes, _mm256_set1_epi32(0x0f));
  *high = _mm256_srli_epi32(bytes, 4);
}

inline __m256i lane_ids() { return _mm256_setr_epi32(0, 1, 2, 3, 4, 5, 6, 7); }

// Q5_0 codes already biased: nibble when the fifth bit is set, nibble-16 when
// clear (x86.rs:537-544)
inline __m256i q5_0_codes(__m256i nib, __m256i qh, int base) {
  const __m256i bit =
      _mm256_sllv_epi32(_mm256_set1_epi32(1), _mm256_add_epi32(_mm256_set1_epi32(base), lane_ids()));
  const __m256i clear = _mm256_cmpeq_epi32(_mm256_and_si256(qh, bit), _mm256_setzero_si256());
  return _mm256_add_epi32(nib, _mm256_and_si256(clear, _mm256_set1_epi32(-16)));
}

// Q5_1 codes: nibble | fifth << 4, unbiased (x86.rs:553-559)
inline __m256i q5_1_codes(__m256i nib, __m256i qh, int base) {
  const __m256i sh = _mm256_srlv_epi32(qh, _mm256_add_epi32(_mm256_set1_epi32(base), lane_ids()));
  return _mm256_or_si256(nib, _mm256_slli_epi32(_mm256_and_si256(sh, _mm256_set1_epi32(1)), 4));
}

// One accumulator for the whole row, reduced once at the end (x86.rs:588-625)
float dot_q4_0(const uint8_t* row, int64_t row_len, const float* x, int64_t x_len) {
  __m256 acc = _mm256_setzero_ps();
  for (int64_t b = 0; b < row_len / 18; ++b) {
    if ((b + 1) * 32 > x_len) continue;
    const uint8_t* wb = row + b * 18;
    const float* xr = x + b * 32;
    const __m256 dv = f16_scale(wb);
    for (int c = 0; c < 2; ++c) {
      __m256i low, high;
      nibbles8(wb + 2 + c * 8, &low, &high);
      const __m256 w_lo =
          _mm256_mul_ps(_mm256_cvtepi32_ps(_mm256_sub_epi32(low, _mm256_set1_epi32(8))), dv);
      const __m256 w_hi =
          _mm256_mul_ps(_mm256_cvtepi32_ps(_mm256_sub_epi32(high, _mm256_set1_epi32(8))), dv);
      acc = _mm256_fmadd_ps(w_lo, _mm256_loadu_ps(xr + c * 8), acc);
      acc = _mm256_fmadd_ps(w_hi, _mm256_loadu_ps(xr + c * 8 + 16), acc);
    }
  }
  return hsum_ps(acc);
}

float dot_q5_0(const uint8_t* row, int64_t row_len, const float* x, int64_t x_len) {  // :639-686
  __m256 acc = _mm256_setzero_ps();
  for (int64_t b = 0; b < row_len / 22; ++b) {
    if ((b + 1) * 32 > x_len) continue;
    const uint8_t* wb = row + b * 22;
    const float* xr = x + b * 32;
    const __m256 dv = f16_scale(wb);
    const __m256i qh = _mm256_set1_epi32((int)ld32(wb + 2));
    for (int c = 0; c < 2; ++c) {
      __m256i low, high;
      nibbles8(wb + 6 + c * 8, &low, &high);
      const __m256 w_lo = _mm256_mul_ps(_mm256_cvtepi32_ps(q5_0_codes(low, qh, c * 8)), dv);
      const __m256 w_hi = _mm256_mul_ps(_mm256_cvtepi32_ps(q5_0_codes(high, qh, c * 8 + 16)), dv);
      acc = _mm256_fmadd_ps(w_lo, _mm256_loadu_ps(xr + c * 8), acc);
      acc = _mm256_fmadd_ps(w_hi, _mm256_loadu_ps(xr + c * 8 + 16), acc);
    }
  }
  return hsum_ps(acc);
}

float dot_q5_1(const uint8_t* row, int64_t row_len, const float* x, int64_t x_len) {  // :693-740
  __m256 acc = _mm256_setzero_ps();
  for (int64_t b = 0; b < row_len / 24; ++b) {
    if ((b + 1) * 32 > x_len) continue;
    const uint8_t* wb = row + b * 24;
    const float* xr = x + b * 32;
    const __m256 dv = f16_scale(wb), mv = f16_scale(wb + 2);
    const __m256i qh = _mm256_set1_epi32((int)ld32(wb + 4));
    for (int c = 0; c < 2; ++c) {
      __m256i low, high;
      nibbles8(wb + 8 + c * 8, &low, &high);
      // q*d then +m: two roundings, never an FMA
      const __m256 w_lo =
          _mm256_add_ps(_mm256_mul_ps(_mm256_cvtepi32_ps(q5_1_codes(low, qh, c * 8)), dv), mv);
      const __m256 w_hi = _mm256_add_ps(
          _mm256_mul_ps(_mm256_cvtepi32_ps(q5_1_codes(high, qh, c * 8 + 16)), dv), mv);
      acc = _mm256_fmadd_ps(w_lo, _mm256_loadu_ps(xr + c * 8), acc);
      acc = _mm256_fmadd_ps(w_hi, _mm256_loadu_ps(xr + c * 8 + 16), acc);
    }
  }
  return hsum_ps(acc);
}

float dot_q8_0(const uint8_t* row, int64_t row_len, const float* x, int64_t x_len) {  // :747-775
  __m256 acc = _mm256_setzero_ps();
  for (int64_t b = 0; b < row_len / 34; ++b) {
    if ((b + 1) * 32 > x_len) continue;
    const uint8_t* wb = row + b * 34;
    const float* xr = x + b * 32;
    const __m256 dv = f16_scale(wb);
    for (int c = 0; c < 4; ++c) {
      const __m256 q = _mm256_cvtepi32_ps(_mm256_cvtepi8_epi32(load8(wb + 2 + c * 8)));
      acc = _mm256_fmadd_ps(_mm256_mul_ps(q, dv), _mm256_loadu_ps(xr + c * 8), acc);
    }
  }
  return hsum_ps(acc);
}

// Q8_0 x Q8_0, x86.rs:459-492: exact int32 block dot, scale product from
// hardware binary16 decode, `sum = sum + term` (bit-identical to scalar).
float dot_q8_0_q8_0(const uint8_t* row, const uint8_t* xq, int64_t nb) {
  float sum = 0.0f;
  for (int64_t b = 0; b < nb; ++b) {
    const uint8_t* wb = row + b * 34;
    const uint8_t* xb = xq + b * 34;
    const __m256i wv = _mm256_loadu_si256((const __m256i*)(wb + 2));
    const __m256i xv = _mm256_loadu_si256((const __m256i*)(xb + 2));
    const __m256i prod = _mm256_add_epi32(
        _mm256_madd_epi16(_mm256_cvtepi8_epi16(_mm256_castsi256_si128(wv)),
                          _mm256_cvtepi8_epi16(_mm256_castsi256_si128(xv))),
        _mm256_madd_epi16(_mm256_cvtepi8_epi16(_mm256_extracti128_si256(wv, 1)),
                          _mm256_cvtepi8_epi16(_mm256_extracti128_si256(xv, 1))));
    const __m128 both =
        _mm_cvtph_ps(_mm_cvtsi32_si128((int)((uint32_t)ld16(wb) | ((uint32_t)ld16(xb) << 16))));
    const float scale = _mm_cvtss_f32(_mm_mul_ss(both, _mm_shuffle_ps(both, both, 0x55)));
    const float term = (float)hsum_epi32(prod) * scale;
    sum = sum + term;
  }
  return sum;
}

bool cpu_ok() {
  static const bool ok = __builtin_cpu_supports("avx2") && __builtin_cpu_supports("fma") &&
                         __builtin_cpu_supports("f16c");
  return ok;
}

typedef float (*RowDot)(int kind, const uint8_t*, int64_t, const float*, int64_t);

// pool.rs:70-79: min(available_parallelism, rows, 10)
int worker_count(int64_t n_rows, int threads) {
  if (n_rows <= 1) return 1;
  int hw = threads > 0 ? threads : (int)std::thread::hardware_concurrency();
  if (hw < 1) hw = 1;
  if (threads <= 0 && hw > 10) hw = 10;
  return (int)std::min<int64_t>(hw, n_rows);
}

// pool.rs:83-148: contiguous chunks of ceil(rows/workers) rows, one scoped
// thread per chunk.
template <class F>
void for_each_row_chunk(int64_t n_rows, int threads, F&& body) {
  const int workers = worker_count(n_rows, threads);
  if (workers <= 1) {
    body(0, n_rows);
    return;
  }
  const int64_t chunk = (n_rows + workers - 1) / workers;
  std::vector<std::thread> pool;
  for (int64_t start = chunk; start < n_rows; start += chunk)
    pool.emplace_back([=, &body] { body(start, std::min(n_rows, start + chunk)); });
  body(0, std::min(n_rows, chunk));  // the calling thread takes the first chunk
  for (auto& t : pool) t.join();
}

}  // namespace

extern "C" {

int orc_have_simd(void) { return cpu_ok() ? 1 : 0; }

float orc_dot_row_simd(int kind, const uint8_t* row, int64_t row_len, const float* x,
                       int64_t x_len) {
  if (!cpu_ok()) return orc_dot_row_scalar(kind, row, row_len, x, x_len);
  switch (kind) {
    case ORC_F32: return dot_f32(row, row_len, x, x_len);
    case ORC_F16: return dot_f16(row, row_len, x, x_len);
    case ORC_Q4_0: return dot_q4_0(row, row_len, x, x_len);
    case ORC_Q4_K: return dot_q4_k(row, row_len, x, x_len);
    case ORC_Q5_0: return dot_q5_0(row, row_len, x, x_len);
    case ORC_Q5_1: return dot_q5_1(row, row_len, x, x_len);
    case ORC_Q6_K: return dot_q6_k(row, row_len, x, x_len);
    case ORC_Q8_0: return dot_q8_0(row, row_len, x, x_len);
    default: return orc_dot_row_scalar(kind, row, row_len, x, x_len);  // BF16 has no SIMD kernel
  }
}

// Validation order of gemv_<t>_f32 (e.g. quant.rs:7199-7219): row bytes
// (column alignment), x length, W length, then empty y is a no-op.
int orc_gemv(int kind, int64_t n_cols, const uint8_t* w, int64_t w_len, const float* x,
             int64_t x_len, float* y, int64_t y_len, int simd, int threads) {
  const int64_t rb = orc_row_bytes(kind, n_cols);
  if (rb < 0) return (int)-rb;
  if (x_len != n_cols) return ORC_ERR_SIZE;
  if (rb != 0 && y_len > INT64_MAX / rb) return ORC_ERR_OVERFLOW;
  if (w_len != rb * y_len) return ORC_ERR_SIZE;
  if (y_len == 0) return ORC_OK;
  RowDot dot = simd ? orc_dot_row_simd : orc_dot_row_scalar;
  for_each_row_chunk(y_len, threads, [&](int64_t r0, int64_t r1) {
    for (int64_t r = r0; r < r1; ++r) y[r] = dot(kind, w + r * rb, rb, x, n_cols);
  });
  return ORC_OK;
}

// gemm_<t>_f32 -> gemm_f32_x (quant.rs:6760-6888): n_tokens == 1 forwards to
// the GEMV; otherwise each weight row is dotted with every token (the row is
// re-read per token), rows fanned out in contiguous groups, then the
// row-major scratch is transposed to token-major y[t*n_rows + r].
int orc_gemm(int kind, int64_t n_cols, int64_t n_tokens, const uint8_t* w, int64_t w_len,
             const float* x, int64_t x_len, float* y, int64_t y_len, int simd, int threads) {
  if (n_tokens == 1) return orc_gemv(kind, n_cols, w, w_len, x, x_len, y, y_len, simd, threads);
  if (n_tokens <= 0) return ORC_ERR_SIZE;
  if (n_cols != 0 && n_tokens > INT64_MAX / (n_cols > 0 ? n_cols : 1)) return ORC_ERR_OVERFLOW;
  if (x_len != n_tokens * n_cols) return ORC_ERR_SIZE;
  if (y_len % n_tokens != 0) return ORC_ERR_SIZE;
  const int64_t n_rows = y_len / n_tokens;
  const int64_t rb = orc_row_bytes(kind, n_cols);
  if (rb < 0) return (int)-rb;
  if (rb != 0 && n_rows > INT64_MAX / rb) return ORC_ERR_OVERFLOW;
  if (w_len != rb * n_rows) return ORC_ERR_SIZE;
  if (n_rows == 0) return ORC_OK;
  RowDot dot = simd ? orc_dot_row_simd : orc_dot_row_scalar;
  std::vector<float> scratch((size_t)y_len);
  for_each_row_chunk(n_rows, threads, [&](int64_t r0, int64_t r1) {
    for (int64_t r = r0; r < r1; ++r)
      for (int64_t t = 0; t < n_tokens; ++t)
        scratch[(size_t)(r * n_tokens + t)] = dot(kind, w + r * rb, rb, x + t * n_cols, n_cols);
  });
  for (int64_t t = 0; t < n_tokens; ++t)
    for (int64_t r = 0; r < n_rows; ++r) y[t * n_rows + r] = scratch[(size_t)(r * n_tokens + t)];
  return ORC_OK;
}

// native_cuda_parity.rs:124-148: dequantize every row to f32 with the CPU
// kernels, then f64 dots, token-major.
int orc_gemm_f64(int kind, int64_t n_cols, int64_t n_tokens, const uint8_t* w, int64_t w_len,
                 const float* x, int64_t x_len, double* out, int64_t out_len) {
  const int64_t rb = orc_row_bytes(kind, n_cols);
  if (rb < 0) return (int)-rb;
  if (n_tokens <= 0 || x_len != n_tokens * n_cols || out_len % n_tokens != 0) return ORC_ERR_SIZE;
  const int64_t n_rows = out_len / n_tokens;
  if (w_len != rb * n_rows) return ORC_ERR_SIZE;
  std::vector<float> wr((size_t)n_cols);
  for (int64_t r = 0; r < n_rows; ++r) {
    const int rc = orc_dequant_row(kind, n_cols, w + r * rb, rb, wr.data(), n_cols);
    if (rc) return rc;
    for (int64_t t = 0; t < n_tokens; ++t) {
      double s = 0.0;
      const float* xt = x + t * n_cols;
      for (int64_t c = 0; c < n_cols; ++c) s += (double)wr[(size_t)c] * (double)xt[c];
      out[t * n_rows + r] = s;
    }
  }
  return ORC_OK;
}

int orc_gemv_q8_0_q8_0(int64_t n_cols, const uint8_t* w, int64_t w_len, const uint8_t* xq,
                       int64_t xq_len, float* y, int64_t y_len, int simd) {
  const int64_t rb = orc_row_bytes(ORC_Q8_0, n_cols);
  if (rb < 0) return (int)-rb;
  if (xq_len != rb || w_len != rb * y_len) return ORC_ERR_SIZE;
  const bool vec = simd && cpu_ok();
  for (int64_t r = 0; r < y_len; ++r)
    y[r] = vec ? dot_q8_0_q8_0(w + r * rb, xq, n_cols / 32)
               : orc_dot_q8_0_q8_0_row_scalar(w + r * rb, xq, n_cols / 32);
  return ORC_OK;
}

}  // extern "C"
