// Device building blocks of the integer tensor-core decode kernels (llr_gemv_stream.cu):
// shared-memory geometry, TMA / mbarrier / mma.sync wrappers, the per-format block routines
// and the activation digit split.
//
// Arithmetic.  Per 256-column block an activation row is scaled by a power of two so that the
// block maximum lands in [2^29, 2^30) and rounded to an integer X; X is written as four signed
// base-256 digits, X = d0 + 256 d1 + 256^2 d2 + 256^3 d3 with d in [-128, 127]: the digits are
// simply the bytes of (X + 0x80808080) ^ 0x80808080.  Each digit plane is an int8 B operand
// of mma.sync, the quants are the A operand, the int32 sums are exact, sub-block scales are
// folded in with integer multiply-adds, and one int->float conversion plus one FMA per (row,
// super-block, digit) applies d * 2^-e * 256^p.  The conversion rounds once when a sum exceeds
// 2^24 (relative 2^-25), everything before it is exact.
#pragma once
#include "llr_formats.cuh"
#include "llr_kernels.cuh"

namespace llr {
namespace mma {

constexpr int NWARP = 8;
constexpr int NST = 2;          // chunks in flight per CTA
// Columns whose digit planes live in shared memory at a time, and the plane pitch (32 mod 128
// bytes: conflict-free 8-byte reads).  An n-tile has eight B columns = two activation rows x four
// digits.  With a single activation row the second row's planes would be all zero: they are not
// stored, and the span is twice as long in the same
// shared memory, which halves the number of activation splits of a long row (ffn_down).
template <int MT> struct Sp {
  static constexpr int SPAN = MT == 1 ? 8192 : 4096;
  static constexpr int DS = SPAN + 32;
  static constexpr int PLANES = MT == 1 ? 4 : ((MT + 1) / 2) * 8;
};
// plane of B column g of n-tile nt; with one activation row columns 4..7 alias 0..3: their integer
// sums are garbage, and are multiplied by the zero scale every routine applies to rows >= MT
template <int MT> __device__ __forceinline__ const uint8_t* plane_of(const uint8_t* dig, int nt, int g) {
  return dig + (size_t)(MT == 1 ? (g & 3) : nt * 8 + g) * Sp<MT>::DS;
}
constexpr int SPIN_LIMIT = 1 << 22;

template <int DT> struct Fmt;
template <> struct Fmt<DT_Q4_K> { static constexpr int KSEG = 4096, BB = 144, BE = 256; };
template <> struct Fmt<DT_Q6_K> { static constexpr int KSEG = 2048, BB = 210, BE = 256; };
template <> struct Fmt<DT_Q8_0> { static constexpr int KSEG = 2048, BB = 34, BE = 32; };
template <> struct Fmt<DT_Q4_0> { static constexpr int KSEG = 4096, BB = 18, BE = 32; };
template <> struct Fmt<DT_Q5_0> { static constexpr int KSEG = 2048, BB = 22, BE = 32; };
template <> struct Fmt<DT_Q5_1> { static constexpr int KSEG = 2048, BB = 24, BE = 32; };
template <> struct Fmt<DT_Q4_1> { static constexpr int KSEG = 2048, BB = 20, BE = 32; };
template <> struct Fmt<DT_Q5_K> { static constexpr int KSEG = 2048, BB = 176, BE = 256; };

template <int DT, int MT> struct Lay {
  using F = Fmt<DT>;
  static constexpr int NT = (MT + 1) / 2;                       // n-tiles of 2 activation rows
  static constexpr int SEGB = F::KSEG / F::BE * F::BB;          // bytes of one row segment
  // row stride mod 128: 32 spreads the 8-byte fragment reads of eight rows over all banks,
  // 16 does the same for the 4-byte reads of Q6_K
  static constexpr int RMOD = (DT == DT_Q6_K || DT == DT_Q4_0 || DT == DT_Q5_0 || DT == DT_Q5_1 || DT == DT_Q4_1) ? 16 : 32;
  static constexpr int RS = SEGB + (RMOD + 128 - SEGB % 128) % 128;
  static constexpr int CHUNK = 16 * RS;
  static_assert(RS % 16 == 0 && RS % 128 == RMOD, "row stride");
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t* b, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(b)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* b, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(b)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* b, uint32_t parity) {
  uint32_t ok;
  asm volatile("{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
               : "=r"(ok) : "r"(smem_u32(b)), "r"(parity) : "memory");
  return ok != 0;
}
// untiled bulk copy global -> this CTA's shared memory; both addresses and the
// size are multiples of 16 bytes (checked on the host before this kernel is chosen)
// L2 policies: weights are read once per token and must not push the (tiny, re-read by every
// CTA) activations out of L2; activations are kept.
__device__ __forceinline__ uint64_t l2_policy_evict_first() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
  return p;
}
__device__ __forceinline__ uint64_t l2_policy_evict_last() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(p));
  return p;
}
__device__ __forceinline__ void bulk_g2s_hint(void* dst, const void* src, uint32_t bytes, uint64_t* bar, uint64_t policy) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;"
               ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)), "l"(policy) : "memory");
}
// 16 bytes of activations, L2-coherent (ld.global.cg semantics: never from a stale L1 line), kept in L2
__device__ __forceinline__ float4 ld_x_keep(const float4* p, uint64_t policy) {
  float4 v;
  asm volatile("ld.global.cg.L2::cache_hint.v4.f32 {%0,%1,%2,%3}, [%4], %5;"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p), "l"(policy) : "memory");
  return v;
}
// 16 bytes global -> shared, asynchronous (cp.async.commit_group / wait_group complete it); both addresses 16-byte aligned
__device__ __forceinline__ void cp_async16(void* dst, const void* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}
// tiled TMA loads (global -> this CTA's shared memory) with an L2 policy; the innermost
// coordinate times the element size is a multiple of 16 bytes at every call site
__device__ __forceinline__ void tma_box_2d(void* dst, const void* map, int x, int y, uint64_t* bar, uint64_t policy) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%2, %3}], [%4], %5;"
               ::"r"(smem_u32(dst)), "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar)), "l"(policy) : "memory");
}
__device__ __forceinline__ void tma_box_3d(void* dst, const void* map, int x, int y, int z, uint64_t* bar, uint64_t policy) {
  asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%2, %3, %4}], [%5], %6;"
               ::"r"(smem_u32(dst)), "l"(map), "r"(x), "r"(y), "r"(z), "r"(smem_u32(bar)), "l"(policy) : "memory");
}
__device__ __forceinline__ void mma_k32(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                        uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
               : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
}
// unsigned A operand (bytes 0..255) against signed B
__device__ __forceinline__ void mma_k32_us(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                           uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
               : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
}
__device__ __forceinline__ void mma_k16(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t b0) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%7,%7,%7,%7};"
               : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
               : "r"(a0), "r"(a1), "r"(b0), "r"(0));
}
__device__ __forceinline__ float h2f(uint32_t h) { return __half2float(__ushort_as_half((unsigned short)h)); }

// Per-thread accumulators of one chunk: yacc[nt][0..1] row g, [2..3] row g+8,
// columns 2t, 2t+1 of n-tile nt; ymin only for Q4_K.
template <int MT> struct AccT {
  static constexpr int NT = (MT + 1) / 2;
  float y[NT][4];
  float mn[2][MT];
};
template <int DT, int MT> using Acc = AccT<MT>;

// One Q4_K super-block (256 columns) of rows g and g+8 against every n-tile; pA / pB point at
// the 144 bytes of the block in row g / g+8.
// Low nibbles are an int8 A operand after one AND.  High nibbles stay where they are: the bytes
// 16 q are an unsigned A operand, their sums go to a second accumulator, and the 1/16 is part of
// the final scale (a power of two, so the int -> float rounding is the same).
// K5: the block is a Q5_K one (176 bytes: the same 16-byte header, then 32 bytes whose bit 2G / 2G+1 is the fifth
// bit of the low / high nibble of quant byte l of group G, then the 128 quant bytes).  Codes 0..31 are built in
// the low five bits of every byte for both halves, so both sums carry the same weight.
template <int MT, bool K5 = false>
__device__ __forceinline__ void block_q4k(const uint8_t* pA, const uint8_t* pB, int cb,
                                          const uint8_t* dig, const float* sxf, const float* xsi,
                                          int g, int t, Acc<DT_Q4_K, MT>& acc) {
  constexpr int NT = (MT + 1) / 2;
  constexpr int QS = K5 ? 48 : 16;
  uint2 fA = make_uint2(0u, 0u), fB = make_uint2(0u, 0u);
  if (K5) { fA = *(const uint2*)(pA + 16 + 8 * t); fB = *(const uint2*)(pB + 16 + 8 * t); }
  const uint4 hA = *(const uint4*)pA, hB = *(const uint4*)pB;
  // 6-bit scales and mins packed four to a word: bytes 0..3 = sub-blocks 0..3 (word 0), 4..7 (word 1)
  const uint32_t scA0 = hA.y & 0x3f3f3f3fu, scA1 = (hA.w & 0x0f0f0f0fu) | ((hA.y >> 2) & 0x30303030u);
  const uint32_t scB0 = hB.y & 0x3f3f3f3fu, scB1 = (hB.w & 0x0f0f0f0fu) | ((hB.y >> 2) & 0x30303030u);
  int Tl[NT][4], Th[NT][4];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt)
#pragma unroll
    for (int i = 0; i < 4; ++i) Tl[nt][i] = Th[nt][i] = 0;
#pragma unroll
  for (int G = 0; G < 4; ++G) {
    const uint2 wA = *(const uint2*)(pA + QS + G * 32 + 8 * t);
    const uint2 wB = *(const uint2*)(pB + QS + G * 32 + 8 * t);
    constexpr uint32_t M4 = 0x0f0f0f0fu, MH = 0xf0f0f0f0u, B5 = 0x10101010u;
    const uint32_t scAp = G < 2 ? scA0 : scA1, scBp = G < 2 ? scB0 : scB1;
    // byte 2 (G & 1) and the next one, zero-extended: one byte permute each
    const int sAlo = (int)__byte_perm(scAp, 0, 0x4440 + 2 * (G & 1)), sAhi = (int)__byte_perm(scAp, 0, 0x4441 + 2 * (G & 1));
    const int sBlo = (int)__byte_perm(scBp, 0, 0x4440 + 2 * (G & 1)), sBhi = (int)__byte_perm(scBp, 0, 0x4441 + 2 * (G & 1));
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      const uint8_t* dp = plane_of<MT>(dig, nt, g) + cb * 256 + G * 64 + 8 * t;
      const uint2 blo = *(const uint2*)dp, bhi = *(const uint2*)(dp + 32);
      int clo[4], chi[4];
      if (K5) {
        // bit 2G of a mask byte moves to bit 4: a shift by 4 - 2G (left for G < 2, right for G = 3)
        auto fifth = [](uint32_t f, int bit) { return (bit <= 4 ? f << (4 - bit) : f >> (bit - 4)) & B5; };
        mma_k32(clo, (wA.x & M4) | fifth(fA.x, 2 * G), (wB.x & M4) | fifth(fB.x, 2 * G),
                (wA.y & M4) | fifth(fA.y, 2 * G), (wB.y & M4) | fifth(fB.y, 2 * G), blo.x, blo.y);
        mma_k32(chi, ((wA.x >> 4) & M4) | fifth(fA.x, 2 * G + 1), ((wB.x >> 4) & M4) | fifth(fB.x, 2 * G + 1),
                ((wA.y >> 4) & M4) | fifth(fA.y, 2 * G + 1), ((wB.y >> 4) & M4) | fifth(fB.y, 2 * G + 1), bhi.x, bhi.y);
      } else {
        mma_k32(clo, wA.x & M4, wB.x & M4, wA.y & M4, wB.y & M4, blo.x, blo.y);
        mma_k32_us(chi, wA.x & MH, wB.x & MH, wA.y & MH, wB.y & MH, bhi.x, bhi.y);
      }
      Tl[nt][0] += sAlo * clo[0]; Th[nt][0] += sAhi * chi[0];
      Tl[nt][1] += sAlo * clo[1]; Th[nt][1] += sAhi * chi[1];
      Tl[nt][2] += sBlo * clo[2]; Th[nt][2] += sBhi * chi[2];
      Tl[nt][3] += sBlo * clo[3]; Th[nt][3] += sBhi * chi[3];
    }
  }
  const float dA = h2f(hA.x & 0xffffu), dminA = h2f(hA.x >> 16);
  const float dB = h2f(hB.x & 0xffffu), dminB = h2f(hB.x >> 16);
  // columns 2t, 2t+1 of an n-tile are activation row (t >> 1), digits 2(t&1) and 2(t&1)+1;
  // the weights are 256^digit / 16
  const float pw0 = K5 ? ((t & 1) ? 65536.f : 1.f) : ((t & 1) ? 4096.f : 0.0625f), pw1 = pw0 * 256.f;
  constexpr int LW = K5 ? 1 : 16;  // weight of the low-nibble sums relative to the high-nibble ones
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    const int tok = 2 * nt + (t >> 1);
    const float xs = tok < MT ? xsi[tok * (Sp<MT>::SPAN / 256) + cb] : 0.f;
    // 16 Tl + Th < 2^31: |Tl| <= 4 * 63 * 32 * 15 * 128 < 2^24 and |Th| <= 16 times that (Q5_K: both < 2^25)
    acc.y[nt][0] = fmaf((float)(Tl[nt][0] * LW + Th[nt][0]), dA * xs * pw0, acc.y[nt][0]);
    acc.y[nt][1] = fmaf((float)(Tl[nt][1] * LW + Th[nt][1]), dA * xs * pw1, acc.y[nt][1]);
    acc.y[nt][2] = fmaf((float)(Tl[nt][2] * LW + Th[nt][2]), dB * xs * pw0, acc.y[nt][2]);
    acc.y[nt][3] = fmaf((float)(Tl[nt][3] * LW + Th[nt][3]), dB * xs * pw1, acc.y[nt][3]);
  }
  // mins: this thread covers sub-blocks t and t + 4 of both rows.  Byte t of header words 2 and 3
  // of both rows side by side (row g in byte 0, row g+8 in byte 2), so that the 6-bit fields of
  // the two rows are assembled together.
  const uint32_t sel = 0x4040u + (uint32_t)t + ((uint32_t)(4 + t) << 8);  // bytes 1 and 3 are masked off below
  const uint32_t zz = __byte_perm(hA.z, hB.z, sel), ww = __byte_perm(hA.w, hB.w, sel);
  const uint32_t mlo = zz & 0x003f003fu;
  const uint32_t mhi = ((ww >> 4) & 0x000f000fu) | ((zz >> 2) & 0x00300030u);
  const float a0 = dminA * (float)(mlo & 0xffu), a1 = dminA * (float)(mhi & 0xffu);
  const float b0 = dminB * (float)((mlo >> 16) & 0xffu), b1 = dminB * (float)((mhi >> 16) & 0xffu);
#pragma unroll
  for (int k = 0; k < MT; ++k) {
    const float s0 = sxf[k * (Sp<MT>::SPAN / 32) + cb * 8 + t], s1 = sxf[k * (Sp<MT>::SPAN / 32) + cb * 8 + t + 4];
    acc.mn[0][k] = fmaf(a0, s0, fmaf(a1, s1, acc.mn[0][k]));
    acc.mn[1][k] = fmaf(b0, s0, fmaf(b1, s1, acc.mn[1][k]));
  }
}

// Four bytes at p.  Q6_K blocks are 210 bytes long and row pieces start 16-byte aligned, so the
// bytes of an odd block sit 2 bytes off a word boundary: two aligned words and a funnel shift.
template <bool ODD> __device__ __forceinline__ uint32_t lds32_par(const uint8_t* p) {
  if (!ODD) return *(const uint32_t*)p;
  return __funnelshift_r(*(const uint32_t*)(p - 2), *(const uint32_t*)(p + 2), 16);
}

// One Q6_K super-block: 16 scale groups of 16 columns, one m16n8k16 each; pA / pB point at the
// 210 bytes of the block in row g / g+8, ODD says whether they are 2 bytes off a word boundary
// (a template parameter: with a run-time flag the compiler issued the loads of both cases).
// The A operand is (code << 2) ^ 0x80 per byte = 4 (code - 32) as int8: the two high bits come
// from qh, whose bit 1 of every 2-bit field is flipped once per word, the four low bits from
// ql shifted by two; the 1/4 is part of the final scale (a power of two, so the int -> float
// rounding is the same).
template <int MT, bool ODD>
__device__ __forceinline__ void block_q6k_par(const uint8_t* pA, const uint8_t* pB, int cb,
                                              const uint8_t* dig, const float* xsi, int g, int t,
                                              Acc<DT_Q6_K, MT>& acc) {
  constexpr int NT = (MT + 1) / 2;
  int T[NT][4];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt)
#pragma unroll
    for (int i = 0; i < 4; ++i) T[nt][i] = 0;
#pragma unroll
  for (int half = 0; half < 2; ++half) {
#pragma unroll
    for (int hg = 0; hg < 2; ++hg) {  // l = 16*hg + 4t .. +3 of the 32-wide runs
      const int l = 16 * hg + 4 * t;
      const uint32_t qlA0 = lds32_par<ODD>(pA + half * 64 + l), qlA1 = lds32_par<ODD>(pA + half * 64 + 32 + l);
      const uint32_t qhA = lds32_par<ODD>(pA + 128 + half * 32 + l) ^ 0xaaaaaaaau;
      const uint32_t qlB0 = lds32_par<ODD>(pB + half * 64 + l), qlB1 = lds32_par<ODD>(pB + half * 64 + 32 + l);
      const uint32_t qhB = lds32_par<ODD>(pB + 128 + half * 32 + l) ^ 0xaaaaaaaau;
      constexpr uint32_t ML = 0x3c3c3c3cu, MH = 0xc0c0c0c0u;
#pragma unroll
      for (int qtr = 0; qtr < 4; ++qtr) {
        const uint32_t lA = (qtr & 1) ? qlA1 : qlA0, lB = (qtr & 1) ? qlB1 : qlB0;
        const uint32_t lsA = (qtr & 2) ? (lA >> 2) : (lA << 2), lsB = (qtr & 2) ? (lB >> 2) : (lB << 2);
        const uint32_t cA = (lsA & ML) | ((qhA << (6 - 2 * qtr)) & MH);
        const uint32_t cB = (lsB & ML) | ((qhB << (6 - 2 * qtr)) & MH);
        const int sidx = 192 + half * 8 + hg + 2 * qtr;
        const int sA = (int)(int8_t)pA[sidx], sB = (int)(int8_t)pB[sidx];
        const int col = cb * 256 + half * 128 + qtr * 32 + l;  // first of this thread's 4 columns
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          const uint32_t bd = *(const uint32_t*)(plane_of<MT>(dig, nt, g) + col);
          int c[4];
          mma_k16(c, cA, cB, bd);
          T[nt][0] += sA * c[0]; T[nt][1] += sA * c[1];
          T[nt][2] += sB * c[2]; T[nt][3] += sB * c[3];
        }
      }
    }
  }
  // |T| <= 16 groups * 128 * 16 columns * 128 * 128 < 2^31
  const float dA = h2f(*(const uint16_t*)(pA + 208)), dB = h2f(*(const uint16_t*)(pB + 208));
  const float pw0 = (t & 1) ? 16384.f : 0.25f, pw1 = pw0 * 256.f;  // 256^digit / 4
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    const int tok = 2 * nt + (t >> 1);
    const float xs = tok < MT ? xsi[tok * (Sp<MT>::SPAN / 256) + cb] : 0.f;
    acc.y[nt][0] = fmaf((float)T[nt][0], dA * xs * pw0, acc.y[nt][0]);
    acc.y[nt][1] = fmaf((float)T[nt][1], dA * xs * pw1, acc.y[nt][1]);
    acc.y[nt][2] = fmaf((float)T[nt][2], dB * xs * pw0, acc.y[nt][2]);
    acc.y[nt][3] = fmaf((float)T[nt][3], dB * xs * pw1, acc.y[nt][3]);
  }
}
// block b of the row pieces rowA / rowB
template <int MT>
__device__ __forceinline__ void block_q6k(const uint8_t* rowA, const uint8_t* rowB, int b, int cb,
                                          const uint8_t* dig, const float* xsi, int g, int t,
                                          Acc<DT_Q6_K, MT>& acc) {
  if (b & 1) block_q6k_par<MT, true>(rowA + b * 210, rowB + b * 210, cb, dig, xsi, g, t, acc);
  else block_q6k_par<MT, false>(rowA + b * 210, rowB + b * 210, cb, dig, xsi, g, t, acc);
}

// For the 32-column formats: per pair of activation rows, the scale of this thread's row in the 256-column group c256
// times `pw`, the weight of the lower of the two digits the thread holds (a power of two, so the order of the
// products does not matter).  Computed once per group of eight blocks.
template <int MT>
__device__ __forceinline__ void group_scales(const float* xsi, int c256, int t, float pw, float (&xw)[(MT + 1) / 2]) {
#pragma unroll
  for (int nt = 0; nt < (MT + 1) / 2; ++nt) {
    const int tok = 2 * nt + (t >> 1);
    xw[nt] = (tok < MT ? xsi[tok * (Sp<MT>::SPAN / 256) + c256] : 0.f) * pw;
  }
}

// One Q8_0 block (32 columns): the int8 quants are the A fragment as they lie.  Blocks are 34
// bytes long: the quants of an even block start 2 bytes off a word boundary (OFF).
template <int MT, bool OFF>
__device__ __forceinline__ void block_q80_par(const uint8_t* pA, const uint8_t* pB, int c32,
                                              const uint8_t* dig, const float (&xw)[(MT + 1) / 2], int g, int t,
                                              Acc<DT_Q8_0, MT>& acc) {
  constexpr int NT = (MT + 1) / 2;
  uint2 wA, wB;
  if (!OFF) {
    wA = make_uint2(*(const uint32_t*)(pA + 2 + 8 * t), *(const uint32_t*)(pA + 6 + 8 * t));
    wB = make_uint2(*(const uint32_t*)(pB + 2 + 8 * t), *(const uint32_t*)(pB + 6 + 8 * t));
  } else {
    const uint32_t a0 = *(const uint32_t*)(pA + 8 * t), a1 = *(const uint32_t*)(pA + 4 + 8 * t), a2 = *(const uint32_t*)(pA + 8 + 8 * t);
    const uint32_t b0 = *(const uint32_t*)(pB + 8 * t), b1 = *(const uint32_t*)(pB + 4 + 8 * t), b2 = *(const uint32_t*)(pB + 8 + 8 * t);
    wA = make_uint2(__funnelshift_r(a0, a1, 16), __funnelshift_r(a1, a2, 16));
    wB = make_uint2(__funnelshift_r(b0, b1, 16), __funnelshift_r(b1, b2, 16));
  }
  const float dA = h2f(*(const uint16_t*)pA), dB = h2f(*(const uint16_t*)pB);
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    const uint2 bd = *(const uint2*)(plane_of<MT>(dig, nt, g) + c32 * 32 + 8 * t);
    int c[4];
    mma_k32(c, wA.x, wB.x, wA.y, wB.y, bd.x, bd.y);
    // the two digits a thread holds are joined as integers (|sum| < 2^20 each, so c0 + 256 c1 fits 32 bits): one
    // conversion and one FMA per row instead of two; the conversion rounds to 24 bits, relative 2^-25 of the pair
    acc.y[nt][0] = fmaf((float)(c[0] + 256 * c[1]), dA * xw[nt], acc.y[nt][0]);
    acc.y[nt][2] = fmaf((float)(c[2] + 256 * c[3]), dB * xw[nt], acc.y[nt][2]);
  }
}
// block b of the row pieces rowA / rowB (row pieces start 16-byte aligned)
template <int MT>
__device__ __forceinline__ void block_q80(const uint8_t* rowA, const uint8_t* rowB, int b, int c32,
                                          const uint8_t* dig, const float (&xw)[(MT + 1) / 2], int g, int t,
                                          Acc<DT_Q8_0, MT>& acc) {
  if (b & 1) block_q80_par<MT, false>(rowA + b * 34, rowB + b * 34, c32, dig, xw, g, t, acc);
  else block_q80_par<MT, true>(rowA + b * 34, rowB + b * 34, c32, dig, xw, g, t, acc);
}


// ---- Q4_0 / Q5_0 / Q5_1: 32-column blocks whose codes are nibbles (plus a fifth bit in a 32-bit mask) --------
// Word t of the 16 quant bytes holds elements 4t..4t+3 in its low nibbles and 16+4t..16+4t+3 in its high nibbles:
// one 32-bit load per row gives thread t both of its k-slices of the A fragment, and the B fragment takes the digit
// bytes of the same elements (a sum over k does not care about the order of k as long as A and B agree).
// Signed codes become int8 without a subtraction: (code << s) ^ 0x80 is 2^s * (code - 2^(7-s)), i.e. 16 (q - 8) for
// Q4_0 and 8 (code - 16) for Q5_0; the power of two goes into the final scale.  Q5_1 codes are an unsigned operand
// and its offset m multiplies the f32 sum of the block's activations, like the mins of Q4_K.
// four bits -> the low bit of four bytes
__device__ __forceinline__ uint32_t spread4(uint32_t x) { return ((x & 15u) * 0x00204081u) & 0x01010101u; }

template <int MT, bool ODD>
__device__ __forceinline__ void block_q40_par(const uint8_t* pA, const uint8_t* pB, int c32, const uint8_t* dig,
                                              const float (&xw)[(MT + 1) / 2], int g, int t, AccT<MT>& acc) {
  constexpr int NT = (MT + 1) / 2;
  const uint32_t wA = lds32_par<ODD>(pA + 2 + 4 * t), wB = lds32_par<ODD>(pB + 2 + 4 * t);
  constexpr uint32_t MH = 0xf0f0f0f0u, SG = 0x80808080u;
  const uint32_t a0 = ((wA << 4) & MH) ^ SG, a2 = (wA & MH) ^ SG, a1 = ((wB << 4) & MH) ^ SG, a3 = (wB & MH) ^ SG;
  const float dA = h2f(*(const uint16_t*)pA), dB = h2f(*(const uint16_t*)pB);
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    const uint8_t* dp = plane_of<MT>(dig, nt, g) + c32 * 32 + 4 * t;
    int c[4];
    mma_k32(c, a0, a1, a2, a3, *(const uint32_t*)dp, *(const uint32_t*)(dp + 16));
    // the two digits a thread holds are joined as integers (|sum| < 2^20 each, so c0 + 256 c1 fits 32 bits): one
    // conversion and one FMA per row instead of two; the conversion rounds to 24 bits, relative 2^-25 of the pair
    acc.y[nt][0] = fmaf((float)(c[0] + 256 * c[1]), dA * xw[nt], acc.y[nt][0]);
    acc.y[nt][2] = fmaf((float)(c[2] + 256 * c[3]), dB * xw[nt], acc.y[nt][2]);
  }
}
template <int MT>
__device__ __forceinline__ void block_q40(const uint8_t* rowA, const uint8_t* rowB, int b, int c32, const uint8_t* dig,
                                          const float (&xw)[(MT + 1) / 2], int g, int t, AccT<MT>& acc) {
  // 18-byte blocks in a 16-byte aligned row piece: the quants of an even block start 2 bytes off a word boundary
  if (b & 1) block_q40_par<MT, false>(rowA + b * 18, rowB + b * 18, c32, dig, xw, g, t, acc);
  else block_q40_par<MT, true>(rowA + b * 18, rowB + b * 18, c32, dig, xw, g, t, acc);
}

// HDR: bytes before the fifth-bit mask (2: Q5_0, 4: Q5_1)
template <int MT, bool ODD, bool Q51>
__device__ __forceinline__ void block_q5_par(const uint8_t* pA, const uint8_t* pB, int c32, const uint8_t* dig,
                                             const float* sxf, const float (&xw)[(MT + 1) / 2], int g, int t, AccT<MT>& acc) {
  constexpr int NT = (MT + 1) / 2;
  constexpr int HDR = Q51 ? 4 : 2;
  const uint32_t hA = lds32_par<ODD>(pA + HDR), hB = lds32_par<ODD>(pB + HDR);
  const uint32_t wA = lds32_par<ODD>(pA + HDR + 4 + 4 * t), wB = lds32_par<ODD>(pB + HDR + 4 + 4 * t);
  uint32_t a0, a1, a2, a3;
  if (Q51) {  // codes 0..31 as they are
    constexpr uint32_t M4 = 0x0f0f0f0fu;
    a0 = (wA & M4) | (spread4(hA >> (4 * t)) << 4);
    a2 = ((wA >> 4) & M4) | (spread4(hA >> (16 + 4 * t)) << 4);
    a1 = (wB & M4) | (spread4(hB >> (4 * t)) << 4);
    a3 = ((wB >> 4) & M4) | (spread4(hB >> (16 + 4 * t)) << 4);
  } else {    // 8 (code - 16)
    constexpr uint32_t M5 = 0x78787878u, SG = 0x80808080u;
    a0 = (((wA << 3) & M5) | (spread4(hA >> (4 * t)) << 7)) ^ SG;
    a2 = (((wA >> 1) & M5) | (spread4(hA >> (16 + 4 * t)) << 7)) ^ SG;
    a1 = (((wB << 3) & M5) | (spread4(hB >> (4 * t)) << 7)) ^ SG;
    a3 = (((wB >> 1) & M5) | (spread4(hB >> (16 + 4 * t)) << 7)) ^ SG;
  }
  const float dA = h2f(*(const uint16_t*)pA), dB = h2f(*(const uint16_t*)pB);
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    const uint8_t* dp = plane_of<MT>(dig, nt, g) + c32 * 32 + 4 * t;
    int c[4];
    if (Q51) mma_k32_us(c, a0, a1, a2, a3, *(const uint32_t*)dp, *(const uint32_t*)(dp + 16));
    else mma_k32(c, a0, a1, a2, a3, *(const uint32_t*)dp, *(const uint32_t*)(dp + 16));
    // the two digits a thread holds are joined as integers (|sum| < 2^20 each, so c0 + 256 c1 fits 32 bits): one
    // conversion and one FMA per row instead of two; the conversion rounds to 24 bits, relative 2^-25 of the pair
    acc.y[nt][0] = fmaf((float)(c[0] + 256 * c[1]), dA * xw[nt], acc.y[nt][0]);
    acc.y[nt][2] = fmaf((float)(c[2] + 256 * c[3]), dB * xw[nt], acc.y[nt][2]);
  }
  if (Q51 && t == (c32 & 3)) {
    // the offset: m * sum of the block's activations, kept negative so that the tile's `sum - mn` adds it; one of the
    // four threads that see this block does it (the four are summed when the tile is handed over)
    const float mA = h2f(*(const uint16_t*)(pA + 2)), mB = h2f(*(const uint16_t*)(pB + 2));
#pragma unroll
    for (int k = 0; k < MT; ++k) {
      const float sx = sxf[k * (Sp<MT>::SPAN / 32) + c32];
      acc.mn[0][k] = fmaf(-mA, sx, acc.mn[0][k]);
      acc.mn[1][k] = fmaf(-mB, sx, acc.mn[1][k]);
    }
  }
}
template <int MT>
__device__ __forceinline__ void block_q50(const uint8_t* rowA, const uint8_t* rowB, int b, int c32, const uint8_t* dig,
                                          const float* sxf, const float (&xw)[(MT + 1) / 2], int g, int t, AccT<MT>& acc) {
  if (b & 1) block_q5_par<MT, false, false>(rowA + b * 22, rowB + b * 22, c32, dig, sxf, xw, g, t, acc);
  else block_q5_par<MT, true, false>(rowA + b * 22, rowB + b * 22, c32, dig, sxf, xw, g, t, acc);
}
template <int MT>
__device__ __forceinline__ void block_q51(const uint8_t* rowA, const uint8_t* rowB, int b, int c32, const uint8_t* dig,
                                          const float* sxf, const float (&xw)[(MT + 1) / 2], int g, int t, AccT<MT>& acc) {
  block_q5_par<MT, false, true>(rowA + b * 24, rowB + b * 24, c32, dig, sxf, xw, g, t, acc);  // 24-byte blocks stay word aligned
}

// Q4_1: 20-byte blocks {d, m, 16 quant bytes}; codes 0..15 as an unsigned operand, the offset like Q5_1's
template <int MT>
__device__ __forceinline__ void block_q41(const uint8_t* rowA, const uint8_t* rowB, int b, int c32, const uint8_t* dig,
                                          const float* sxf, const float (&xw)[(MT + 1) / 2], int g, int t, AccT<MT>& acc) {
  constexpr int NT = (MT + 1) / 2;
  const uint8_t* pA = rowA + b * 20;  // 20-byte blocks stay word aligned
  const uint8_t* pB = rowB + b * 20;
  const uint32_t wA = *(const uint32_t*)(pA + 4 + 4 * t), wB = *(const uint32_t*)(pB + 4 + 4 * t);
  constexpr uint32_t M4 = 0x0f0f0f0fu;
  const uint32_t a0 = wA & M4, a2 = (wA >> 4) & M4, a1 = wB & M4, a3 = (wB >> 4) & M4;
  const uint32_t hdA = *(const uint32_t*)pA, hdB = *(const uint32_t*)pB;
  const float dA = h2f(hdA & 0xffffu), dB = h2f(hdB & 0xffffu);
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    const uint8_t* dp = plane_of<MT>(dig, nt, g) + c32 * 32 + 4 * t;
    int c[4];
    mma_k32(c, a0, a1, a2, a3, *(const uint32_t*)dp, *(const uint32_t*)(dp + 16));
    acc.y[nt][0] = fmaf((float)(c[0] + 256 * c[1]), dA * xw[nt], acc.y[nt][0]);
    acc.y[nt][2] = fmaf((float)(c[2] + 256 * c[3]), dB * xw[nt], acc.y[nt][2]);
  }
  if (t == (c32 & 3)) {
    const float mA = h2f(hdA >> 16), mB = h2f(hdB >> 16);
#pragma unroll
    for (int k = 0; k < MT; ++k) {
      const float sx = sxf[k * (Sp<MT>::SPAN / 32) + c32];
      acc.mn[0][k] = fmaf(-mA, sx, acc.mn[0][k]);
      acc.mn[1][k] = fmaf(-mB, sx, acc.mn[1][k]);
    }
  }
}

// ---- where activations come from ---------------------------------------------------------
// Plain f32 memory that is ready when the launch starts, or tagged pairs {f32 bits, tag} that an
// earlier phase of the same launch writes (on this GPU or, in a row-sharded program, on another):
// a pair whose tag is the expected one carries a finished value, so loading it IS the wait.
struct XSrc {
  const float* x;     // plain input (used when xt is null)
  const uint2* xt;    // tagged input
  const void* x2;     // XOP_RMSNORM: norm weights (plain, may be null); XOP_SWIGLU: `up`, plain or tagged
  uint32_t tag, tag2; // expected tags of xt / x2
  int op;             // XOP_*
  int x2_tagged;
};
// State of a warp's bounded waits on tagged data.  Once a wait has run out anywhere in the launch
// (this warp: dead; another CTA: the abort word holds this run's epoch) later waits return at once,
// so a launch that lost a producer finishes in about its normal time.
struct WaitCtx {
  int* err;
  unsigned long long* abort_word;
  unsigned long long epoch;
  int limit;
  bool dead;
};
template <bool SYS> __device__ __forceinline__ void ld_pairs2(const void* p, unsigned long long& a, unsigned long long& b) {
  if (SYS) asm volatile("ld.relaxed.sys.global.v2.b64 {%0,%1}, [%2];" : "=l"(a), "=l"(b) : "l"(p) : "memory");
  else asm volatile("ld.relaxed.gpu.global.v2.b64 {%0,%1}, [%2];" : "=l"(a), "=l"(b) : "l"(p) : "memory");
}
template <bool SYS> __device__ __forceinline__ unsigned long long ld_pair(const void* p) {
  unsigned long long a;
  if (SYS) asm volatile("ld.relaxed.sys.global.b64 %0, [%1];" : "=l"(a) : "l"(p) : "memory");
  else asm volatile("ld.relaxed.gpu.global.b64 %0, [%1];" : "=l"(a) : "l"(p) : "memory");
  return a;
}
template <bool SYS> __device__ __forceinline__ void st_pair(void* p, float v, uint32_t tag) {
  const unsigned long long a = ((unsigned long long)tag << 32) | (unsigned long long)__float_as_uint(v);
  if (SYS) asm volatile("st.relaxed.sys.global.b64 [%0], %1;" ::"l"(p), "l"(a) : "memory");
  else asm volatile("st.relaxed.gpu.global.b64 [%0], %1;" ::"l"(p), "l"(a) : "memory");
}
// A wait on tagged data ran out, or another CTA's did: record it.  Returns true when the caller should stop waiting.
__device__ __forceinline__ bool wait_step(int& polls, WaitCtx& wc) {
  ++polls;
  if ((polls & 15) == 0 && ld_pair<false>(wc.abort_word) == wc.epoch) { wc.dead = true; return true; }
  if (polls > wc.limit) {
    wc.dead = true;
    *(volatile unsigned long long*)wc.abort_word = wc.epoch;
    report_error(wc.err, 2);
    return true;
  }
  __nanosleep(polls < 8 ? 32 : 128);
  return false;
}
// One pair, polled until its tag arrives (the reducer's residual).
template <bool SYS> __device__ __forceinline__ void poll_pair(const void* p, uint32_t want, WaitCtx& wc) {
  int polls = 0;
  while ((uint32_t)(ld_pair<SYS>(p) >> 32) != want)
    if (wait_step(polls, wc)) return;
}
// Eight consecutive values per lane for NJ jobs at once (element offsets off[], inactive jobs
// skipped) from tagged pairs: all loads of all jobs are in flight before any is used.  A lane whose
// pairs do not all carry the expected tag yet loads them again after a short sleep, on its own (a
// lane's eight values are neighbours in one result tile and arrive together; lanes of different
// tiles need not wait for each other's round trips), until they do or the wait limit is reached.
template <bool SYS, int NJ>
__device__ __forceinline__ void load_tagged(const uint2* base, uint32_t want, const int64_t (&off)[NJ], const bool (&act)[NJ],
                                            float (&v)[NJ][8], WaitCtx& wc) {
  int polls = 0;
  for (;;) {
    bool late = false;
#pragma unroll
    for (int j = 0; j < NJ; ++j)
      if (act[j]) {
        unsigned long long a[8];
#pragma unroll
        for (int q = 0; q < 4; ++q) ld_pairs2<SYS>(base + off[j] + 2 * q, a[2 * q], a[2 * q + 1]);
#pragma unroll
        for (int q = 0; q < 8; ++q) {
          v[j][q] = __uint_as_float((uint32_t)a[q]);
          late = late || (uint32_t)(a[q] >> 32) != want;
        }
      }
    if (!late || wc.dead || wait_step(polls, wc)) break;
  }
  __syncwarp();
  wc.dead = __any_sync(~0u, wc.dead);
}
template <int NJ>
__device__ __forceinline__ void load_plain(const float* base, const int64_t (&off)[NJ], const bool (&act)[NJ],
                                           float (&v)[NJ][8], uint64_t keep) {
#pragma unroll
  for (int j = 0; j < NJ; ++j)
    if (act[j]) {
      const float4 pa = ld_x_keep((const float4*)(base + off[j]), keep), pb = ld_x_keep((const float4*)(base + off[j]) + 1, keep);
      v[j][0] = pa.x; v[j][1] = pa.y; v[j][2] = pa.z; v[j][3] = pa.w;
      v[j][4] = pb.x; v[j][5] = pb.y; v[j][6] = pb.z; v[j][7] = pb.w;
    }
}
// The activations of NJ jobs with the entry's element-wise operation applied (XOP_SWIGLU; the
// normalisation of XOP_RMSNORM is applied by the caller, which needs the row's sum of squares first).
template <bool SYS, int NJ>
__device__ __forceinline__ void fetch_jobs(const XSrc& s, const int64_t (&off)[NJ], const bool (&act)[NJ],
                                           float (&v)[NJ][8], WaitCtx& wc, uint64_t keep) {
  if (s.xt) load_tagged<SYS, NJ>(s.xt, s.tag, off, act, v, wc);
  else load_plain<NJ>(s.x, off, act, v, keep);
  if (s.op != XOP_SWIGLU) return;
  // silu(g) * u as the reference computes it: g / (1 + exp(-g)), then the product (decode.rs:11826, :2984)
#pragma unroll
  for (int j = 0; j < NJ; ++j)
    if (act[j]) {
#pragma unroll
      for (int q = 0; q < 8; ++q) v[j][q] = __fdiv_rn(v[j][q], 1.0f + expf(-v[j][q]));
    }
  float u[NJ][8];
  if (s.x2_tagged) load_tagged<SYS, NJ>((const uint2*)s.x2, s.tag2, off, act, u, wc);
  else load_plain<NJ>((const float*)s.x2, off, act, u, keep);
#pragma unroll
  for (int j = 0; j < NJ; ++j)
    if (act[j]) {
#pragma unroll
      for (int q = 0; q < 8; ++q) v[j][q] = __fmul_rn(v[j][q], u[j][q]);
    }
}

// Sum of squares of every activation row of an XOP_RMSNORM entry -> 1 / sqrt(mean + eps) per row
// (rmsnorm_inplace, decode.rs:11498; the reference adds sequentially, here lanes, then warps, add
// in a fixed order, so the value is reproducible but may differ from the sequential sum in the
// last bits).  Called by all eight consumer warps; part is float[NWARP][8] and inv float[8] in
// shared memory.  The second barrier also keeps a warp from writing its next partial sums while
// another still adds up these.
template <int MT, bool SYS>
__device__ __forceinline__ void row_inv_rms(const XSrc& s, int cols, int tokens, float eps, float* part, float* inv,
                                            int warp, int lane, WaitCtx& wc, uint64_t keep) {
  const int nblk = cols >> 8;
  float ss[MT];
#pragma unroll
  for (int k = 0; k < MT; ++k) ss[k] = 0.f;
  XSrc raw = s;
  raw.op = XOP_NONE;
  for (int b0 = warp; b0 < nblk; b0 += 2 * NWARP)
#pragma unroll
    for (int k = 0; k < MT; ++k) {
      if (k >= tokens) break;
      const int64_t off[2] = {(int64_t)k * cols + b0 * 256 + 8 * lane, (int64_t)k * cols + (b0 + NWARP) * 256 + 8 * lane};
      const bool act[2] = {true, b0 + NWARP < nblk};
      float v[2][8];
      fetch_jobs<SYS, 2>(raw, off, act, v, wc, keep);
#pragma unroll
      for (int j = 0; j < 2; ++j)
        if (act[j]) {
#pragma unroll
          for (int q = 0; q < 8; ++q) ss[k] = fmaf(v[j][q], v[j][q], ss[k]);
        }
    }
  float* mine = part + warp * 8;
#pragma unroll
  for (int k = 0; k < MT; ++k) {
    float t = ss[k];
#pragma unroll
    for (int m = 16; m > 0; m >>= 1) t += __shfl_xor_sync(~0u, t, m);
    if (lane == 0) mine[k] = t;
  }
  asm volatile("bar.sync 1, %0;" ::"n"(NWARP * 32) : "memory");
  if (lane < tokens) {
    float t = 0.f;
#pragma unroll
    for (int w = 0; w < NWARP; ++w) t += part[w * 8 + lane];
    const float rms = sqrtf(__fadd_rn(__fdiv_rn(t, (float)(cols <= 65535 ? cols : 1)), eps));
    if (warp == 0) inv[lane] = rms > 0.f ? __fdiv_rn(1.0f, rms) : 0.f;
  }
  asm volatile("bar.sync 1, %0;" ::"n"(NWARP * 32) : "memory");
}

// Activations of one span (nblk256 blocks of 256 columns starting at column col0, `tokens`
// activation rows) -> four int8 digit planes per activation row, the f32 sums of x per 32
// columns (Q4_K mins) and 2^-e per block.  Plain loads are L2-coherent and kept in L2 (policy
// `keep`); tagged loads wait for their values (see XSrc).
// Warp w of the eight consumer warps splits the blocks b = w (mod 8) of every activation row, and
// those are exactly the blocks whose planes, sums and scales it reads in the block routines: no
// other warp depends on what it writes here, so a __syncwarp() is all the caller needs.
template <int MT, bool SYS, bool FLOW>
__device__ __forceinline__ void split_activations(const XSrc& src, int cols, int col0,
                                                  int nblk256, int tokens, uint8_t* dig, float* sxf,
                                                  float* xsi, const float* inv, int warp, int lane, WaitCtx& wc, uint64_t keep) {
  // two jobs per pass: both loads are in flight before either is used.  One activation row: blocks
  // b0 and b0 + 8; several: rows tok0 and tok0 + 1 of block b0.
  for (int b0 = warp; b0 < nblk256; b0 += (MT == 1 ? 2 * NWARP : NWARP))
  for (int tok0 = 0; tok0 < tokens; tok0 += (MT == 1 ? 1 : 2)) {
   float vv[2][8];
   int64_t off[2];
   bool act[2];
#pragma unroll
   for (int u = 0; u < 2; ++u) {
    const int jb = MT == 1 ? b0 + u * NWARP : b0, jt = MT == 1 ? 0 : tok0 + u;
    act[u] = MT == 1 ? jb < nblk256 : jt < tokens;
    off[u] = (int64_t)jt * cols + col0 + jb * 256 + 8 * lane;
   }
   if (FLOW) fetch_jobs<SYS, 2>(src, off, act, vv, wc, keep);
   else load_plain<2>(src.x, off, act, vv, keep);
#pragma unroll
   for (int u = 0; u < 2; ++u) {
    const int b = MT == 1 ? b0 + u * NWARP : b0, tok = MT == 1 ? 0 : tok0 + u;
    if (!act[u]) break;
    float v[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = vv[u][j];
    if (FLOW && src.op == XOP_RMSNORM) {  // (x * inv) * w, two roundings as in the reference
      const float r = inv[tok];
      if (src.x2) {
        const float4 wa = __ldg((const float4*)((const float*)src.x2 + col0 + b * 256 + 8 * lane));
        const float4 wb = __ldg((const float4*)((const float*)src.x2 + col0 + b * 256 + 8 * lane) + 1);
        const float wv[8] = {wa.x, wa.y, wa.z, wa.w, wb.x, wb.y, wb.z, wb.w};
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = __fmul_rn(__fmul_rn(v[j], r), wv[j]);
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = __fmul_rn(v[j], r);
      }
    }
    // Largest magnitude of the block as a bit pattern: for non-negative floats the unsigned order of
    // the bits is the numeric order, infinities and NaNs sort above every finite value, and one
    // redux.sync replaces a five-step shuffle reduction on the latency-critical start of a phase.
    uint32_t mb = 0;
    float sum = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) { mb = max(mb, __float_as_uint(v[j]) & 0x7fffffffu); sum += v[j]; }
    mb = __reduce_max_sync(~0u, mb);
    const bool bad = mb >= 0x7f800000u;  // a non-finite activation anywhere in the block
    sum += __shfl_xor_sync(~0u, sum, 1);
    sum += __shfl_xor_sync(~0u, sum, 2);
    const int be = (int)(mb >> 23);
    float s = 0.f, sinv = 0.f;  // an all-zero (or denormal) block contributes nothing
    if (be != 0 && !bad) {
      int e = 29 - (be - 127);
      e = e > 126 ? 126 : e;
      s = __uint_as_float((uint32_t)(e + 127) << 23);
      sinv = __uint_as_float((uint32_t)(127 - e) << 23);
    }
    // digits of a value = bytes of (X + 0x80808080) ^ 0x80808080; a 4 x 4 byte transpose (eight
    // byte permutes) turns four values into one word per digit plane
    uint32_t pk[4][2];
#pragma unroll
    for (int hq = 0; hq < 2; ++hq) {
      uint32_t D[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int xi = bad ? 0 : __float2int_rn(v[4 * hq + j] * s);
        D[j] = ((uint32_t)xi + 0x80808080u) ^ 0x80808080u;
      }
      const uint32_t t0 = __byte_perm(D[0], D[1], 0x5140), t1 = __byte_perm(D[2], D[3], 0x5140);
      const uint32_t t2 = __byte_perm(D[0], D[1], 0x7362), t3 = __byte_perm(D[2], D[3], 0x7362);
      pk[0][hq] = __byte_perm(t0, t1, 0x5410);
      pk[1][hq] = __byte_perm(t0, t1, 0x7632);
      pk[2][hq] = __byte_perm(t2, t3, 0x5410);
      pk[3][hq] = __byte_perm(t2, t3, 0x7632);
    }
    const int nt = tok >> 1, plane0 = (tok & 1) * 4;
#pragma unroll
    for (int p = 0; p < 4; ++p)
      *(uint2*)(dig + (size_t)(nt * 8 + plane0 + p) * Sp<MT>::DS + b * 256 + 8 * lane) = make_uint2(pk[p][0], pk[p][1]);
    if ((lane & 3) == 0) sxf[tok * (Sp<MT>::SPAN / 32) + b * 8 + (lane >> 2)] = sum;
    // a non-finite activation makes the whole output row of that token NaN
    if (lane == 0) xsi[tok * (Sp<MT>::SPAN / 256) + b] = bad ? __uint_as_float(0x7fc00000u) : sinv;
   }
  }
}

}  // namespace mma
}  // namespace llr
