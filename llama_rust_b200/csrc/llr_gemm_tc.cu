// Chunk GEMM for many activation rows (prefill / continuous-batching chunks, routed experts):
// packed GGUF weights are dequantized tile by tile into tensor memory and fed to the
// 5th-generation tensor cores (tcgen05.mma, accumulators in tensor memory).
//
// What it computes: gemm_<t>_f32 (langtax/src/quant.rs:6282, 6366, 6380, 6478 ->
// gemm_f32_x :6760; gemm_q6_k_f32 :6296), y[t*rows + r] = sum_c W[r,c] x[t*cols + c], for Q4_K, Q6_K,
// Q8_0, Q5_0, Q5_1 and Q4_0.  Operands are 16-bit (binary16 when the matrix's weights fit its range,
// bfloat16 otherwise; see dequant_sub_h), products are exact, accumulation is f32 in
// tensor memory: this is the tensor-core path with the looser, separately stated tolerance
// (tests/test_gpu_gemm.py); the f32-faithful path for any number of rows stays the
// integer kernel of llr_gemv_stream.cu.
//
// One CTA computes a 128-row x BN-token tile of y over its K range; twenty warps:
//   * packed bytes: the packed matrix is described to the TMA unit as a 2-D array of 32-bit
//     words (row pitch = bytes per row); per 256-column macro-step one elected lane issues one
//     tiled copy of a 128-row x (144 / 272 / 176 / 208)-byte box into a shared-memory ring
//     (mbarrier transaction count).  The box width is an odd number of 16-byte chunks, so a
//     warp whose lanes are consecutive rows reads 16-byte chunks without bank conflicts
//     (Q5_1 copies 16 bytes more than its 192 to get there).
//   * dequantization: sixteen warps in two groups that alternate 64-column steps; in a
//     group two threads per row, 32 columns each.  A warp decodes both of its steps of a
//     macro-step back to back, then does one round of barrier waits, tensor-memory stores
//     and arrivals for the two.  Quants are turned into binary16 pairs with a mask-and-or
//     against a magic exponent (1024+q, or 64+q for high nibbles): no integer to float
//     conversions.  binary16 path: exact offset subtraction and one HFMA2 per two weights;
//     bfloat16 path: widen, one FMA, pack.
//   * the dequantized tile never touches shared memory: a thread owns one weight row = one
//     tensor-memory lane and writes its 32 values with tcgen05.st into a ring of A-operand
//     stages that lives in tensor memory next to the accumulators (32 columns per stage;
//     12 / 8 / 8 stages for BN = 64 / 128 / 256).  The MMA takes A from tensor memory and
//     B from shared memory.  A stage hand-off (store -> mma -> commit -> store) takes about
//     a microsecond of barrier latency, so the ring depth, not the step time, is what keeps
//     the tensor pipe fed; shared memory could not hold that many 16-bit weight tiles.
//   * one warp TMA-loads the matching BN x 64 activation tiles (2-D tensor map, 128-byte
//     swizzle, out-of-range tokens read as zero) into a 128 KB ring; one MMA warp (two with
//     separate accumulators at BN <= 128) issues four tcgen05.mma (M=128, N=BN, K=16) per
//     step, whose commits release the stages.  The issue warps run their loops converged and
//     issue through one elected lane.
// Launch forms: one product (split along K when it has few row tiles, slices added in
// order by a second kernel), or a grouped launch with the tiles of several products.
// All hand-offs are mbarriers with bounded waits.  The epilogue reads the accumulators
// with tcgen05.ld (one TMEM lane = one weight row per thread) and stores token-major.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <atomic>

#include <cstring>
#include <type_traits>
#include <vector>

#include "llr_formats.cuh"
#include "llr_kernels.cuh"
#include "llr_tmap.cuh"

namespace llr {
namespace {

constexpr int BM = 128;     // weight rows per CTA = UMMA M
constexpr int BK = 64;      // columns per stage: 64 bf16 = one 128-byte swizzle row
constexpr int MACRO = 256;  // columns per packed-byte ring stage
constexpr int DQ_WARPS = 16; // dequant warps: two groups of eight, alternating 64-column steps; the first eight also run the epilogue
constexpr int W_PACKED = DQ_WARPS, W_ACT = DQ_WARPS + 1, W_MMA = DQ_WARPS + 2;
constexpr int TC_THREADS = (DQ_WARPS + 4) * 32;  // + packed-byte, activation and two MMA issue warps
constexpr int TC_SPIN = 1 << 24;
constexpr int SMEM_LIMIT = 232448;  // 227 KB opt-in maximum per CTA

// packed bytes per row per macro-step, and the ring's row pitch (odd multiple of 16 bytes)
template <int DT> struct Pk;
template <> struct Pk<DT_Q4_K> { static constexpr int RB = 144, PITCH = 144; };
template <> struct Pk<DT_Q8_0> { static constexpr int RB = 272, PITCH = 272; };
template <> struct Pk<DT_Q5_0> { static constexpr int RB = 176, PITCH = 176; };
template <> struct Pk<DT_Q4_0> { static constexpr int RB = 144, PITCH = 144; };
template <> struct Pk<DT_Q5_1> { static constexpr int RB = 192, PITCH = 208; };
template <> struct Pk<DT_Q4_1> { static constexpr int RB = 160, PITCH = 176; };
template <> struct Pk<DT_Q5_K> { static constexpr int RB = 176, PITCH = 176; };
// Q6_K blocks are 210 bytes: the block of macro-step ms starts at 210*ms, which is a multiple of 16 bytes only
// for every eighth step.  The copy starts at the 16-byte boundary below (TMA needs that) and is 240 bytes wide
// (14 bytes of lead at most + 210, rounded up to an odd number of 16-byte chunks); the decoder adds the lead back.
template <> struct Pk<DT_Q6_K> { static constexpr int RB = 210, PITCH = 240; };

// Rings: A-operand stages in tensor memory (NA), activation tiles in shared memory (NB, 128 KB),
// packed bytes in shared memory (NPK macro-steps, whatever is left, at most 6).
template <int DT, int BN> struct GLay {
  static constexpr int TMEM_COLS = 512;
  static constexpr int A_COLS = BK / 2;  // 64 bf16 per row = 32 columns of 32 bits
  // MMA issue warps, each with its own accumulator (added in the epilogue): one thread can issue a
  // 64-column step every ~475 cycles, which at BN <= 128 is slower than the tensor pipe and the
  // dequant warps; two threads on alternating steps double that.  At BN = 256 tensor memory has no
  // room for a second accumulator and the step is bound elsewhere.
  static constexpr int NMMA = BN > 128 ? 1 : 2;
  static constexpr int NA = ((TMEM_COLS - NMMA * BN) / A_COLS) & ~1;  // even: see the dequant loop
  static constexpr int B_STAGE = BN * 128;
  static constexpr int NB = (128 * 1024) / B_STAGE;
  static constexpr int P_STAGE = BM * Pk<DT>::PITCH;
  static constexpr int B = 0;
  static constexpr int P = B + NB * B_STAGE;
  static constexpr int FIXED = 1024 /*alignment slack*/ + 1024 /*barriers*/ + 64 /*chunk reads may pass a row's end*/;
  static constexpr int NPK_FIT = (SMEM_LIMIT - FIXED - P) / P_STAGE;
  static constexpr int NPK = NPK_FIT > 6 ? 6 : NPK_FIT;
  static_assert(NPK >= 2, "packed ring needs two stages");
  static constexpr int BAR = P + NPK * P_STAGE + 64;  // full_a, empty_a [NA]; full_b, empty_b [NB]; pk_full, pk_empty [NPK]; acc_full; tmem slot
  static constexpr int TOTAL = BAR + 1024 + 1024;
  static_assert((2 * NA + 2 * NB + 2 * NPK + 2) * 8 <= 1024, "barrier block");
  static_assert(TOTAL <= SMEM_LIMIT, "shared memory");
};

// one product of a grouped launch; tile_begin = first tile number of the product in the grid
struct alignas(64) GemmGroup {
  CUtensorMap wmap, xmap;
  const float* xscale;
  float* y;
  int rows, cols, tokens, tile_begin;
};

__device__ __forceinline__ uint32_t s32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void bar_init(uint64_t* b, int n) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(s32(b)), "r"(n) : "memory");
}
__device__ __forceinline__ void bar_arrive(uint64_t* b) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(s32(b)) : "memory");
}
__device__ __forceinline__ void bar_expect(uint64_t* b, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(s32(b)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool bar_wait(uint64_t* b, uint32_t parity) {
  for (int spins = 0; spins < TC_SPIN; ++spins) {
    uint32_t ok;
    asm volatile("{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
                 : "=r"(ok) : "r"(s32(b)), "r"(parity) : "memory");
    if (ok) return true;
  }
  return false;
}

// both barriers tested in one go, so that the two round trips to the barrier unit overlap
__device__ __forceinline__ bool bar_wait2(uint64_t* a, uint32_t pa, uint64_t* b, uint32_t pb) {
  for (int spins = 0; spins < TC_SPIN; ++spins) {
    uint32_t ok;
    asm volatile(
        "{ .reg .pred p, q; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; mbarrier.try_wait.parity.shared::cta.b64 q, [%3], %4; "
        "and.pred p, p, q; selp.u32 %0, 1, 0, p; }"
        : "=r"(ok) : "r"(s32(a)), "r"(pa), "r"(s32(b)), "r"(pb) : "memory");
    if (ok) return true;
  }
  return false;
}
__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile("{ .reg .pred p; elect.sync _|p, 0xffffffff; selp.u32 %0, 1, 0, p; }" : "=r"(pred));
  return pred != 0;
}

// K-major, 128-byte swizzle shared-memory matrix descriptor: rows of 128 bytes, eight-row
// groups 1024 bytes apart, descriptor version 1 (sm_100), layout type 2 (SWIZZLE_128B).
__device__ __forceinline__ uint64_t smem_desc_u(uint32_t saddr) {
  const uint64_t addr = (uint64_t)(saddr >> 4) & 0x3fffu;
  return addr | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}

// kind::f16 instruction descriptor: D f32, A (tensor memory) and B (shared, K-major) both bf16 or both
// binary16 (format code 1 / 0; the hardware rejects a mixed pair), M = 128, N = BN.
template <int BN, bool F16> __host__ __device__ constexpr uint32_t instr_desc() {
  return (1u << 4) | ((F16 ? 0u : 1u) << 7) | ((F16 ? 0u : 1u) << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *(const uint32_t*)&v;
}
__device__ __forceinline__ float h2f(uint32_t h) { return __half2float(__ushort_as_half((unsigned short)h)); }
__device__ __forceinline__ float2 hh2ff(uint32_t h2) { return __half22float2(*(const __half2*)&h2); }

// 32 / 16 bits at a compile-time even byte offset of a word array
template <int OFF> __device__ __forceinline__ uint32_t w_at(const uint32_t* w) {
  if constexpr (OFF % 4 == 0) return w[OFF / 4];
  else return __funnelshift_r(w[OFF / 4], w[OFF / 4 + 1], 16);
}
template <int OFF> __device__ __forceinline__ uint32_t h_at(const uint32_t* w) {
  if constexpr (OFF % 4 == 0) return w[OFF / 4] & 0xffffu;
  else return w[OFF / 4] >> 16;
}
// Shared memory is addressed through 32-bit shared-window addresses and explicit ld/st.shared:
// the tile base is aligned by integer arithmetic, which would otherwise turn every access
// into a generic-address load or store.
template <int NCH> __device__ __forceinline__ void lds_chunks(uint32_t p, uint32_t (&w)[4 * NCH]) {
#pragma unroll
  for (int i = 0; i < NCH; ++i)
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(w[4 * i]), "=r"(w[4 * i + 1]), "=r"(w[4 * i + 2]), "=r"(w[4 * i + 3]) : "r"(p + 16 * i));
}

// Four unsigned bytes c0..c3 (each < 1024) -> out[0] = bf16(c0*a+nb), bf16(c1*a+nb); out[1] = c2, c3.
// MASK/MAGIC pick the bits and the binary16 exponent whose unit in the last place is one
// quant step; nb already contains minus the magic offset times a.  XORM flips a sign bit (Q8_0).
template <uint32_t MASK, uint32_t MAGIC>
__device__ __forceinline__ void emit4(uint32_t w, float a, float nb, uint32_t& o0, uint32_t& o1) {
  const float2 f = hh2ff((w & MASK) ^ MAGIC);         // elements 0 and 2
  const float2 g = hh2ff(((w >> 8) & MASK) ^ MAGIC);  // elements 1 and 3
  o0 = pack_bf16(fmaf(f.x, a, nb), fmaf(g.x, a, nb));
  o1 = pack_bf16(fmaf(f.y, a, nb), fmaf(g.y, a, nb));
}

// bit k of x (k = 0..3) -> bit 8k+4
__device__ __forceinline__ uint32_t spread_hi(uint32_t x) { return (x * 0x02040810u) & 0x10101010u; }

// Sub-block SB (32 columns; 0..7) of one row's 256-column macro-step, from the row's bytes in the
// packed ring, as 16 packed bf16 pairs in column order.
__device__ __forceinline__ void emit4r(uint32_t w, uint32_t mask, uint32_t magic, float a, float nb, uint32_t& o0, uint32_t& o1) {
  const float2 f = hh2ff((w & mask) | magic);
  const float2 g = hh2ff(((w >> 8) & mask) | magic);
  o0 = pack_bf16(fmaf(f.x, a, nb), fmaf(g.x, a, nb));
  o1 = pack_bf16(fmaf(f.y, a, nb), fmaf(g.y, a, nb));
}

// 32 bytes at byte offset off (even, the same for all threads of the CTA) of a row in the packed ring, as eight
// words: three aligned 16-byte loads, then a shift by whole words (four cases, uniform branch) and by a half word.
__device__ __forceinline__ void lds_32_at(uint32_t prow, int off, uint32_t (&q)[8]) {
  uint32_t w[12];
  lds_chunks<3>(prow + (uint32_t)(off & ~15), w);
  const uint32_t hs = (uint32_t)(off & 2) * 8u;
  switch ((off & 15) >> 2) {
    case 0:
#pragma unroll
      for (int i = 0; i < 8; ++i) q[i] = __funnelshift_r(w[i], w[i + 1], hs);
      break;
    case 1:
#pragma unroll
      for (int i = 0; i < 8; ++i) q[i] = __funnelshift_r(w[i + 1], w[i + 2], hs);
      break;
    case 2:
#pragma unroll
      for (int i = 0; i < 8; ++i) q[i] = __funnelshift_r(w[i + 2], w[i + 3], hs);
      break;
    default:
#pragma unroll
      for (int i = 0; i < 8; ++i) q[i] = __funnelshift_r(w[i + 3], w[i + 4], hs);
      break;
  }
}
__device__ __forceinline__ uint32_t lds_u16(uint32_t p) {
  uint32_t v;
  asm volatile("ld.shared.u16 %0, [%1];" : "=r"(v) : "r"(p));
  return v;
}
// Q6_K sub-block sb (32 columns) of the block that starts `lead` bytes into the ring row: the six-bit codes
// c = ql nibble | two qh bits << 4 of columns 4i..4i+3 in the bytes of c[i], the two signed scales (columns 0..15,
// 16..31) and d.  Layout of dequant_q6_k_row (langtax/src/quant.rs): per 128 columns, ql bytes 64n + 32(j & 1) + l
// give nibble j >> 1, qh bytes 32n + l give bits 2j.., scales 8n + 2j + l / 16.
__device__ __forceinline__ void q6k_codes(uint32_t prow, int lead, int sb, uint32_t (&c)[8], float& d, int& s0, int& s1) {
  const int n = sb >> 2, j = sb & 3;
  uint32_t ql[8], qh[8];
  lds_32_at(prow, lead + 64 * n + 32 * (j & 1), ql);
  lds_32_at(prow, lead + 128 + 32 * n, qh);
  const uint32_t sc = lds_u16(prow + (uint32_t)(lead + 192 + 8 * n + 2 * j));
  d = h2f(lds_u16(prow + (uint32_t)(lead + 208)));
  s0 = (int)(int8_t)(sc & 255u);
  s1 = (int)(int8_t)(sc >> 8);
  const int nsh = 4 * (j >> 1), hsh = 2 * j;
#pragma unroll
  for (int i = 0; i < 8; ++i) c[i] = ((ql[i] >> nsh) & 0x0f0f0f0fu) | (((qh[i] >> hsh) & 0x03030303u) << 4);
}

// SB < 0: the sub-block index is the run-time value rsb (formats whose code does not depend on it);
// lead: bytes between the start of the ring row and the block (Q6_K only)
template <int DT, int SB>
__device__ __forceinline__ void dequant_sub(uint32_t prow, uint32_t (&out)[16], int rsb = 0, int lead = 0) {
  if constexpr (DT == DT_Q6_K) {
    uint32_t c[8];
    float d;
    int s0, s1;
    q6k_codes(prow, lead, SB < 0 ? rsb : SB, c, d, s0, s1);
    const float a0 = d * (float)s0, a1 = d * (float)s1;  // w = d * scale * (c - 32), magic 1024: nb = -1056 a
#pragma unroll
    for (int i = 0; i < 4; ++i) emit4<0x00ff00ffu, 0x64006400u>(c[i], a0, -1056.0f * a0, out[2 * i], out[2 * i + 1]);
#pragma unroll
    for (int i = 4; i < 8; ++i) emit4<0x00ff00ffu, 0x64006400u>(c[i], a1, -1056.0f * a1, out[2 * i], out[2 * i + 1]);
  } else if constexpr (DT == DT_Q4_K) {
    // SB enters only through shift counts, masks and an address: one code path for all eight
    // sub-blocks keeps the dequant loop inside the instruction cache.
    const int sb = SB < 0 ? rsb : SB;
    uint32_t hdr[4], q[8];
    lds_chunks<1>(prow, hdr);
    lds_chunks<2>(prow + 16 + 32 * (sb >> 1), q);
    const float d = h2f(hdr[0] & 0xffffu), dmin = h2f(hdr[0] >> 16);
    // get_scale_min_k4: sub-blocks 0..3 use the low six bits of bytes sb / sb+4; 4..7 use a nibble of
    // byte sb+4 plus the top two bits of bytes sb-4 / sb
    const int j = sb & 3, sh = 8 * j;
    const uint32_t b_lo = (hdr[1] >> sh) & 255u, b_mid = (hdr[2] >> sh) & 255u, b_hi = (hdr[3] >> sh) & 255u;
    uint32_t sc, mn;
    if (sb < 4) { sc = b_lo & 63u; mn = b_mid & 63u; }
    else { sc = (b_hi & 15u) | ((b_lo >> 6) << 4); mn = (b_hi >> 4) | ((b_mid >> 6) << 4); }
    const float a = d * (float)sc;
    // low nibbles: 0x6400 | q is binary16 1024 + q; high nibbles in place: 0x5400 | (q << 4) is 64 + q
    const bool hi = sb & 1;
    const uint32_t mask = hi ? 0x00f000f0u : 0x000f000fu, magic = hi ? 0x54005400u : 0x64006400u;
    const float nb = fmaf(hi ? -64.0f : -1024.0f, a, -(dmin * (float)mn));
#pragma unroll
    for (int i = 0; i < 8; ++i) emit4r(q[i], mask, magic, a, nb, out[2 * i], out[2 * i + 1]);
  } else if constexpr (DT == DT_Q5_K) {
    // the Q4_K header, then 32 bytes whose bit sb is the fifth bit of column l of sub-block sb, then the nibbles
    const int sb = SB < 0 ? rsb : SB;
    uint32_t hdr[4], q[8], fh[8];
    lds_chunks<1>(prow, hdr);
    lds_chunks<2>(prow + 16, fh);
    lds_chunks<2>(prow + 48 + 32 * (sb >> 1), q);
    const float d = h2f(hdr[0] & 0xffffu), dmin = h2f(hdr[0] >> 16);
    const int sh = 8 * (sb & 3);
    const uint32_t b_lo = (hdr[1] >> sh) & 255u, b_mid = (hdr[2] >> sh) & 255u, b_hi = (hdr[3] >> sh) & 255u;
    uint32_t sc, mn;
    if (sb < 4) { sc = b_lo & 63u; mn = b_mid & 63u; }
    else { sc = (b_hi & 15u) | ((b_lo >> 6) << 4); mn = (b_hi >> 4) | ((b_mid >> 6) << 4); }
    const float a = d * (float)sc;
    const float nb = fmaf(-1024.0f, a, -(dmin * (float)mn));
    const int nsh = 4 * (sb & 1);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const uint32_t c = ((q[i] >> nsh) & 0x0f0f0f0fu) | (((fh[i] >> sb) & 0x01010101u) << 4);
      emit4<0x00ff00ffu, 0x64006400u>(c, a, nb, out[2 * i], out[2 * i + 1]);
    }
  } else if constexpr (DT == DT_Q4_1) {
    // 20-byte blocks: d, m, sixteen bytes whose low nibbles are columns 0..15 and high nibbles 16..31; w = q d + m
    constexpr int C0 = (20 * SB) / 16, OFF = 20 * SB - 16 * C0, NCH = (OFF + 20 + 15) / 16;
    uint32_t w[4 * NCH + 1];
    {
      uint32_t t[4 * NCH];
      lds_chunks<NCH>(prow + 16 * C0, t);
#pragma unroll
      for (int i = 0; i < 4 * NCH; ++i) w[i] = t[i];
      w[4 * NCH] = 0;
    }
    const float d = h2f(h_at<OFF>(w));
    const float nb = fmaf(-1024.0f, d, h2f(h_at<OFF + 2>(w)));
    auto go = [&](auto I) {
      constexpr int i = decltype(I)::value;
      const uint32_t qs = w_at<OFF + 4 + 4 * i>(w);
      emit4<0x00ff00ffu, 0x64006400u>(qs & 0x0f0f0f0fu, d, nb, out[2 * i], out[2 * i + 1]);
      emit4<0x00ff00ffu, 0x64006400u>((qs >> 4) & 0x0f0f0f0fu, d, nb, out[8 + 2 * i], out[8 + 2 * i + 1]);
    };
    go(std::integral_constant<int, 0>{}); go(std::integral_constant<int, 1>{});
    go(std::integral_constant<int, 2>{}); go(std::integral_constant<int, 3>{});
  } else if constexpr (DT == DT_Q8_0) {
    constexpr int C0 = (34 * SB) / 16, OFF = 34 * SB - 16 * C0;
    uint32_t w[12];
    lds_chunks<3>(prow + 16 * C0, w);
    const float d = h2f(h_at<OFF>(w));
    const float nb = -1152.0f * d;  // byte ^ 0x80 = q + 128, magic adds 1024; exact
    auto go = [&](auto I) {
      constexpr int i = decltype(I)::value;
      emit4<0x00ff00ffu, 0x64806480u>(w_at<OFF + 2 + 4 * i>(w), d, nb, out[2 * i], out[2 * i + 1]);
    };
    go(std::integral_constant<int, 0>{}); go(std::integral_constant<int, 1>{});
    go(std::integral_constant<int, 2>{}); go(std::integral_constant<int, 3>{});
    go(std::integral_constant<int, 4>{}); go(std::integral_constant<int, 5>{});
    go(std::integral_constant<int, 6>{}); go(std::integral_constant<int, 7>{});
  } else if constexpr (DT == DT_Q4_0) {
    // 18-byte blocks: d, then sixteen bytes whose low nibbles are columns 0..15 and high nibbles 16..31; w = (q - 8) d
    constexpr int C0 = (18 * SB) / 16, OFF = 18 * SB - 16 * C0, NCH = (OFF + 18 + 15) / 16;
    uint32_t w[4 * NCH + 1];
    {
      uint32_t t[4 * NCH];
      lds_chunks<NCH>(prow + 16 * C0, t);
#pragma unroll
      for (int i = 0; i < 4 * NCH; ++i) w[i] = t[i];
      w[4 * NCH] = 0;
    }
    const float d = h2f(h_at<OFF>(w));
    const float nb = -1032.0f * d;  // (q - 8) * d with the magic 1024; exact
    auto go = [&](auto I) {
      constexpr int i = decltype(I)::value;
      const uint32_t qs = w_at<OFF + 2 + 4 * i>(w);
      emit4<0x00ff00ffu, 0x64006400u>(qs & 0x0f0f0f0fu, d, nb, out[2 * i], out[2 * i + 1]);
      emit4<0x00ff00ffu, 0x64006400u>((qs >> 4) & 0x0f0f0f0fu, d, nb, out[8 + 2 * i], out[8 + 2 * i + 1]);
    };
    go(std::integral_constant<int, 0>{}); go(std::integral_constant<int, 1>{});
    go(std::integral_constant<int, 2>{}); go(std::integral_constant<int, 3>{});
  } else {
    constexpr int BB = DT == DT_Q5_0 ? 22 : 24, HDR = DT == DT_Q5_0 ? 2 : 4;
    constexpr int C0 = (BB * SB) / 16, OFF = BB * SB - 16 * C0, NCH = (OFF + BB + 15) / 16;
    uint32_t w[4 * NCH + 1];
    {
      uint32_t t[4 * NCH];
      lds_chunks<NCH>(prow + 16 * C0, t);
#pragma unroll
      for (int i = 0; i < 4 * NCH; ++i) w[i] = t[i];
      w[4 * NCH] = 0;
    }
    const float d = h2f(h_at<OFF>(w));
    float nb;
    if constexpr (DT == DT_Q5_0) nb = -1040.0f * d;  // (c - 16) * d with the magic 1024; exact
    else nb = fmaf(-1024.0f, d, h2f(h_at<OFF + 2>(w)));
    const uint32_t qh = w_at<OFF + HDR>(w);
    auto go = [&](auto I) {
      constexpr int i = decltype(I)::value;
      const uint32_t qs = w_at<OFF + HDR + 4 + 4 * i>(w);
      const uint32_t cl = (qs & 0x0f0f0f0fu) | spread_hi((qh >> (4 * i)) & 15u);          // columns 4i .. 4i+3
      const uint32_t ch = ((qs >> 4) & 0x0f0f0f0fu) | spread_hi((qh >> (16 + 4 * i)) & 15u);  // columns 16+4i ..
      emit4<0x00ff00ffu, 0x64006400u>(cl, d, nb, out[2 * i], out[2 * i + 1]);
      emit4<0x00ff00ffu, 0x64006400u>(ch, d, nb, out[8 + 2 * i], out[8 + 2 * i + 1]);
    };
    go(std::integral_constant<int, 0>{}); go(std::integral_constant<int, 1>{});
    go(std::integral_constant<int, 2>{}); go(std::integral_constant<int, 3>{});
  }
}

// ---- binary16 operand path ----------------------------------------------------------------
// Same decoding, but the arithmetic stays in packed binary16: quants are masked into 1024+q (or
// 64+q) pairs, the offset is subtracted exactly, and one HFMA2 applies scale and min to two
// weights.  Under two instructions per weight instead of four to six, and 11 significant bits
// instead of bfloat16's 8.  binary16 has a narrow range: the executor runs this path only for
// matrices whose largest possible |weight| (from the block headers) is between 2^-8 and 30000,
// and activations are rescaled per row by a power of two (undone in the epilogue).
__device__ __forceinline__ uint32_t h2_bits(__half2 v) { return *(const uint32_t*)&v; }
__device__ __forceinline__ __half2 bits_h2(uint32_t v) { return *(const __half2*)&v; }
// bytes b0..b3 of w hold unsigned codes under MASK; out0 = (c0, c1) * a + nb, out1 = (c2, c3) * a + nb
template <uint32_t MASK, uint32_t MAGIC>
__device__ __forceinline__ void emit4h(uint32_t w, __half2 off, __half2 a, __half2 nb, uint32_t& o0, uint32_t& o1) {
  const uint32_t p01 = __byte_perm(w, 0, 0x4140), p23 = __byte_perm(w, 0, 0x4342);  // (b0, b1), (b2, b3) in the low bytes of each half
  const __half2 q01 = __hsub2(bits_h2((p01 & MASK) ^ MAGIC), off), q23 = __hsub2(bits_h2((p23 & MASK) ^ MAGIC), off);
  o0 = h2_bits(__hfma2(q01, a, nb));
  o1 = h2_bits(__hfma2(q23, a, nb));
}

template <int DT, int SB>
__device__ __forceinline__ void dequant_sub_h(uint32_t prow, uint32_t (&out)[16], int rsb = 0, int lead = 0) {
  if constexpr (DT == DT_Q6_K) {
    uint32_t c[8];
    float d;
    int s0, s1;
    q6k_codes(prow, lead, SB < 0 ? rsb : SB, c, d, s0, s1);
    const __half2 a0 = __float2half2_rn(d * (float)s0), a1 = __float2half2_rn(d * (float)s1);
    const __half2 off = __float2half2_rn(1056.f), zero = __float2half2_rn(0.f);
#pragma unroll
    for (int i = 0; i < 4; ++i) emit4h<0x00ff00ffu, 0x64006400u>(c[i], off, a0, zero, out[2 * i], out[2 * i + 1]);
#pragma unroll
    for (int i = 4; i < 8; ++i) emit4h<0x00ff00ffu, 0x64006400u>(c[i], off, a1, zero, out[2 * i], out[2 * i + 1]);
  } else if constexpr (DT == DT_Q4_K) {
    const int sb = SB < 0 ? rsb : SB;
    uint32_t hdr[4], q[8];
    lds_chunks<1>(prow, hdr);
    lds_chunks<2>(prow + 16 + 32 * (sb >> 1), q);
    const float d = h2f(hdr[0] & 0xffffu), dmin = h2f(hdr[0] >> 16);
    const int sh = 8 * (sb & 3);
    const uint32_t b_lo = (hdr[1] >> sh) & 255u, b_mid = (hdr[2] >> sh) & 255u, b_hi = (hdr[3] >> sh) & 255u;
    uint32_t sc, mn;
    if (sb < 4) { sc = b_lo & 63u; mn = b_mid & 63u; }
    else { sc = (b_hi & 15u) | ((b_lo >> 6) << 4); mn = (b_hi >> 4) | ((b_mid >> 6) << 4); }
    const __half2 a = __float2half2_rn(d * (float)sc), nb = __float2half2_rn(-(dmin * (float)mn));
    if (sb & 1) {
#pragma unroll
      for (int i = 0; i < 8; ++i) emit4h<0x00f000f0u, 0x54005400u>(q[i], __float2half2_rn(64.f), a, nb, out[2 * i], out[2 * i + 1]);
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) emit4h<0x000f000fu, 0x64006400u>(q[i], __float2half2_rn(1024.f), a, nb, out[2 * i], out[2 * i + 1]);
    }
  } else if constexpr (DT == DT_Q5_K) {
    const int sb = SB < 0 ? rsb : SB;
    uint32_t hdr[4], q[8], fh[8];
    lds_chunks<1>(prow, hdr);
    lds_chunks<2>(prow + 16, fh);
    lds_chunks<2>(prow + 48 + 32 * (sb >> 1), q);
    const float d = h2f(hdr[0] & 0xffffu), dmin = h2f(hdr[0] >> 16);
    const int sh = 8 * (sb & 3);
    const uint32_t b_lo = (hdr[1] >> sh) & 255u, b_mid = (hdr[2] >> sh) & 255u, b_hi = (hdr[3] >> sh) & 255u;
    uint32_t sc, mn;
    if (sb < 4) { sc = b_lo & 63u; mn = b_mid & 63u; }
    else { sc = (b_hi & 15u) | ((b_lo >> 6) << 4); mn = (b_hi >> 4) | ((b_mid >> 6) << 4); }
    const __half2 a = __float2half2_rn(d * (float)sc), nb = __float2half2_rn(-(dmin * (float)mn));
    const __half2 off = __float2half2_rn(1024.f);
    const int nsh = 4 * (sb & 1);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const uint32_t c = ((q[i] >> nsh) & 0x0f0f0f0fu) | (((fh[i] >> sb) & 0x01010101u) << 4);
      emit4h<0x00ff00ffu, 0x64006400u>(c, off, a, nb, out[2 * i], out[2 * i + 1]);
    }
  } else if constexpr (DT == DT_Q4_1) {
    constexpr int C0 = (20 * SB) / 16, OFF = 20 * SB - 16 * C0, NCH = (OFF + 20 + 15) / 16;
    uint32_t w[4 * NCH + 1];
    {
      uint32_t t[4 * NCH];
      lds_chunks<NCH>(prow + 16 * C0, t);
#pragma unroll
      for (int i = 0; i < 4 * NCH; ++i) w[i] = t[i];
      w[4 * NCH] = 0;
    }
    const uint32_t dh = h_at<OFF>(w), mh = h_at<OFF + 2>(w);
    const __half2 d = bits_h2(dh | (dh << 16)), off = __float2half2_rn(1024.f), nb = bits_h2(mh | (mh << 16));
    auto go = [&](auto I) {
      constexpr int i = decltype(I)::value;
      const uint32_t qs = w_at<OFF + 4 + 4 * i>(w);
      emit4h<0x00ff00ffu, 0x64006400u>(qs & 0x0f0f0f0fu, off, d, nb, out[2 * i], out[2 * i + 1]);
      emit4h<0x00ff00ffu, 0x64006400u>((qs >> 4) & 0x0f0f0f0fu, off, d, nb, out[8 + 2 * i], out[8 + 2 * i + 1]);
    };
    go(std::integral_constant<int, 0>{}); go(std::integral_constant<int, 1>{});
    go(std::integral_constant<int, 2>{}); go(std::integral_constant<int, 3>{});
  } else if constexpr (DT == DT_Q8_0) {
    constexpr int C0 = (34 * SB) / 16, OFF = 34 * SB - 16 * C0;
    uint32_t w[12];
    lds_chunks<3>(prow + 16 * C0, w);
    const uint32_t dh = h_at<OFF>(w);
    const __half2 d = bits_h2(dh | (dh << 16)), off = __float2half2_rn(1152.f), zero = __float2half2_rn(0.f);
    auto go = [&](auto I) {
      constexpr int i = decltype(I)::value;
      emit4h<0x00ff00ffu, 0x64806480u>(w_at<OFF + 2 + 4 * i>(w), off, d, zero, out[2 * i], out[2 * i + 1]);
    };
    go(std::integral_constant<int, 0>{}); go(std::integral_constant<int, 1>{});
    go(std::integral_constant<int, 2>{}); go(std::integral_constant<int, 3>{});
    go(std::integral_constant<int, 4>{}); go(std::integral_constant<int, 5>{});
    go(std::integral_constant<int, 6>{}); go(std::integral_constant<int, 7>{});
  } else if constexpr (DT == DT_Q4_0) {
    constexpr int C0 = (18 * SB) / 16, OFF = 18 * SB - 16 * C0, NCH = (OFF + 18 + 15) / 16;
    uint32_t w[4 * NCH + 1];
    {
      uint32_t t[4 * NCH];
      lds_chunks<NCH>(prow + 16 * C0, t);
#pragma unroll
      for (int i = 0; i < 4 * NCH; ++i) w[i] = t[i];
      w[4 * NCH] = 0;
    }
    const uint32_t dh = h_at<OFF>(w);
    const __half2 d = bits_h2(dh | (dh << 16)), off = __float2half2_rn(1032.f), zero = __float2half2_rn(0.f);
    auto go = [&](auto I) {
      constexpr int i = decltype(I)::value;
      const uint32_t qs = w_at<OFF + 2 + 4 * i>(w);
      emit4h<0x00ff00ffu, 0x64006400u>(qs & 0x0f0f0f0fu, off, d, zero, out[2 * i], out[2 * i + 1]);
      emit4h<0x00ff00ffu, 0x64006400u>((qs >> 4) & 0x0f0f0f0fu, off, d, zero, out[8 + 2 * i], out[8 + 2 * i + 1]);
    };
    go(std::integral_constant<int, 0>{}); go(std::integral_constant<int, 1>{});
    go(std::integral_constant<int, 2>{}); go(std::integral_constant<int, 3>{});
  } else {
    constexpr int BB = DT == DT_Q5_0 ? 22 : 24, HDR = DT == DT_Q5_0 ? 2 : 4;
    constexpr int C0 = (BB * SB) / 16, OFF = BB * SB - 16 * C0, NCH = (OFF + BB + 15) / 16;
    uint32_t w[4 * NCH + 1];
    {
      uint32_t t[4 * NCH];
      lds_chunks<NCH>(prow + 16 * C0, t);
#pragma unroll
      for (int i = 0; i < 4 * NCH; ++i) w[i] = t[i];
      w[4 * NCH] = 0;
    }
    const uint32_t dh = h_at<OFF>(w);
    const __half2 d = bits_h2(dh | (dh << 16));
    __half2 off, nb;
    if constexpr (DT == DT_Q5_0) { off = __float2half2_rn(1040.f); nb = __float2half2_rn(0.f); }
    else { const uint32_t mh = h_at<OFF + 2>(w); off = __float2half2_rn(1024.f); nb = bits_h2(mh | (mh << 16)); }
    const uint32_t qh = w_at<OFF + HDR>(w);
    auto go = [&](auto I) {
      constexpr int i = decltype(I)::value;
      const uint32_t qs = w_at<OFF + HDR + 4 + 4 * i>(w);
      const uint32_t cl = (qs & 0x0f0f0f0fu) | spread_hi((qh >> (4 * i)) & 15u);
      const uint32_t ch = ((qs >> 4) & 0x0f0f0f0fu) | spread_hi((qh >> (16 + 4 * i)) & 15u);
      emit4h<0x00ff00ffu, 0x64006400u>(cl, off, d, nb, out[2 * i], out[2 * i + 1]);
      emit4h<0x00ff00ffu, 0x64006400u>(ch, off, d, nb, out[8 + 2 * i], out[8 + 2 * i + 1]);
    };
    go(std::integral_constant<int, 0>{}); go(std::integral_constant<int, 1>{});
    go(std::integral_constant<int, 2>{}); go(std::integral_constant<int, 3>{});
  }
}

// One 128-row x BN-token tile.  The tensor maps are addressed generically: kernel parameters for a
// single product, an array in global memory for a grouped launch.
template <int DT, int BN, bool F16>
__device__ __forceinline__ void gemm_tc_tile(const CUtensorMap* wmap_p, const CUtensorMap* xmap_p, int rows, int ms_begin,
                                             int ms_count, int tokens, const float* __restrict__ xscale,
                                             float* __restrict__ Y, int row_tile, int tok_tile, int* __restrict__ err) {
  using L = GLay<DT, BN>;
  constexpr int NA = L::NA, NB = L::NB, NPK = L::NPK, NMMA = L::NMMA, PITCH = Pk<DT>::PITCH, RB = Pk<DT>::RB;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);  // swizzle atoms are 1024 bytes
  uint8_t* sB = smem + L::B;
  uint8_t* sP = smem + L::P;
  uint64_t* full_a = (uint64_t*)(smem + L::BAR);
  uint64_t* empty_a = full_a + NA;
  uint64_t* full_b = empty_a + NA;
  uint64_t* empty_b = full_b + NB;
  uint64_t* pk_full = empty_b + NB;
  uint64_t* pk_empty = pk_full + NPK;
  uint64_t* acc_full = pk_empty + NPK;
  uint32_t* tmem_slot = (uint32_t*)(acc_full + 1);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int row0 = row_tile * BM, tok0 = tok_tile * BN;
  const int nms = ms_count, nk = nms * (MACRO / BK);  // this CTA's share of K: macro-steps ms_begin .. ms_begin + nms

  if (tid == 0) {
    for (int s = 0; s < NA; ++s) { bar_init(&full_a[s], DQ_WARPS / 2); bar_init(&empty_a[s], 1); }
    for (int s = 0; s < NB; ++s) { bar_init(&full_b[s], 1); bar_init(&empty_b[s], 1); }
    for (int s = 0; s < NPK; ++s) { bar_init(&pk_full[s], 1); bar_init(&pk_empty[s], DQ_WARPS); }
    bar_init(acc_full, NMMA);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == W_MMA) {  // the MMA warp owns the tensor-memory allocation
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(s32(tmem_slot)), "r"(L::TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem = *tmem_slot;
  bool ok = true;

  if (warp < DQ_WARPS) {
    // ---------------------------------------------------------------- dequant
    // weight row inside the tile, column half of the step, step parity (the last two warp-uniform)
    const int r = tid & 127, h = (tid >> 7) & 1, g = tid >> 8;
    // this thread's A-operand words: lane = row (the warp's lane quarter is warp % 4), 16 columns per half
    const uint32_t a_dst0 = tmem + ((uint32_t)(32 * (warp & 3)) << 16) + (uint32_t)(NMMA * BN + 16 * h);
    int lead = 0;  // Q6_K: where the block starts in the ring row (set per macro-step)
    auto decode = [&](auto KQ, uint32_t prow, uint32_t (&out)[16]) {
      constexpr int kq = decltype(KQ)::value;
      if constexpr (DT == DT_Q6_K) {
        if constexpr (F16) dequant_sub_h<DT, -1>(prow, out, 2 * kq + h, lead);
        else dequant_sub<DT, -1>(prow, out, 2 * kq + h, lead);
      } else if constexpr (F16) {
        if constexpr (DT == DT_Q4_K || DT == DT_Q5_K) dequant_sub_h<DT, -1>(prow, out, 2 * kq + h);
        else if (h == 0) dequant_sub_h<DT, 2 * kq>(prow, out);
        else dequant_sub_h<DT, 2 * kq + 1>(prow, out);
      } else {
        if constexpr (DT == DT_Q4_K || DT == DT_Q5_K) dequant_sub<DT, -1>(prow, out, 2 * kq + h);
        else if (h == 0) dequant_sub<DT, 2 * kq>(prow, out);
        else dequant_sub<DT, 2 * kq + 1>(prow, out);
      }
    };
    auto put = [&](const uint32_t (&out)[16], int s) {
      asm volatile(
          "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
          ::"r"(a_dst0 + (uint32_t)(s * L::A_COLS)), "r"(out[0]), "r"(out[1]), "r"(out[2]), "r"(out[3]), "r"(out[4]), "r"(out[5]),
            "r"(out[6]), "r"(out[7]), "r"(out[8]), "r"(out[9]), "r"(out[10]), "r"(out[11]), "r"(out[12]), "r"(out[13]),
            "r"(out[14]), "r"(out[15]) : "memory");
    };
    // Per macro-step a warp decodes both of its 64-column steps (g and g + 2) back to back: two
    // independent instruction streams for the scheduler, and one round of barrier waits, tensor
    // memory store completion and arrivals for two steps instead of one each.
    static_assert(NA % 2 == 0 && NA >= 4, "a group's two steps of a macro-step use different stages");
    for (int ms = 0; ms < nms; ++ms) {
      const int ps = ms % NPK;
      if (ok && !bar_wait(&pk_full[ps], (uint32_t)((ms / NPK) & 1))) { ok = false; report_error(err, 3); }
      const uint32_t prow = s32(sP) + ps * L::P_STAGE + r * PITCH;
      if constexpr (DT == DT_Q6_K) lead = ((ms_begin + ms) * RB) & 15;
      uint32_t o0[16], o1[16];
      if (g == 0) {
        decode(std::integral_constant<int, 0>{}, prow, o0);
        decode(std::integral_constant<int, 2>{}, prow, o1);
      } else {
        decode(std::integral_constant<int, 1>{}, prow, o0);
        decode(std::integral_constant<int, 3>{}, prow, o1);
      }
      __syncwarp();
      if (lane == 0) bar_arrive(&pk_empty[ps]);  // the packed bytes are in registers now
      const int ks0 = 4 * ms + g, ks1 = ks0 + 2, s0 = ks0 % NA, s1 = ks1 % NA;
      if (ok && !bar_wait2(&empty_a[s0], (uint32_t)(((ks0 / NA) & 1) ^ 1), &empty_a[s1], (uint32_t)(((ks1 / NA) & 1) ^ 1))) {
        ok = false;
        report_error(err, 3);
      }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      put(o0, s0);
      put(o1, s1);
      asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) { bar_arrive(&full_a[s0]); bar_arrive(&full_a[s1]); }
    }
    // --------------------------------------------------------------- epilogue
    if (warp < 8) {
    asm volatile("griddepcontrol.wait;" ::: "memory");  // row scales from the conversion kernel; y may still be read by an earlier kernel
    if (ok && !bar_wait(acc_full, 0)) { ok = false; report_error(err, 3); }
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const int q = warp & 3, half = warp >> 2;  // TMEM lane quarter of this warp, column half
    const int out_row = row0 + 32 * q + lane;
    constexpr int CPW = BN / 2;  // columns per warp
#pragma unroll 1
    for (int c0 = half * CPW; c0 < (half + 1) * CPW; c0 += 16) {
      float acc[16];
#pragma unroll
      for (int a = 0; a < NMMA; ++a) {
        uint32_t v[16];
        const uint32_t taddr = tmem + ((uint32_t)(32 * q) << 16) + (uint32_t)(a * BN + c0);
        asm volatile(
            "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
            : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
              "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
            : "r"(taddr) : "memory");
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
        for (int j = 0; j < 16; ++j) acc[j] = a == 0 ? __uint_as_float(v[j]) : acc[j] + __uint_as_float(v[j]);
      }
      if (out_row < rows) {
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const int tok = tok0 + c0 + j;
          if (tok < tokens) {
            float r = acc[j];
            if constexpr (F16) r *= __ldg(xscale + tok);  // undo the activation row's power-of-two scale
            Y[(int64_t)tok * rows + out_row] = r;
          }
        }
      }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    }
  } else if (warp == W_PACKED) {
    // ------------------------------------- packed weight bytes (one 2-D TMA box per macro-step)
    if (lane == 0) {
      for (int ms = 0; ms < nms; ++ms) {
        const int ps = ms % NPK;
        if (ok && !bar_wait(&pk_empty[ps], (uint32_t)(((ms / NPK) & 1) ^ 1))) { ok = false; report_error(err, 3); }
        bar_expect(&pk_full[ps], BM * PITCH);
        // x in 32-bit elements; x*4 = ms*RB rounded down to a multiple of 16 bytes (only Q6_K's 210 needs the
        // rounding).  Rows past the end and words past a row's end read as zero.
        asm volatile(
            "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
            ::"r"(s32(sP + ps * L::P_STAGE)), "l"(wmap_p), "r"((((ms_begin + ms) * RB) & ~15) / 4), "r"(row0), "r"(s32(&pk_full[ps])) : "memory");
      }
    }
  } else if (warp == W_ACT) {
    // ---------------------------------------------------- activation tiles (TMA)
    // the warp walks the ring converged (uniform registers for the addresses), one elected lane issues
    const uint32_t sb_u = __shfl_sync(0xffffffffu, s32(sB), 0);
    asm volatile("griddepcontrol.wait;" ::: "memory");  // the activations are the conversion kernel's output
    for (int ks = 0; ks < nk; ++ks) {
      const int s = ks % NB;
      if (ok && !bar_wait(&empty_b[s], (uint32_t)(((ks / NB) & 1) ^ 1))) { ok = false; report_error(err, 3); }
      if (elect_one()) {
        bar_expect(&full_b[s], BN * 128);
        asm volatile(
            "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
            ::"r"(sb_u + (uint32_t)(s * L::B_STAGE)), "l"(xmap_p), "r"((ms_begin * (MACRO / BK) + ks) * BK), "r"(tok0), "r"(s32(&full_b[s])) : "memory");
      }
      __syncwarp();
    }
  } else {
    // ------------------------------------------------------------------- MMA
    // The whole warp walks the loop converged and one elected lane issues: addresses, descriptors
    // and the loop state then live in uniform registers, which is what the MMA instruction reads.
    // A loop entered by a single lane pays a vector-to-uniform move per operand instead and
    // becomes the bottleneck of the CTA at small BN.
    constexpr uint32_t idesc = instr_desc<BN, F16>();
    const int mw = warp - W_MMA;  // which MMA warp: 64-column steps mw, mw + NMMA, ... into accumulator mw
    if (mw < NMMA) {
      const uint32_t tmem_u = __shfl_sync(0xffffffffu, tmem, 0);
      const uint32_t sb_u = __shfl_sync(0xffffffffu, s32(sB), 0);
      const uint32_t td = tmem_u + (uint32_t)(mw * BN);
      for (int ks = mw; ks < nk; ks += NMMA) {  // nk is a multiple of 4
        const int sa = ks % NA, sb = ks % NB;
        if (ok && !bar_wait2(&full_a[sa], (uint32_t)((ks / NA) & 1), &full_b[sb], (uint32_t)((ks / NB) & 1))) {
          ok = false;
          report_error(err, 3);
        }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if (elect_one()) {
          const uint32_t ta = tmem_u + (uint32_t)(NMMA * BN + sa * L::A_COLS);
          const uint64_t db = smem_desc_u(sb_u + (uint32_t)(sb * L::B_STAGE));
#pragma unroll
          for (int kk = 0; kk < BK / 16; ++kk) {
            // 16 values along K: eight 32-bit columns of A; 32 bytes inside B's swizzled row = 2 x 16-byte units
            if (kk == 0 && ks == mw)
              asm volatile("{ .reg .pred p; setp.ne.b32 p, 0, 0; tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p; }"
                           ::"r"(td), "r"(ta), "l"(db), "r"(idesc) : "memory");
            else
              asm volatile("{ .reg .pred p; setp.eq.b32 p, 0, 0; tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p; }"
                           ::"r"(td), "r"(ta + 8 * kk), "l"(db + 2 * kk), "r"(idesc) : "memory");
          }
          // free both stages once the MMAs that read them have completed
          asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(s32(&empty_a[sa])) : "memory");
          asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(s32(&empty_b[sb])) : "memory");
        }
        __syncwarp();
      }
      if (elect_one())
        asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(s32(acc_full)) : "memory");
      __syncwarp();
    }
  }
  __syncthreads();
  if (warp == W_MMA) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(L::TMEM_COLS) : "memory");
  }
}

template <int DT, int BN, bool F16>
__global__ void __launch_bounds__(TC_THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap wmap, int rows, int cols, int tokens,
               const __grid_constant__ CUtensorMap xmap, const float* __restrict__ xscale, float* __restrict__ Y,
               int* __restrict__ err) {
  // split-K: gridDim.z CTAs share a tile's K range; slice z writes its partial sums to Y + z * tokens * rows
  // (with one slice Y is the result itself), and a second kernel adds the slices in order
  const int per = cols / MACRO / (int)gridDim.z;
  gemm_tc_tile<DT, BN, F16>(&wmap, &xmap, rows, (int)blockIdx.z * per, per, tokens, xscale,
                            Y + (size_t)blockIdx.z * (size_t)tokens * (size_t)rows, (int)blockIdx.x, (int)blockIdx.y, err);
}

__global__ void add_slices_kernel(const float* __restrict__ part, float* __restrict__ y, int64_t n, int slices) {
  asm volatile("griddepcontrol.wait;" ::: "memory");
  for (int64_t i = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * 4; i < n; i += (int64_t)gridDim.x * blockDim.x * 4) {
    float4 acc = *(const float4*)(part + i);
    for (int z = 1; z < slices; ++z) {  // ascending slice order: the result does not depend on scheduling
      const float4 v = *(const float4*)(part + (int64_t)z * n + i);
      acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    *(float4*)(y + i) = acc;
  }
}

// Grouped launch (routed experts, decode.rs:10006 grouped_routed_ffn): the tiles of several
// products in one grid.  groups[] lies in global memory; a CTA finds its product by its tile number.
template <int DT, int BN, bool F16>
__global__ void __launch_bounds__(TC_THREADS, 1)
gemm_tc_grouped_kernel(const GemmGroup* __restrict__ groups, int n_groups, int* __restrict__ err) {
  const int tile = (int)blockIdx.x;
  int g = 0;
  while (g + 1 < n_groups && tile >= groups[g + 1].tile_begin) ++g;
  const GemmGroup* G = groups + g;
  const int local = tile - G->tile_begin, row_tiles = (G->rows + BM - 1) / BM;
  gemm_tc_tile<DT, BN, F16>(&G->wmap, &G->xmap, G->rows, 0, G->cols / MACRO, G->tokens, G->xscale, G->y, local % row_tiles,
                            local / row_tiles, err);
}

__global__ void to_bf16_kernel(const float* __restrict__ x, __nv_bfloat16* __restrict__ o, int64_t n) {
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  for (int64_t i = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * 4; i < n; i += (int64_t)gridDim.x * blockDim.x * 4) {
    if (i + 3 < n) {
      const float4 v = *(const float4*)(x + i);
      const __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
      *(uint2*)(o + i) = make_uint2(*(const uint32_t*)&a, *(const uint32_t*)&b);
    } else {
      for (int64_t j = i; j < n; ++j) o[j] = __float2bfloat16_rn(x[j]);
    }
  }
}

// binary16 activations: one CTA per activation row.  The row is multiplied by the power of two that
// puts its largest magnitude into [2^14, 2^15) (binary16 tops out at 65504), and the inverse goes
// to inv_scale[row] for the epilogue.  A zero or non-finite row is left unscaled.
__global__ void to_f16_rows_kernel(const float* __restrict__ x, __half* __restrict__ o, float* __restrict__ inv_scale, int cols) {
  __shared__ float wmax[8];
  asm volatile("griddepcontrol.wait;" ::: "memory");               // x may come from the kernel before
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");  // the GEMM may start its weight pipeline
  const float* xr = x + (int64_t)blockIdx.x * cols;
  __half* orow = o + (int64_t)blockIdx.x * cols;
  float m = 0.f;
  for (int i = threadIdx.x * 4; i < cols; i += blockDim.x * 4) {
    const float4 v = *(const float4*)(xr + i);
    m = fmaxf(fmaxf(m, fmaxf(fabsf(v.x), fabsf(v.y))), fmaxf(fabsf(v.z), fabsf(v.w)));
  }
#pragma unroll
  for (int o2 = 16; o2; o2 >>= 1) m = fmaxf(m, __shfl_xor_sync(~0u, m, o2));
  if ((threadIdx.x & 31) == 0) wmax[threadIdx.x >> 5] = m;
  __syncthreads();
  m = wmax[0];
#pragma unroll
  for (int w = 1; w < 8; ++w) m = fmaxf(m, wmax[w]);
  const int be = (int)((__float_as_uint(m) >> 23) & 0xff);
  float s = 1.f, sinv = 1.f;
  if (be != 0 && be != 255) {  // normal and finite: exponent of the scale = 14 - (be - 127), kept in the normal range
    int e = 14 - (be - 127);
    e = e > 126 ? 126 : (e < -126 ? -126 : e);
    s = __uint_as_float((uint32_t)(e + 127) << 23);
    sinv = __uint_as_float((uint32_t)(127 - e) << 23);
  }
  if (threadIdx.x == 0) inv_scale[blockIdx.x] = sinv;
  for (int i = threadIdx.x * 4; i < cols; i += blockDim.x * 4) {
    const float4 v = *(const float4*)(xr + i);
    const __half2 a = __floats2half2_rn(v.x * s, v.y * s), b = __floats2half2_rn(v.z * s, v.w * s);
    *(uint2*)(orow + i) = make_uint2(*(const uint32_t*)&a, *(const uint32_t*)&b);
  }
}

// Routed-expert layer: the 16-bit operand rows of the gate / up products gathered straight from the
// layer's activations, one CTA per packed row: row r is read from row src_row[r] of x (the gather
// of the rows routed to an expert, decode.rs:10062) and no packed f32 copy is made.  F16: per-row
// power-of-two scaling as in to_f16_rows_kernel; otherwise bfloat16 without scaling.
// (silu(g) * u was tried in here as well: with one CTA per row it took longer than the two
// separate element-wise kernels.)
template <bool F16>
__global__ void expert_rows_16bit_kernel(const float* __restrict__ x, const int* __restrict__ src_row,
                                         void* __restrict__ o, float* __restrict__ inv_scale, int cols) {
  __shared__ float wmax[8];
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const int64_t r = blockIdx.x;
  const float* xr = x + (int64_t)src_row[r] * cols;
  float s = 1.f;
  if (F16) {
    float m = 0.f;
    for (int i = threadIdx.x * 4; i < cols; i += blockDim.x * 4) {
      const float4 v = *(const float4*)(xr + i);
      m = fmaxf(fmaxf(m, fmaxf(fabsf(v.x), fabsf(v.y))), fmaxf(fabsf(v.z), fabsf(v.w)));
    }
#pragma unroll
    for (int o2 = 16; o2; o2 >>= 1) m = fmaxf(m, __shfl_xor_sync(~0u, m, o2));
    if ((threadIdx.x & 31) == 0) wmax[threadIdx.x >> 5] = m;
    __syncthreads();
    m = wmax[0];
#pragma unroll
    for (int w = 1; w < 8; ++w) m = fmaxf(m, wmax[w]);
    const int be = (int)((__float_as_uint(m) >> 23) & 0xff);
    float sinv = 1.f;
    if (be != 0 && be != 255) {
      int e = 14 - (be - 127);
      e = e > 126 ? 126 : (e < -126 ? -126 : e);
      s = __uint_as_float((uint32_t)(e + 127) << 23);
      sinv = __uint_as_float((uint32_t)(127 - e) << 23);
    }
    if (threadIdx.x == 0) inv_scale[r] = sinv;
  }
  for (int i = threadIdx.x * 4; i < cols; i += blockDim.x * 4) {
    const float4 v = *(const float4*)(xr + i);
    uint2 packed;
    if (F16) {
      const __half2 a = __floats2half2_rn(v.x * s, v.y * s), b = __floats2half2_rn(v.z * s, v.w * s);
      packed = make_uint2(*(const uint32_t*)&a, *(const uint32_t*)&b);
    } else {
      const __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
      packed = make_uint2(*(const uint32_t*)&a, *(const uint32_t*)&b);
    }
    *(uint2*)((uint16_t*)o + r * cols + i) = packed;
  }
}

// Largest |weight| any block of the matrix can decode to, from the block headers alone, as the bit
// pattern of a non-negative float (so that an integer max orders it); NaN or infinite headers give
// 0x7f800000 or more.
template <int DT>
__global__ void weight_bound_kernel(const uint8_t* __restrict__ W, int64_t n_blocks, unsigned int* __restrict__ out) {
  constexpr int BB = DT == DT_Q4_K ? 144 : DT == DT_Q5_K ? 176 : DT == DT_Q6_K ? 210 : DT == DT_Q8_0 ? 34 : DT == DT_Q5_0 ? 22
                     : DT == DT_Q4_0 ? 18 : DT == DT_Q4_1 ? 20 : 24;
  float m = 0.f;
  for (int64_t b = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; b < n_blocks; b += (int64_t)gridDim.x * blockDim.x) {
    const uint16_t* hp = (const uint16_t*)(W + b * BB);
    const float d = fabsf(__half2float(__ushort_as_half(hp[DT == DT_Q6_K ? 104 : 0])));  // Q6_K keeps d behind the quants
    float bound;
    if (DT == DT_Q6_K) bound = d * (128.f * 32.f);  // |scale| <= 128, |c - 32| <= 32
    else if (DT == DT_Q4_K) bound = d * (63.f * 15.f) + fabsf(__half2float(__ushort_as_half(hp[1]))) * 63.f;
    else if (DT == DT_Q5_K) bound = d * (63.f * 31.f) + fabsf(__half2float(__ushort_as_half(hp[1]))) * 63.f;
    else if (DT == DT_Q4_1) bound = d * 15.f + fabsf(__half2float(__ushort_as_half(hp[1])));
    else if (DT == DT_Q8_0) bound = d * 128.f;
    else if (DT == DT_Q5_0) bound = d * 16.f;
    else if (DT == DT_Q4_0) bound = d * 8.f;
    else bound = d * 31.f + fabsf(__half2float(__ushort_as_half(hp[1])));
    if (!(bound <= 3.4028234e38f)) bound = __uint_as_float(0x7f800000u);
    m = fmaxf(m, bound);
  }
#pragma unroll
  for (int o2 = 16; o2; o2 >>= 1) m = fmaxf(m, __shfl_xor_sync(~0u, m, o2));
  if ((threadIdx.x & 31) == 0) atomicMax(out, __float_as_uint(m));
}

inline EncodeTiledFn encode_fn() { return tensor_map_encoder(); }

template <int DT, int BN, bool F16>
cudaError_t launch_bn(const MatView& m, const CUtensorMap& wmap, const CUtensorMap& xmap, const float* xscale, float* y,
                      int tokens, int splits, cudaStream_t stream, int* err) {
  auto kern = gemm_tc_kernel<DT, BN, F16>;
  constexpr int smem = GLay<DT, BN>::TOTAL;
  static PerDevice ready;  // per instantiation
  std::atomic<int>& slot = ready.here();
  if (slot.load(std::memory_order_relaxed) == 0) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return e;
    slot.store(1, std::memory_order_relaxed);
  }
  // Programmatic dependent launch: the packed-weight pipeline and the dequantization start while the
  // conversion kernel before it is still running; what depends on that kernel waits inside.
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr.val.programmaticStreamSerializationAllowed = 1;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)((m.rows + BM - 1) / BM), (unsigned)((tokens + BN - 1) / BN), (unsigned)splits);
  cfg.blockDim = dim3(TC_THREADS);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cfg.attrs = &attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kern, wmap, (int)m.rows, (int)m.cols, tokens, xmap, xscale, y, err);
}

template <int DT, bool F16>
cudaError_t launch_dt(const MatView& m, const void* xb, const float* xscale, float* y, int tokens, int splits,
                      cudaStream_t stream, int* err) {
  EncodeTiledFn enc = encode_fn();
  if (!enc) return cudaErrorNotSupported;
  const int bn = tokens > 128 ? 256 : tokens > 64 ? 128 : 64;
  CUtensorMap xmap;
  const cuuint64_t dims[2] = {(cuuint64_t)m.cols, (cuuint64_t)tokens};
  const cuuint64_t strides[1] = {(cuuint64_t)m.cols * 2};
  const cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)bn};
  const cuuint32_t estr[2] = {1, 1};
  if (enc(&xmap, F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (void*)xb, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
          CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return cudaErrorInvalidValue;
  // packed weights as rows of 32-bit words; one box = 128 rows x the ring pitch
  CUtensorMap wmap;
  const cuuint64_t wdims[2] = {(cuuint64_t)(m.row_bytes / 4), (cuuint64_t)m.rows};
  const cuuint64_t wstrides[1] = {(cuuint64_t)m.row_bytes};
  const cuuint32_t wbox[2] = {(cuuint32_t)(Pk<DT>::PITCH / 4), (cuuint32_t)BM};
  if (enc(&wmap, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, (void*)m.w, wdims, wstrides, wbox, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
          CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return cudaErrorInvalidValue;
  if (bn == 256) return launch_bn<DT, 256, F16>(m, wmap, xmap, xscale, y, tokens, splits, stream, err);
  if (bn == 128) return launch_bn<DT, 128, F16>(m, wmap, xmap, xscale, y, tokens, splits, stream, err);
  return launch_bn<DT, 64, F16>(m, wmap, xmap, xscale, y, tokens, splits, stream, err);
}

}  // namespace

bool gemm_tc_supported(const MatView& m, int64_t tokens) {
  if (m.dtype != DT_Q4_K && m.dtype != DT_Q6_K && m.dtype != DT_Q8_0 && m.dtype != DT_Q5_0 && m.dtype != DT_Q5_1 && m.dtype != DT_Q4_0 &&
      m.dtype != DT_Q4_1 && m.dtype != DT_Q5_K)
    return false;
  if (m.dtype == DT_Q6_K && m.cols % 2048 != 0) return false;  // the tensor map wants rows a multiple of 16 bytes apart: 8 x 210
  if (tokens < 16 || tokens > (1 << 24) || m.rows <= 0 || m.rows > (1 << 30)) return false;
  if (m.cols % MACRO != 0 || m.cols <= 0 || m.cols > (1 << 30)) return false;
  return ((uintptr_t)m.w & 15) == 0;
}

// Split-K: a shape with few 128-row tiles and a long K (ffn_down: 32 tiles of 224 steps) would leave
// most SMs idle.  The K range is cut into the largest power of two of slices that keeps the grid within
// one wave of the 148 SMs and every slice at least 1024 columns long and a whole number of macro-steps.
int gemm_tc_splits(const MatView& m, int64_t tokens) {
  const int bn = tokens > 128 ? 256 : tokens > 64 ? 128 : 64;
  const int64_t tiles = ((m.rows + BM - 1) / BM) * ((tokens + bn - 1) / bn);
  const int64_t nms = m.cols / MACRO;
  int s = 1;
  while (s < 8 && tiles * (s * 2) <= 148 && nms % (s * 2) == 0 && nms / (s * 2) >= 4) s *= 2;
  return s;
}

// 16-bit activations, one f32 scale per activation row (binary16 path), split-K partial sums
static size_t tc_x16_bytes(const MatView& m, int64_t tokens) { return ((size_t)tokens * (size_t)m.cols * 2 + 255) / 256 * 256; }
static size_t tc_scale_bytes(int64_t tokens) { return ((size_t)tokens * 4 + 255) / 256 * 256; }
size_t gemm_tc_scratch_bytes(const MatView& m, int64_t tokens) {
  const int s = gemm_tc_splits(m, tokens);
  return tc_x16_bytes(m, tokens) + tc_scale_bytes(tokens) + (s > 1 ? (size_t)s * (size_t)tokens * (size_t)m.rows * 4 : 0);
}

cudaError_t launch_weight_bound(const MatView& m, unsigned int* out_dev, cudaStream_t stream, uint64_t* launches) {
  const int64_t nb = m.rows * (m.cols / (m.dtype == DT_Q4_K || m.dtype == DT_Q6_K || m.dtype == DT_Q5_K ? 256 : 32));
  int64_t blocks = (nb + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  cudaError_t e = cudaMemsetAsync(out_dev, 0, sizeof(unsigned int), stream);
  if (e != cudaSuccess) return e;
  switch (m.dtype) {
    case DT_Q4_K: weight_bound_kernel<DT_Q4_K><<<(unsigned)blocks, 256, 0, stream>>>(m.w, nb, out_dev); break;
    case DT_Q6_K: weight_bound_kernel<DT_Q6_K><<<(unsigned)blocks, 256, 0, stream>>>(m.w, nb, out_dev); break;
    case DT_Q8_0: weight_bound_kernel<DT_Q8_0><<<(unsigned)blocks, 256, 0, stream>>>(m.w, nb, out_dev); break;
    case DT_Q5_0: weight_bound_kernel<DT_Q5_0><<<(unsigned)blocks, 256, 0, stream>>>(m.w, nb, out_dev); break;
    case DT_Q4_0: weight_bound_kernel<DT_Q4_0><<<(unsigned)blocks, 256, 0, stream>>>(m.w, nb, out_dev); break;
    case DT_Q5_1: weight_bound_kernel<DT_Q5_1><<<(unsigned)blocks, 256, 0, stream>>>(m.w, nb, out_dev); break;
    case DT_Q4_1: weight_bound_kernel<DT_Q4_1><<<(unsigned)blocks, 256, 0, stream>>>(m.w, nb, out_dev); break;
    case DT_Q5_K: weight_bound_kernel<DT_Q5_K><<<(unsigned)blocks, 256, 0, stream>>>(m.w, nb, out_dev); break;
    default: return cudaErrorInvalidValue;
  }
  if (launches) ++*launches;
  return cudaGetLastError();
}

bool weight_bound_allows_f16(unsigned int bound_bits) {
  float b;
  static_assert(sizeof(b) == sizeof(bound_bits), "float bits");
  memcpy(&b, &bound_bits, sizeof(b));
  return bound_bits < 0x7f800000u && b < 30000.f && b > 1.f / 256.f;
}

cudaError_t launch_gemm_tc(const MatView& m, const float* x, float* y, int64_t tokens, void* scratch, size_t scratch_bytes,
                           cudaStream_t stream, int* err_flag, uint64_t* launches) {
  const int64_t n = tokens * m.cols;
  const bool f16 = m.f16_ok == 1;
  float* xscale = (float*)((char*)scratch + tc_x16_bytes(m, tokens));
  float* part = (float*)((char*)xscale + tc_scale_bytes(tokens));
  int splits = gemm_tc_splits(m, tokens);
  if (scratch_bytes < gemm_tc_scratch_bytes(m, tokens)) splits = 1;  // a fixed-size staging area may not hold the slices
  if (((uintptr_t)y & 15) != 0 || (tokens * m.rows) % 4 != 0) splits = 1;  // the slice adder works on aligned float4
  if (f16) {
    to_f16_rows_kernel<<<(unsigned)tokens, 256, 0, stream>>>(x, (__half*)scratch, xscale, (int)m.cols);
  } else {
    int64_t blocks = (n / 4 + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    if (blocks < 1) blocks = 1;
    to_bf16_kernel<<<(unsigned)blocks, 256, 0, stream>>>(x, (__nv_bfloat16*)scratch, n);
  }
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  if (launches) ++*launches;
  float* dst = splits > 1 ? part : y;
#define LLR_TC(D) (f16 ? launch_dt<D, true>(m, scratch, xscale, dst, (int)tokens, splits, stream, err_flag) \
                       : launch_dt<D, false>(m, scratch, nullptr, dst, (int)tokens, splits, stream, err_flag))
  switch (m.dtype) {
    case DT_Q4_K: e = LLR_TC(DT_Q4_K); break;
    case DT_Q6_K: e = LLR_TC(DT_Q6_K); break;
    case DT_Q8_0: e = LLR_TC(DT_Q8_0); break;
    case DT_Q5_0: e = LLR_TC(DT_Q5_0); break;
    case DT_Q4_0: e = LLR_TC(DT_Q4_0); break;
    case DT_Q5_1: e = LLR_TC(DT_Q5_1); break;
    case DT_Q4_1: e = LLR_TC(DT_Q4_1); break;
    case DT_Q5_K: e = LLR_TC(DT_Q5_K); break;
    default: return cudaErrorInvalidValue;
  }
#undef LLR_TC
  if (e != cudaSuccess) return e;
  if (launches) ++*launches;
  if (splits > 1) {
    const int64_t ny = tokens * m.rows;
    int64_t blocks = (ny / 4 + 255) / 256;
    if (blocks > 148 * 8) blocks = 148 * 8;
    add_slices_kernel<<<(unsigned)blocks, 256, 0, stream>>>(part, y, ny, splits);
    e = cudaGetLastError();
    if (e == cudaSuccess && launches) ++*launches;
  }
  return e;
}

// ---- grouped launch --------------------------------------------------------------------
namespace {
template <int DT>
bool encode_maps(const MatView& m, const void* x16, int tokens, int bn, bool f16, CUtensorMap* wmap, CUtensorMap* xmap) {
  EncodeTiledFn enc = encode_fn();
  if (!enc) return false;
  const cuuint64_t dims[2] = {(cuuint64_t)m.cols, (cuuint64_t)tokens};
  const cuuint64_t strides[1] = {(cuuint64_t)m.cols * 2};
  const cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)bn};
  const cuuint32_t estr[2] = {1, 1};
  if (enc(xmap, f16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (void*)x16, dims, strides, box, estr,
          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return false;
  const cuuint64_t wdims[2] = {(cuuint64_t)(m.row_bytes / 4), (cuuint64_t)m.rows};
  const cuuint64_t wstrides[1] = {(cuuint64_t)m.row_bytes};
  const cuuint32_t wbox[2] = {(cuuint32_t)(Pk<DT>::PITCH / 4), (cuuint32_t)BM};
  return enc(wmap, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, (void*)m.w, wdims, wstrides, wbox, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
             CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int DT, int BN, bool F16>
cudaError_t launch_grouped_bn(const GemmGroup* desc_dev, int n_groups, int tiles, cudaStream_t stream, int* err) {
  auto kern = gemm_tc_grouped_kernel<DT, BN, F16>;
  constexpr int smem = GLay<DT, BN>::TOTAL;
  static PerDevice ready;  // per instantiation
  std::atomic<int>& slot = ready.here();
  if (slot.load(std::memory_order_relaxed) == 0) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return e;
    slot.store(1, std::memory_order_relaxed);
  }
  kern<<<(unsigned)tiles, TC_THREADS, smem, stream>>>(desc_dev, n_groups, err);
  return cudaGetLastError();
}

template <int DT>
cudaError_t launch_grouped_dt(const GemmGroupSpec* specs, int n, bool f16, void* desc_dev, cudaStream_t stream, int* err) {
  int max_tokens = 0;
  for (int i = 0; i < n; ++i) max_tokens = specs[i].tokens > max_tokens ? specs[i].tokens : max_tokens;
  // the narrowest tile that holds the busiest product's rows: the MMA and activation-tile work of a
  // tile grows with its width, padding included (512 tokens over 8 experts, top-2: 113-144 rows each)
  const int bn = max_tokens > 192 ? 256 : max_tokens > 160 ? 192 : max_tokens > 128 ? 160 : max_tokens > 64 ? 128 : 64;
  std::vector<GemmGroup> host((size_t)n);
  int tiles = 0;
  for (int i = 0; i < n; ++i) {
    const GemmGroupSpec& sp = specs[i];
    GemmGroup& g = host[(size_t)i];
    if (!encode_maps<DT>(sp.m, sp.x16, sp.tokens, bn, f16, &g.wmap, &g.xmap)) return cudaErrorInvalidValue;
    g.xscale = sp.xscale;
    g.y = sp.y;
    g.rows = (int)sp.m.rows;
    g.cols = (int)sp.m.cols;
    g.tokens = sp.tokens;
    g.tile_begin = tiles;
    tiles += (int)((sp.m.rows + BM - 1) / BM) * ((sp.tokens + bn - 1) / bn);
  }
  // pageable source: the copy is staged before this call returns, so `host` may go out of scope
  cudaError_t e = cudaMemcpyAsync(desc_dev, host.data(), host.size() * sizeof(GemmGroup), cudaMemcpyHostToDevice, stream);
  if (e != cudaSuccess) return e;
  const GemmGroup* d = (const GemmGroup*)desc_dev;
#define LLR_GROUPED(B) (f16 ? launch_grouped_bn<DT, B, true>(d, n, tiles, stream, err) : launch_grouped_bn<DT, B, false>(d, n, tiles, stream, err))
  if (bn == 256) return LLR_GROUPED(256);
  if (bn == 192) return LLR_GROUPED(192);
  if (bn == 160) return LLR_GROUPED(160);
  if (bn == 128) return LLR_GROUPED(128);
  return LLR_GROUPED(64);
#undef LLR_GROUPED
}
}  // namespace

size_t gemm_tc_group_desc_bytes(int n_groups) { return (size_t)n_groups * sizeof(GemmGroup); }

cudaError_t tc_convert_activations(const float* x, int64_t n_rows, int cols, bool f16, void* out16, float* xscale,
                                   cudaStream_t stream, uint64_t* launches) {
  if (f16) {
    to_f16_rows_kernel<<<(unsigned)n_rows, 256, 0, stream>>>(x, (__half*)out16, xscale, cols);
  } else {
    const int64_t n = n_rows * cols;
    int64_t blocks = (n / 4 + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    if (blocks < 1) blocks = 1;
    to_bf16_kernel<<<(unsigned)blocks, 256, 0, stream>>>(x, (__nv_bfloat16*)out16, n);
  }
  if (launches) ++*launches;
  return cudaGetLastError();
}

cudaError_t tc_convert_expert_rows(const float* x, const int* src_row, int64_t n_rows, int cols, bool f16,
                                   void* out16, float* xscale, cudaStream_t stream, uint64_t* launches) {
  if (n_rows <= 0) return cudaSuccess;
  if (f16) expert_rows_16bit_kernel<true><<<(unsigned)n_rows, 256, 0, stream>>>(x, src_row, out16, xscale, cols);
  else expert_rows_16bit_kernel<false><<<(unsigned)n_rows, 256, 0, stream>>>(x, src_row, out16, xscale, cols);
  if (launches) ++*launches;
  return cudaGetLastError();
}

cudaError_t launch_gemm_tc_grouped(const GemmGroupSpec* specs, int n, bool f16, void* desc_dev, cudaStream_t stream,
                                   int* err_flag, uint64_t* launches) {
  if (n <= 0 || ((uintptr_t)desc_dev & 63) != 0) return cudaErrorInvalidValue;
  for (int i = 0; i < n; ++i)
    if (specs[i].m.dtype != specs[0].m.dtype || specs[i].tokens < 1 || !gemm_tc_supported(specs[i].m, 16)) return cudaErrorInvalidValue;
  cudaError_t e;
  switch (specs[0].m.dtype) {
    case DT_Q4_K: e = launch_grouped_dt<DT_Q4_K>(specs, n, f16, desc_dev, stream, err_flag); break;
    case DT_Q6_K: e = launch_grouped_dt<DT_Q6_K>(specs, n, f16, desc_dev, stream, err_flag); break;
    case DT_Q8_0: e = launch_grouped_dt<DT_Q8_0>(specs, n, f16, desc_dev, stream, err_flag); break;
    case DT_Q5_0: e = launch_grouped_dt<DT_Q5_0>(specs, n, f16, desc_dev, stream, err_flag); break;
    case DT_Q4_0: e = launch_grouped_dt<DT_Q4_0>(specs, n, f16, desc_dev, stream, err_flag); break;
    case DT_Q5_1: e = launch_grouped_dt<DT_Q5_1>(specs, n, f16, desc_dev, stream, err_flag); break;
    case DT_Q4_1: e = launch_grouped_dt<DT_Q4_1>(specs, n, f16, desc_dev, stream, err_flag); break;
    case DT_Q5_K: e = launch_grouped_dt<DT_Q5_K>(specs, n, f16, desc_dev, stream, err_flag); break;
    default: return cudaErrorInvalidValue;
  }
  if (e == cudaSuccess && launches) ++*launches;
  return e;
}

// ---- allocation-free variant ---------------------------------------------------------
// The bf16 activation staging of the GEMM normally lives in a buffer the executor grows on
// demand.  This variant uses a fixed array that is part of the library image instead, so the
// call path contains no allocation at all.  Every GPU that loads the library holds these
// bytes until the process exits.
// the stated limit applies to the 16-bit activations; the per-row scales of the binary16 path (at most
// 256 KB for shapes within the limit) lie behind them
static __device__ __align__(256) unsigned char g_static_scratch[GEMM_STATIC_SCRATCH_BYTES + (512 << 10)];

size_t gemm_tc_static_scratch_limit() { return GEMM_STATIC_SCRATCH_BYTES; }

cudaError_t launch_gemm_tc_static(int device, const MatView& m, const float* x, float* y, int64_t tokens,
                                  cudaStream_t stream, int* err_flag, uint64_t* launches) {
  // In host code `g_static_scratch` is only a handle for the symbol, not a device address:
  // the address is looked up once per device, with that device current.
  // Executors on different threads may make their first call at the same time: the slot is atomic, and
  // two threads that both look the address up store the same value.
  static std::atomic<void*> addr[64];
  if (device < 0 || device >= 64) return cudaErrorInvalidDevice;
  void* p = addr[device].load(std::memory_order_acquire);
  if (!p) {
    const cudaError_t e = cudaGetSymbolAddress(&p, g_static_scratch);
    if (e != cudaSuccess) return e;
    addr[device].store(p, std::memory_order_release);
  }
  return launch_gemm_tc(m, x, y, tokens, p, GEMM_STATIC_SCRATCH_BYTES + (512 << 10), stream, err_flag, launches);
}

}  // namespace llr
