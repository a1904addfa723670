// Decode GEMV (1..8 activation rows per pass) for Q4_K, Q6_K and Q8_0 on the
// integer tensor cores, fed by TMA bulk copies.
//
// What it computes: gemv_<t>_f32 / gemm_<t>_f32 of langtax/src/quant.rs
// (:6214, :6891, :7199 and the gemm twins), i.e. y[t][r] = sum_c W[r,c] x[t][c]
// with W given as packed GGUF blocks that are never expanded.
//
// How: a CTA owns a contiguous range of 16-row tiles.  One elected thread
// streams each tile's packed bytes HBM -> shared memory with cp.async.bulk (one
// copy per row so rows land on a padded, bank-conflict-free stride), two chunks
// in flight per CTA, completion on mbarriers with bounded waits.  The
// activations of a 4096-column span are split ONCE per CTA into four signed
// base-128 digits per value (x * 2^e rounded to a 28-bit integer, e chosen per
// 256-column block so the block maximum fills the range), stored as int8 planes
// that are exactly the B fragments of mma.sync.m16n8k32.s8 (two activation rows
// x four digits = the eight columns of one n-tile).  The quants go from shared
// memory straight into A fragments: a Q4_K nibble word needs one AND (low
// nibbles) or a shift+AND (high), a Q8_0 word nothing at all, a Q6_K word two
// LOP3 and a sign fix.  The integer dot products are exact; sub-block scales
// are folded in with integer multiply-adds (Q4_K: 6-bit scales, Q6_K: int8
// scales per 16) and only once per super-block / block does the sum become a
// float and meet the binary16 block scale.  Q4_K mins use the float sums of x
// per 32 columns.  Warps split the columns of a chunk, partial sums meet in
// shared memory in a fixed order, so results are bit-reproducible run to run.
//
// Numerics: the integer part is exact; the activation split keeps 28 bits below
// each 256-block's maximum (an element that small next to a large one loses
// relative, not absolute, precision: its error is 1/16 of the f32 rounding the
// reference applies to the block's largest term).  The result differs from the
// f64 dot of the f32-dequantized weights only by (a) those 2^-28 terms, (b) the
// f32 rounding of each dequantized weight that the reference's kernels bake in
// and this kernel does not, (c) one f32 rounding per block when summing.
//
// Launch protocol: kernels are launched with programmatic stream serialization.
// Each CTA signals griddepcontrol.launch_dependents at once, prefetches its
// first weight chunks (weights never depend on earlier kernels), and only then
// executes griddepcontrol.wait before it reads activations or writes results,
// so consecutive decode GEMVs overlap launch latency and weight prefetch with
// the tail of their predecessor.
#include "llr_formats.cuh"
#include "llr_kernels.cuh"

namespace llr {
namespace {

constexpr int NWARP = 8;
constexpr int NST = 2;          // chunks in flight per CTA
constexpr int SPAN = 4096;      // columns whose digit planes live in shared memory
constexpr int DS = SPAN + 32;   // digit plane stride: 32 mod 128 -> conflict-free 8-byte reads
constexpr int SPIN_LIMIT = 1 << 22;

template <int DT> struct Fmt;
template <> struct Fmt<DT_Q4_K> { static constexpr int KSEG = 4096, BB = 144, BE = 256; };
template <> struct Fmt<DT_Q6_K> { static constexpr int KSEG = 2048, BB = 210, BE = 256; };
template <> struct Fmt<DT_Q8_0> { static constexpr int KSEG = 2048, BB = 34, BE = 32; };

template <int DT, int MT> struct Lay {
  using F = Fmt<DT>;
  static constexpr int NT = (MT + 1) / 2;                       // n-tiles of 2 activation rows
  static constexpr int SEGB = F::KSEG / F::BE * F::BB;          // bytes of one row segment
  // row stride mod 128: 32 spreads the 8-byte fragment reads of eight rows over all banks,
  // 16 does the same for the 4-byte reads of Q6_K
  static constexpr int RMOD = DT == DT_Q6_K ? 16 : 32;
  static constexpr int RS = SEGB + (RMOD + 128 - SEGB % 128) % 128;
  static constexpr int CHUNK = 16 * RS;
  static constexpr int RING = 0;
  static constexpr int DIG = RING + NST * CHUNK;                // int8 [NT*8][DS]
  static constexpr int SXF = DIG + NT * 8 * DS;                 // float [MT][SPAN/32]
  static constexpr int XSI = SXF + MT * (SPAN / 32) * 4;        // float [MT][SPAN/256]
  static constexpr int RED = XSI + MT * (SPAN / 256) * 4;       // float [2][NWARP][16][MT]
  static constexpr int BAR = RED + 2 * NWARP * 16 * MT * 4;     // uint64 [NST]
  static constexpr int TOTAL = BAR + NST * 8 + 16;
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
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mma_k32(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                        uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
               : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
}
__device__ __forceinline__ void mma_k16(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t b0) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%7,%7,%7,%7};"
               : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
               : "r"(a0), "r"(a1), "r"(b0), "r"(0));
}
__device__ __forceinline__ float h2f(uint32_t h) { return __half2float(__ushort_as_half((unsigned short)h)); }

// four bytes at p (p is 2-byte aligned; `odd` says p % 4 == 2)
__device__ __forceinline__ uint32_t lds32_a2(const uint8_t* p, bool odd) {
  if (!odd) return *(const uint32_t*)p;
  const uint32_t lo = *(const uint32_t*)(p - 2), hi = *(const uint32_t*)(p + 2);
  return __funnelshift_r(lo, hi, 16);
}
// eight bytes at p, same alignment rule
__device__ __forceinline__ uint2 lds64_a2(const uint8_t* p, bool odd) {
  if (!odd) return make_uint2(*(const uint32_t*)p, *(const uint32_t*)(p + 4));
  const uint32_t x0 = *(const uint32_t*)(p - 2), x1 = *(const uint32_t*)(p + 2), x2 = *(const uint32_t*)(p + 6);
  return make_uint2(__funnelshift_r(x0, x1, 16), __funnelshift_r(x1, x2, 16));
}
// per byte: 6-bit code c (0..63) -> int8 (c - 32); no carries cross bytes
__device__ __forceinline__ uint32_t recentre6(uint32_t c) {
  return ((c | 0x80808080u) - 0x20202020u) ^ 0x80808080u;
}

// Per-thread accumulators of one chunk: yacc[nt][0..1] row g, [2..3] row g+8,
// columns 2t, 2t+1 of n-tile nt; ymin only for Q4_K.
template <int DT, int MT> struct Acc {
  static constexpr int NT = (MT + 1) / 2;
  float y[NT][4];
  float mn[2][MT];
};

// One Q4_K super-block (256 columns) of rows g and g+8 against every n-tile.
template <int MT>
__device__ __forceinline__ void block_q4k(const uint8_t* rowA, const uint8_t* rowB, int b, int cb,
                                          const uint8_t* dig, const float* sxf, const float* xsi,
                                          int g, int t, Acc<DT_Q4_K, MT>& acc) {
  constexpr int NT = (MT + 1) / 2;
  const uint4 hA = *(const uint4*)(rowA + b * 144), hB = *(const uint4*)(rowB + b * 144);
  // 6-bit scales and mins packed four to a word: bytes 0..3 = sub-blocks 0..3 (word 0), 4..7 (word 1)
  const uint32_t scA0 = hA.y & 0x3f3f3f3fu, scA1 = (hA.w & 0x0f0f0f0fu) | ((hA.y >> 2) & 0x30303030u);
  const uint32_t scB0 = hB.y & 0x3f3f3f3fu, scB1 = (hB.w & 0x0f0f0f0fu) | ((hB.y >> 2) & 0x30303030u);
  int T[NT][4];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt)
#pragma unroll
    for (int i = 0; i < 4; ++i) T[nt][i] = 0;
#pragma unroll
  for (int G = 0; G < 4; ++G) {
    const uint2 wA = *(const uint2*)(rowA + b * 144 + 16 + G * 32 + 8 * t);
    const uint2 wB = *(const uint2*)(rowB + b * 144 + 16 + G * 32 + 8 * t);
    constexpr uint32_t M4 = 0x0f0f0f0fu;
    const uint32_t scAp = G < 2 ? scA0 : scA1, scBp = G < 2 ? scB0 : scB1;
    const int sAlo = (scAp >> (16 * (G & 1))) & 255, sAhi = (scAp >> (16 * (G & 1) + 8)) & 255;
    const int sBlo = (scBp >> (16 * (G & 1))) & 255, sBhi = (scBp >> (16 * (G & 1) + 8)) & 255;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      const uint8_t* dp = dig + (size_t)(nt * 8 + g) * DS + cb * 256 + G * 64 + 8 * t;
      const uint2 blo = *(const uint2*)dp, bhi = *(const uint2*)(dp + 32);
      int clo[4], chi[4];
      mma_k32(clo, wA.x & M4, wB.x & M4, wA.y & M4, wB.y & M4, blo.x, blo.y);
      mma_k32(chi, (wA.x >> 4) & M4, (wB.x >> 4) & M4, (wA.y >> 4) & M4, (wB.y >> 4) & M4, bhi.x, bhi.y);
      T[nt][0] += sAlo * clo[0] + sAhi * chi[0];
      T[nt][1] += sAlo * clo[1] + sAhi * chi[1];
      T[nt][2] += sBlo * clo[2] + sBhi * chi[2];
      T[nt][3] += sBlo * clo[3] + sBhi * chi[3];
    }
  }
  const float dA = h2f(hA.x & 0xffffu), dminA = h2f(hA.x >> 16);
  const float dB = h2f(hB.x & 0xffffu), dminB = h2f(hB.x >> 16);
  // columns 2t, 2t+1 of an n-tile are activation row (t >> 1), digits 2(t&1) and 2(t&1)+1
  const float pw0 = (t & 1) ? 16384.f : 1.f, pw1 = pw0 * 128.f;
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    const int tok = 2 * nt + (t >> 1);
    const float xs = tok < MT ? xsi[tok * (SPAN / 256) + cb] : 0.f;
    acc.y[nt][0] = fmaf((float)T[nt][0], dA * xs * pw0, acc.y[nt][0]);
    acc.y[nt][1] = fmaf((float)T[nt][1], dA * xs * pw1, acc.y[nt][1]);
    acc.y[nt][2] = fmaf((float)T[nt][2], dB * xs * pw0, acc.y[nt][2]);
    acc.y[nt][3] = fmaf((float)T[nt][3], dB * xs * pw1, acc.y[nt][3]);
  }
  // mins: this thread covers sub-blocks 2t, 2t+1 of both rows
  const uint32_t mnA = t < 2 ? (hA.z & 0x3f3f3f3fu) : (((hA.w >> 4) & 0x0f0f0f0fu) | ((hA.z >> 2) & 0x30303030u));
  const uint32_t mnB = t < 2 ? (hB.z & 0x3f3f3f3fu) : (((hB.w >> 4) & 0x0f0f0f0fu) | ((hB.z >> 2) & 0x30303030u));
  const float a0 = dminA * (float)((mnA >> (16 * (t & 1))) & 255), a1 = dminA * (float)((mnA >> (16 * (t & 1) + 8)) & 255);
  const float b0 = dminB * (float)((mnB >> (16 * (t & 1))) & 255), b1 = dminB * (float)((mnB >> (16 * (t & 1) + 8)) & 255);
#pragma unroll
  for (int k = 0; k < MT; ++k) {
    const float s0 = sxf[k * (SPAN / 32) + cb * 8 + 2 * t], s1 = sxf[k * (SPAN / 32) + cb * 8 + 2 * t + 1];
    acc.mn[0][k] = fmaf(a0, s0, fmaf(a1, s1, acc.mn[0][k]));
    acc.mn[1][k] = fmaf(b0, s0, fmaf(b1, s1, acc.mn[1][k]));
  }
}

// One Q6_K super-block: 16 scale groups of 16 columns, one m16n8k16 each.
template <int MT>
__device__ __forceinline__ void block_q6k(const uint8_t* rowA, const uint8_t* rowB, int b, int cb,
                                          const uint8_t* dig, const float* xsi, int g, int t,
                                          Acc<DT_Q6_K, MT>& acc) {
  constexpr int NT = (MT + 1) / 2;
  const uint8_t* pA = rowA + b * 210;
  const uint8_t* pB = rowB + b * 210;
  const bool odd = (b & 1) != 0;  // 210 b mod 4 is 2 for odd b (row segments start 16-byte aligned)
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
      const uint32_t qlA0 = lds32_a2(pA + half * 64 + l, odd), qlA1 = lds32_a2(pA + half * 64 + 32 + l, odd);
      const uint32_t qhA = lds32_a2(pA + 128 + half * 32 + l, odd);
      const uint32_t qlB0 = lds32_a2(pB + half * 64 + l, odd), qlB1 = lds32_a2(pB + half * 64 + 32 + l, odd);
      const uint32_t qhB = lds32_a2(pB + 128 + half * 32 + l, odd);
      constexpr uint32_t M4 = 0x0f0f0f0fu, M2 = 0x03030303u;
#pragma unroll
      for (int qtr = 0; qtr < 4; ++qtr) {
        const uint32_t lA = (qtr & 1) ? qlA1 : qlA0, lB = (qtr & 1) ? qlB1 : qlB0;
        const uint32_t cA = recentre6((((qtr & 2) ? (lA >> 4) : lA) & M4) | (((qhA >> (2 * qtr)) & M2) << 4));
        const uint32_t cB = recentre6((((qtr & 2) ? (lB >> 4) : lB) & M4) | (((qhB >> (2 * qtr)) & M2) << 4));
        const int sidx = 192 + half * 8 + hg + 2 * qtr;
        const int sA = (int)(int8_t)pA[sidx], sB = (int)(int8_t)pB[sidx];
        const int col = cb * 256 + half * 128 + qtr * 32 + l;  // first of this thread's 4 columns
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          const uint32_t bd = *(const uint32_t*)(dig + (size_t)(nt * 8 + g) * DS + col);
          int c[4];
          mma_k16(c, cA, cB, bd);
          T[nt][0] += sA * c[0]; T[nt][1] += sA * c[1];
          T[nt][2] += sB * c[2]; T[nt][3] += sB * c[3];
        }
      }
    }
  }
  const float dA = h2f(pA[208] | (pA[209] << 8)), dB = h2f(pB[208] | (pB[209] << 8));
  const float pw0 = (t & 1) ? 16384.f : 1.f, pw1 = pw0 * 128.f;
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    const int tok = 2 * nt + (t >> 1);
    const float xs = tok < MT ? xsi[tok * (SPAN / 256) + cb] : 0.f;
    acc.y[nt][0] = fmaf((float)T[nt][0], dA * xs * pw0, acc.y[nt][0]);
    acc.y[nt][1] = fmaf((float)T[nt][1], dA * xs * pw1, acc.y[nt][1]);
    acc.y[nt][2] = fmaf((float)T[nt][2], dB * xs * pw0, acc.y[nt][2]);
    acc.y[nt][3] = fmaf((float)T[nt][3], dB * xs * pw1, acc.y[nt][3]);
  }
}

// One Q8_0 block (32 columns): the int8 quants are the A fragment as they lie.
template <int MT>
__device__ __forceinline__ void block_q80(const uint8_t* rowA, const uint8_t* rowB, int b, int c32,
                                          const uint8_t* dig, const float* xsi, int g, int t,
                                          Acc<DT_Q8_0, MT>& acc) {
  constexpr int NT = (MT + 1) / 2;
  const uint8_t* pA = rowA + b * 34;
  const uint8_t* pB = rowB + b * 34;
  const bool odd = (b & 1) == 0;  // quants start at 34 b + 2: 4-byte aligned for odd b only
  const uint2 wA = lds64_a2(pA + 2 + 8 * t, odd), wB = lds64_a2(pB + 2 + 8 * t, odd);
  const float dA = h2f(*(const uint16_t*)pA), dB = h2f(*(const uint16_t*)pB);
  const float pw0 = (t & 1) ? 16384.f : 1.f, pw1 = pw0 * 128.f;
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    const uint2 bd = *(const uint2*)(dig + (size_t)(nt * 8 + g) * DS + c32 * 32 + 8 * t);
    int c[4];
    mma_k32(c, wA.x, wB.x, wA.y, wB.y, bd.x, bd.y);
    const int tok = 2 * nt + (t >> 1);
    const float xs = tok < MT ? xsi[tok * (SPAN / 256) + (c32 >> 3)] : 0.f;
    acc.y[nt][0] = fmaf((float)c[0], dA * xs * pw0, acc.y[nt][0]);
    acc.y[nt][1] = fmaf((float)c[1], dA * xs * pw1, acc.y[nt][1]);
    acc.y[nt][2] = fmaf((float)c[2], dB * xs * pw0, acc.y[nt][2]);
    acc.y[nt][3] = fmaf((float)c[3], dB * xs * pw1, acc.y[nt][3]);
  }
}

template <int DT, int MT>
__global__ void __launch_bounds__(NWARP * 32, 1)
gemv_mma_kernel(const uint8_t* __restrict__ W, int64_t row_bytes, int rows, int cols,
                const float* __restrict__ X, float* __restrict__ Y, int tokens, int* __restrict__ err) {
  using L = Lay<DT, MT>;
  using F = Fmt<DT>;
  constexpr int NT = L::NT, SEGB = L::SEGB, RS = L::RS, CHUNK = L::CHUNK, KSEG = F::KSEG;
  constexpr int SUBS = SPAN / KSEG;  // chunks per tile per span
  extern __shared__ __align__(128) uint8_t smem[];
  uint8_t* ring = smem + L::RING;
  uint8_t* dig = smem + L::DIG;
  float* sxf = (float*)(smem + L::SXF);
  float* xsi = (float*)(smem + L::XSI);
  float* red = (float*)(smem + L::RED);
  uint64_t* bars = (uint64_t*)(smem + L::BAR);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;

  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  const int n_tiles = (rows + 15) / 16;
  const int n_span = (cols + SPAN - 1) / SPAN;
  const int base = n_tiles / gridDim.x, extra = n_tiles % gridDim.x;
  const int tile0 = blockIdx.x * base + min((int)blockIdx.x, extra);
  const int my_tiles = base + ((int)blockIdx.x < extra ? 1 : 0);
  // chunk order: span-major, then tile, then the KSEG pieces of the span
  auto subs_of = [&](int span) { return min(SUBS, (min(SPAN, cols - span * SPAN) + KSEG - 1) / KSEG); };
  int n_chunks = 0;
  for (int s = 0; s < n_span; ++s) n_chunks += my_tiles * subs_of(s);

  if (tid == 0) {
    for (int s = 0; s < NST; ++s) mbar_init(&bars[s], 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();

  // producer state (thread 0 only): the next chunk to request
  int p_span = 0, p_tile = 0, p_sub = 0, p_idx = 0;
  auto issue_next = [&]() {
    if (p_idx >= n_chunks) return;
    const int stage = p_idx % NST;
    const int64_t seg_off = ((int64_t)p_span * SUBS + p_sub) * SEGB;
    const int64_t left = row_bytes - seg_off;
    const uint32_t bytes = (uint32_t)(left < SEGB ? left : SEGB);
    mbar_expect_tx(&bars[stage], 16 * bytes);
    for (int r = 0; r < 16; ++r) {
      int row = (tile0 + p_tile) * 16 + r;
      if (row >= rows) row = rows - 1;  // tail tile: refetch a valid row, never written back
      bulk_g2s(ring + stage * CHUNK + r * RS, W + (int64_t)row * row_bytes + seg_off, bytes, &bars[stage]);
    }
    ++p_idx;
    if (++p_sub == subs_of(p_span)) { p_sub = 0; if (++p_tile == my_tiles) { p_tile = 0; ++p_span; } }
  };
  if (tid == 0) for (int i = 0; i < NST; ++i) issue_next();

  // unused activation-row columns of the n-tiles must read as zero
  for (int i = tid; i < NT * 8 * DS / 16; i += blockDim.x) ((uint4*)dig)[i] = make_uint4(0, 0, 0, 0);

  // everything above touches weights only; activations and results wait for the predecessor
  asm volatile("griddepcontrol.wait;" ::: "memory");

  int c = 0;
  for (int span = 0; span < n_span; ++span) {
    const int span_cols = min(SPAN, cols - span * SPAN), nblk256 = span_cols >> 8;
    __syncthreads();
    // ---- activations of this span -> four int8 digit planes per activation row ----
    for (int job = warp; job < nblk256 * tokens; job += NWARP) {
      const int b = job % nblk256, tok = job / nblk256;
      const float4* xp = (const float4*)(X + (int64_t)tok * cols + span * SPAN + b * 256 + 8 * lane);
      const float4 va = __ldg(xp), vb = __ldg(xp + 1);
      const float v[8] = {va.x, va.y, va.z, va.w, vb.x, vb.y, vb.z, vb.w};
      float m = 0.f, sum = 0.f;
#pragma unroll
      for (int j = 0; j < 8; ++j) { m = fmaxf(m, fabsf(v[j])); sum += v[j]; }
      bool bad = false;
#pragma unroll
      for (int j = 0; j < 8; ++j) bad = bad || !(fabsf(v[j]) <= 3.4028234e38f);
#pragma unroll
      for (int o = 16; o; o >>= 1) m = fmaxf(m, __shfl_xor_sync(~0u, m, o));
      bad = __any_sync(~0u, bad);
      sum += __shfl_xor_sync(~0u, sum, 1);
      sum += __shfl_xor_sync(~0u, sum, 2);
      const int be = (int)((__float_as_uint(m) >> 23) & 0xff);
      float s = 0.f, sinv = 0.f;  // an all-zero (or denormal) block contributes nothing
      if (be != 0 && !bad) {
        int e = 26 - (be - 127);
        e = e > 126 ? 126 : e;
        s = __uint_as_float((uint32_t)(e + 127) << 23);
        sinv = __uint_as_float((uint32_t)(127 - e) << 23);
      }
      uint32_t pk[4][2] = {{0, 0}, {0, 0}, {0, 0}, {0, 0}};
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        int xi = bad ? 0 : __float2int_rn(v[j] * s);
#pragma unroll
        for (int p = 0; p < 4; ++p) {
          const int d = p < 3 ? (((xi + 64) & 127) - 64) : xi;
          xi = (xi - d) >> 7;
          pk[p][j >> 2] |= (uint32_t)(d & 255) << (8 * (j & 3));
        }
      }
      const int nt = tok >> 1, plane0 = (tok & 1) * 4;
#pragma unroll
      for (int p = 0; p < 4; ++p)
        *(uint2*)(dig + (size_t)(nt * 8 + plane0 + p) * DS + b * 256 + 8 * lane) = make_uint2(pk[p][0], pk[p][1]);
      if ((lane & 3) == 0) sxf[tok * (SPAN / 32) + b * 8 + (lane >> 2)] = sum;
      // a non-finite activation makes the whole output row of that token NaN
      if (lane == 0) xsi[tok * (SPAN / 256) + b] = bad ? __uint_as_float(0x7fc00000u) : sinv;
    }
    __syncthreads();

    const int nsub = subs_of(span);
    for (int tl = 0; tl < my_tiles; ++tl) {
      const int tile = tile0 + tl;
      Acc<DT, MT> acc;
#pragma unroll
      for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc.y[nt][i] = 0.f;
#pragma unroll
      for (int k = 0; k < MT; ++k) acc.mn[0][k] = acc.mn[1][k] = 0.f;

      for (int sub = 0; sub < nsub; ++sub, ++c) {
        const int stage = c % NST;
        {
          const uint32_t parity = (uint32_t)((c / NST) & 1);
          int spins = 0;
          bool ok = true;
          while (!mbar_try_wait(&bars[stage], parity)) {
            if (++spins > SPIN_LIMIT) { ok = false; break; }
          }
          if (!ok && lane == 0) atomicExch(err, 1);  // keep going: every warp must reach the barriers
        }
        const uint8_t* chunk = ring + stage * CHUNK;
        const uint8_t* rowA = chunk + g * RS;
        const uint8_t* rowB = chunk + (g + 8) * RS;
        const int seg_cols = min(KSEG, span_cols - sub * KSEG);
        if constexpr (DT == DT_Q4_K) {
          for (int b = warp; b < (seg_cols >> 8); b += NWARP)
            block_q4k<MT>(rowA, rowB, b, sub * (KSEG / 256) + b, dig, sxf, xsi, g, t, acc);
        } else if constexpr (DT == DT_Q6_K) {
          for (int b = warp; b < (seg_cols >> 8); b += NWARP)
            block_q6k<MT>(rowA, rowB, b, sub * (KSEG / 256) + b, dig, xsi, g, t, acc);
        } else {
          for (int b = warp; b < (seg_cols >> 5); b += NWARP)
            block_q80<MT>(rowA, rowB, b, sub * (KSEG / 32) + b, dig, xsi, g, t, acc);
        }
        if (sub + 1 < nsub) {
          __syncthreads();  // the stage is free: refill it
          if (tid == 0) issue_next();
        }
      }
      // ---- combine inside the warp and publish this tile's partial sums ----
      const int rb = tl & 1;
      float* myred = red + (rb * NWARP + warp) * 16 * MT;
      if constexpr (DT == DT_Q4_K) {
#pragma unroll
        for (int k = 0; k < MT; ++k)
#pragma unroll
          for (int r = 0; r < 2; ++r) {
            float v = acc.mn[r][k];
            v += __shfl_xor_sync(~0u, v, 1);
            v += __shfl_xor_sync(~0u, v, 2);
            acc.mn[r][k] = v;
          }
      }
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        float vA = acc.y[nt][0] + acc.y[nt][1], vB = acc.y[nt][2] + acc.y[nt][3];
        vA += __shfl_xor_sync(~0u, vA, 1);
        vB += __shfl_xor_sync(~0u, vB, 1);
        const int tok = 2 * nt + (t >> 1);
        if ((t & 1) == 0 && tok < MT) {
          float mA = 0.f, mB = 0.f;
          if constexpr (DT == DT_Q4_K) {
#pragma unroll
            for (int k = 0; k < MT; ++k)
              if (k == tok) { mA = acc.mn[0][k]; mB = acc.mn[1][k]; }
          }
          myred[g * MT + tok] = vA - mA;
          myred[(g + 8) * MT + tok] = vB - mB;
        }
      }
      __syncthreads();
      if (tid == 0) issue_next();
      if (tid < 16 * MT) {
        const int r = tid / MT, k = tid % MT, row = tile * 16 + r;
        if (row < rows && k < tokens) {
          float v = 0.f;
          const float* rp = red + rb * NWARP * 16 * MT + r * MT + k;
#pragma unroll
          for (int w = 0; w < NWARP; ++w) v += rp[w * 16 * MT];
          float* yp = Y + (int64_t)k * rows + row;
          *yp = span == 0 ? v : *yp + v;
        }
      }
    }
  }
}

template <int DT, int MT>
cudaError_t launch_one(const MatView& m, const float* x, float* y, int tokens, cudaStream_t stream,
                       int sm_count, int* err) {
  auto kern = gemv_mma_kernel<DT, MT>;
  constexpr int smem = Lay<DT, MT>::TOTAL;
  static int blocks_per_sm = 0;  // per instantiation
  if (blocks_per_sm == 0) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return e;
    int n = 0;
    e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kern, NWARP * 32, smem);
    if (e != cudaSuccess) return e;
    blocks_per_sm = n > 0 ? n : 1;
  }
  const int n_tiles = (int)((m.rows + 15) / 16);
  int grid = sm_count * blocks_per_sm;
  if (grid > n_tiles) grid = n_tiles;
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr.val.programmaticStreamSerializationAllowed = 1;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)grid);
  cfg.blockDim = dim3(NWARP * 32);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cfg.attrs = &attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kern, m.w, m.row_bytes, (int)m.rows, (int)m.cols, x, y, tokens, err);
}

template <int DT>
cudaError_t launch_mt(const MatView& m, const float* x, float* y, int tokens, cudaStream_t stream,
                      int sm_count, int* err) {
  if (tokens == 1) return launch_one<DT, 1>(m, x, y, tokens, stream, sm_count, err);
  if (tokens == 2) return launch_one<DT, 2>(m, x, y, tokens, stream, sm_count, err);
  if (tokens <= 4) return launch_one<DT, 4>(m, x, y, tokens, stream, sm_count, err);
  return launch_one<DT, 8>(m, x, y, tokens, stream, sm_count, err);
}

}  // namespace

bool gemv_mma_supported(const MatView& m) {
  if (m.dtype != DT_Q4_K && m.dtype != DT_Q6_K && m.dtype != DT_Q8_0) return false;
  if (m.rows <= 0 || m.cols <= 0 || m.rows > (1 << 30) || m.cols > (1 << 30)) return false;
  if (((uintptr_t)m.w & 15) != 0 || m.row_bytes % 16 != 0) return false;
  if (m.cols % 256 != 0) return false;
  // every KSEG piece of a row must start and end on a 16-byte boundary
  if (m.dtype == DT_Q6_K && m.cols % 2048 != 0) return false;
  return true;
}

cudaError_t launch_gemv_mma(const MatView& m, const float* x, float* y, int64_t tokens,
                            cudaStream_t stream, int sm_count, int* err, uint64_t* launches) {
  for (int64_t t0 = 0; t0 < tokens; t0 += 8) {
    const int nt = (int)(tokens - t0 < 8 ? tokens - t0 : 8);
    const float* xp = x + t0 * m.cols;
    float* yp = y + t0 * m.rows;
    cudaError_t e;
    switch (m.dtype) {
      case DT_Q4_K: e = launch_mt<DT_Q4_K>(m, xp, yp, nt, stream, sm_count, err); break;
      case DT_Q6_K: e = launch_mt<DT_Q6_K>(m, xp, yp, nt, stream, sm_count, err); break;
      case DT_Q8_0: e = launch_mt<DT_Q8_0>(m, xp, yp, nt, stream, sm_count, err); break;
      default: return cudaErrorInvalidValue;
    }
    if (e != cudaSuccess) return e;
    if (launches) ++*launches;
  }
  return cudaSuccess;
}

}  // namespace llr
