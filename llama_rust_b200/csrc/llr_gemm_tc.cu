// Chunk GEMM for many activation rows (prefill / continuous-batching chunks):
// packed GGUF weights are dequantized tile by tile into shared memory and fed to
// the 5th-generation tensor cores (tcgen05.mma, accumulators in tensor memory).
//
// What it computes: gemm_<t>_f32 (langtax/src/quant.rs:6282, 6366, 6380, 6478 ->
// gemm_f32_x :6760), y[t*rows + r] = sum_c W[r,c] x[t*cols + c], for Q4_K, Q8_0,
// Q5_0 and Q5_1.  Operands are rounded to bfloat16 (weights after exact f32
// dequantization, activations once up front), products are exact, accumulation is
// f32 in tensor memory: this is the tensor-core path with the looser, separately
// stated tolerance (tests/test_gpu_gemm.py); the f32-faithful path for any number
// of rows stays the integer kernel of llr_gemv_stream.cu.
//
// One CTA computes a 128-row x BN-token tile of y over the whole K.  Per 64-column
// step: eight warps dequantize 128 x 64 weights (two threads per row, packed bytes
// straight from global memory, the next four steps prefetched in registers) into a K-major
// 128-byte-swizzled bf16 tile; one thread TMA-loads the matching BN x 64 bf16
// activation tile (2-D tensor map, 128-byte swizzle, out-of-range tokens read as
// zero); one thread issues four tcgen05.mma (M=128, N=BN, K=16) whose commit
// releases the stage.  Four stages are in flight; all hand-offs are mbarriers
// with bounded waits.  The epilogue reads the accumulators with tcgen05.ld (one
// TMEM lane = one weight row per thread) and stores token-major, coalesced.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "llr_formats.cuh"
#include "llr_kernels.cuh"

namespace llr {
namespace {

constexpr int BM = 128;     // weight rows per CTA = UMMA M
constexpr int BK = 64;      // columns per stage: 64 bf16 = one 128-byte swizzle row
constexpr int NSTAGE = 4;
constexpr int DQ_WARPS = 8; // dequant + epilogue warps
constexpr int TC_THREADS = (DQ_WARPS + 2) * 32;
constexpr int TC_SPIN = 1 << 24;

template <int BN> struct GLay {
  static constexpr int A_STAGE = BM * 128;
  static constexpr int B_STAGE = BN * 128;
  static constexpr int A = 0;
  static constexpr int B = A + NSTAGE * A_STAGE;
  static constexpr int BAR = B + NSTAGE * B_STAGE;     // full_a, full_b, empty [NSTAGE]; acc_full; tmem slot
  static constexpr int TOTAL = BAR + (3 * NSTAGE + 2) * 8 + 1024;  // + slack for the 1024-byte alignment
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

// K-major, 128-byte swizzle shared-memory matrix descriptor: rows of 128 bytes, eight-row
// groups 1024 bytes apart, descriptor version 1 (sm_100), layout type 2 (SWIZZLE_128B).
__device__ __forceinline__ uint64_t smem_desc(const void* p) {
  const uint64_t addr = (uint64_t)(s32(p) >> 4) & 0x3fffu;
  return addr | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}

// kind::f16 instruction descriptor: D f32, A and B bf16, both K-major, M = 128, N = BN.
template <int BN> __host__ __device__ constexpr uint32_t instr_desc() {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *(const uint32_t*)&v;
}

__device__ __forceinline__ float h2f(uint32_t h) { return __half2float(__ushort_as_half((unsigned short)h)); }

// NB bytes at a 2-byte aligned global address -> words holding bytes 0.., realigned
template <int NW>
__device__ __forceinline__ void load_words_a2(const uint8_t* p, uint32_t (&v)[NW]) {
  const uintptr_t a = (uintptr_t)p;
  const uint32_t* base = (const uint32_t*)(a & ~(uintptr_t)3);
  if ((a & 2) == 0) {
#pragma unroll
    for (int i = 0; i < NW; ++i) v[i] = __ldg(base + i);
  } else {
    uint32_t w[NW + 1];
#pragma unroll
    for (int i = 0; i <= NW; ++i) w[i] = __ldg(base + i);  // the matrix allocation is padded past its last row
#pragma unroll
    for (int i = 0; i < NW; ++i) v[i] = __funnelshift_r(w[i], w[i + 1], 16);
  }
}

// The packed bytes one dequant thread needs for its 32 columns of one 64-column step.
template <int DT> struct Raw;
template <> struct Raw<DT_Q4_K> { uint4 hdr, q0, q1; };
template <> struct Raw<DT_Q8_0> { uint32_t w[9]; };
template <> struct Raw<DT_Q5_0> { uint32_t w[6]; };
template <> struct Raw<DT_Q5_1> { uint32_t w[6]; };

template <int DT>
__device__ __forceinline__ void load_raw(const uint8_t* row, int ks, int h, Raw<DT>& r) {
  if constexpr (DT == DT_Q4_K) {
    const uint8_t* blk = row + (ks >> 2) * 144;
    r.hdr = __ldg((const uint4*)blk);
    const uint4* q = (const uint4*)(blk + 16 + (ks & 3) * 32);
    r.q0 = __ldg(q);
    r.q1 = __ldg(q + 1);
  } else if constexpr (DT == DT_Q8_0) {
    load_words_a2<9>(row + (size_t)(2 * ks + h) * 34, r.w);
  } else if constexpr (DT == DT_Q5_0) {
    load_words_a2<6>(row + (size_t)(2 * ks + h) * 22, r.w);
  } else {
    load_words_a2<6>(row + (size_t)(2 * ks + h) * 24, r.w);
  }
}

__device__ __forceinline__ uint32_t byte_of(const uint32_t* w, int i) { return (w[i >> 2] >> (8 * (i & 3))) & 255u; }

// 32 dequantized weights of this thread as 16 packed bf16 pairs (column order).
template <int DT>
__device__ __forceinline__ void dequant32(const Raw<DT>& r, int ks, int h, uint32_t (&out)[16]) {
  if constexpr (DT == DT_Q4_K) {
    const float d = h2f(r.hdr.x & 0xffffu), dmin = h2f(r.hdr.x >> 16);
    const int sub = 2 * (ks & 3) + h;
    uint32_t sc, mn;
    if (sub < 4) {
      sc = (r.hdr.y >> (8 * sub)) & 63u;
      mn = (r.hdr.z >> (8 * sub)) & 63u;
    } else {
      const int jj = sub - 4;
      const uint32_t hb = (r.hdr.w >> (8 * jj)) & 255u;
      sc = (hb & 15u) | (((r.hdr.y >> (8 * jj + 6)) & 3u) << 4);
      mn = (hb >> 4) | (((r.hdr.z >> (8 * jj + 6)) & 3u) << 4);
    }
    const float a = d * (float)sc, nb = -(dmin * (float)mn);
    const uint32_t q[8] = {r.q0.x, r.q0.y, r.q0.z, r.q0.w, r.q1.x, r.q1.y, r.q1.z, r.q1.w};
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const uint32_t w4 = (h ? (q[i] >> 4) : q[i]) & 0x0f0f0f0fu;
      out[2 * i] = pack_bf16(fmaf(a, (float)(w4 & 255u), nb), fmaf(a, (float)((w4 >> 8) & 255u), nb));
      out[2 * i + 1] = pack_bf16(fmaf(a, (float)((w4 >> 16) & 255u), nb), fmaf(a, (float)(w4 >> 24), nb));
    }
  } else if constexpr (DT == DT_Q8_0) {
    const float d = h2f(r.w[0] & 0xffffu);
#pragma unroll
    for (int i = 0; i < 16; ++i)
      out[i] = pack_bf16((float)(int)(int8_t)byte_of(r.w, 2 + 2 * i) * d, (float)(int)(int8_t)byte_of(r.w, 3 + 2 * i) * d);
  } else {
    constexpr int HDR = DT == DT_Q5_0 ? 2 : 4;
    const float d = h2f(r.w[0] & 0xffffu);
    const float m = DT == DT_Q5_1 ? h2f(r.w[0] >> 16) : 0.0f;
    uint32_t qh = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) qh |= byte_of(r.w, HDR + i) << (8 * i);
    float wv[32];
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      const uint32_t p = byte_of(r.w, HDR + 4 + j);
      const int c0 = (int)((p & 15u) | (((qh >> j) & 1u) << 4));
      const int c1 = (int)((p >> 4) | (((qh >> (j + 16)) & 1u) << 4));
      wv[j] = DT == DT_Q5_0 ? (float)(c0 - 16) * d : fmaf((float)c0, d, m);
      wv[j + 16] = DT == DT_Q5_0 ? (float)(c1 - 16) * d : fmaf((float)c1, d, m);
    }
#pragma unroll
    for (int i = 0; i < 16; ++i) out[i] = pack_bf16(wv[2 * i], wv[2 * i + 1]);
  }
}

template <int DT, int BN>
__global__ void __launch_bounds__(TC_THREADS, 1)
gemm_tc_kernel(const uint8_t* __restrict__ W, int64_t row_bytes, int rows, int cols, int tokens,
               const __grid_constant__ CUtensorMap xmap, float* __restrict__ Y, int* __restrict__ err) {
  using L = GLay<BN>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);  // swizzle atoms are 1024 bytes
  uint8_t* sA = smem + L::A;
  uint8_t* sB = smem + L::B;
  uint64_t* full_a = (uint64_t*)(smem + L::BAR);
  uint64_t* full_b = full_a + NSTAGE;
  uint64_t* empty = full_b + NSTAGE;
  uint64_t* acc_full = empty + NSTAGE;
  uint32_t* tmem_slot = (uint32_t*)(acc_full + 1);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int row0 = blockIdx.x * BM, tok0 = blockIdx.y * BN;
  const int nk = cols / BK;

  if (tid == 0) {
    for (int s = 0; s < NSTAGE; ++s) { bar_init(&full_a[s], DQ_WARPS); bar_init(&full_b[s], 1); bar_init(&empty[s], 1); }
    bar_init(acc_full, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == DQ_WARPS + 1) {  // the MMA warp owns the tensor-memory allocation
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(s32(tmem_slot)), "r"(BN < 32 ? 32 : BN) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem = *tmem_slot;
  bool ok = true;

  if (warp < DQ_WARPS) {
    // ---------------------------------------------------------------- dequant
    const int r = tid & 127, h = tid >> 7;  // weight row inside the tile, column half of the step
    int grow = row0 + r;
    if (grow >= rows) grow = rows - 1;
    const uint8_t* wrow = W + (int64_t)grow * row_bytes;
    // packed bytes of the next PF steps are in flight in registers while this one is decoded
    constexpr int PF = 4;
    Raw<DT> buf[PF];
#pragma unroll
    for (int i = 0; i < PF; ++i)
      if (i < nk) load_raw<DT>(wrow, i, h, buf[i]);
    for (int ks0 = 0; ks0 < nk; ks0 += PF) {
#pragma unroll
      for (int i = 0; i < PF; ++i) {
        const int ks = ks0 + i;
        if (ks >= nk) break;
        const int s = ks % NSTAGE;
        uint32_t out[16];
        dequant32<DT>(buf[i], ks, h, out);
        if (ks + PF < nk) load_raw<DT>(wrow, ks + PF, h, buf[i]);
        if (ok && !bar_wait(&empty[s], (uint32_t)(((ks / NSTAGE) & 1) ^ 1))) { ok = false; atomicExch(err, 3); }
        uint8_t* arow = sA + s * L::A_STAGE + (r >> 3) * 1024 + (r & 7) * 128;
#pragma unroll
        for (int c4 = 0; c4 < 4; ++c4) {
          const int chunk = (4 * h + c4) ^ (r & 7);  // 128-byte swizzle: 16-byte chunk index xor row-in-group
          *(uint4*)(arow + chunk * 16) = make_uint4(out[4 * c4], out[4 * c4 + 1], out[4 * c4 + 2], out[4 * c4 + 3]);
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic-proxy stores -> visible to the MMA
        __syncwarp();
        if (lane == 0) bar_arrive(&full_a[s]);
      }
    }
    // --------------------------------------------------------------- epilogue
    if (ok && !bar_wait(acc_full, 0)) { ok = false; atomicExch(err, 3); }
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const int q = warp & 3, half = warp >> 2;  // TMEM lane quarter of this warp, column half
    const int out_row = row0 + 32 * q + lane;
    constexpr int CPW = BN / 2;  // columns per warp
#pragma unroll 1
    for (int c0 = half * CPW; c0 < (half + 1) * CPW; c0 += 32) {
      uint32_t v[32];
      const uint32_t taddr = tmem + ((uint32_t)(32 * q) << 16) + (uint32_t)c0;
      asm volatile(
          "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
          "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
          : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
            "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
            "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
            "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
          : "r"(taddr) : "memory");
      asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
      if (out_row < rows) {
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          const int tok = tok0 + c0 + j;
          if (tok < tokens) Y[(int64_t)tok * rows + out_row] = __uint_as_float(v[j]);
        }
      }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  } else if (warp == DQ_WARPS) {
    // ---------------------------------------------------- activation tiles (TMA)
    if (lane == 0) {
      for (int ks = 0; ks < nk; ++ks) {
        const int s = ks % NSTAGE;
        if (ok && !bar_wait(&empty[s], (uint32_t)(((ks / NSTAGE) & 1) ^ 1))) { ok = false; atomicExch(err, 3); }
        bar_expect(&full_b[s], BN * 128);
        asm volatile(
            "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
            ::"r"(s32(sB + s * L::B_STAGE)), "l"(&xmap), "r"(ks * BK), "r"(tok0), "r"(s32(&full_b[s])) : "memory");
      }
    }
  } else {
    // ------------------------------------------------------------------- MMA
    if (lane == 0) {
      constexpr uint32_t idesc = instr_desc<BN>();
      for (int ks = 0; ks < nk; ++ks) {
        const int s = ks % NSTAGE;
        const uint32_t par = (uint32_t)((ks / NSTAGE) & 1);
        if (ok && !(bar_wait(&full_a[s], par) && bar_wait(&full_b[s], par))) { ok = false; atomicExch(err, 3); }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint64_t da = smem_desc(sA + s * L::A_STAGE), db = smem_desc(sB + s * L::B_STAGE);
#pragma unroll
        for (int kk = 0; kk < BK / 16; ++kk) {
          const uint32_t acc = (ks | kk) ? 1u : 0u;
          // 16 bf16 = 32 bytes along K inside the swizzled row: advance the start address by 2 x 16 bytes
          asm volatile(
              "{ .reg .pred p; setp.ne.b32 p, %4, 0; tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p; }"
              ::"r"(tmem), "l"(da + 2 * kk), "l"(db + 2 * kk), "r"(idesc), "r"(acc) : "memory");
        }
        // frees the stage once the MMAs that read it have completed
        asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(s32(&empty[s])) : "memory");
      }
      asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(s32(acc_full)) : "memory");
    }
  }
  __syncthreads();
  if (warp == DQ_WARPS + 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(BN < 32 ? 32 : BN) : "memory");
  }
}

__global__ void to_bf16_kernel(const float* __restrict__ x, __nv_bfloat16* __restrict__ o, int64_t n) {
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

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)p;
  }
  return fn;
}

template <int DT, int BN>
cudaError_t launch_bn(const MatView& m, const CUtensorMap& xmap, float* y, int tokens, cudaStream_t stream, int* err) {
  auto kern = gemm_tc_kernel<DT, BN>;
  constexpr int smem = GLay<BN>::TOTAL;
  static bool ready = false;
  if (!ready) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return e;
    ready = true;
  }
  dim3 grid((unsigned)((m.rows + BM - 1) / BM), (unsigned)((tokens + BN - 1) / BN));
  kern<<<grid, TC_THREADS, smem, stream>>>(m.w, m.row_bytes, (int)m.rows, (int)m.cols, tokens, xmap, y, err);
  return cudaGetLastError();
}

template <int DT>
cudaError_t launch_dt(const MatView& m, const __nv_bfloat16* xb, float* y, int tokens, cudaStream_t stream, int* err) {
  EncodeTiledFn enc = encode_fn();
  if (!enc) return cudaErrorNotSupported;
  const int bn = tokens > 128 ? 256 : tokens > 64 ? 128 : 64;
  CUtensorMap xmap;
  const cuuint64_t dims[2] = {(cuuint64_t)m.cols, (cuuint64_t)tokens};
  const cuuint64_t strides[1] = {(cuuint64_t)m.cols * 2};
  const cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)bn};
  const cuuint32_t estr[2] = {1, 1};
  if (enc(&xmap, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (void*)xb, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
          CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return cudaErrorInvalidValue;
  if (bn == 256) return launch_bn<DT, 256>(m, xmap, y, tokens, stream, err);
  if (bn == 128) return launch_bn<DT, 128>(m, xmap, y, tokens, stream, err);
  return launch_bn<DT, 64>(m, xmap, y, tokens, stream, err);
}

}  // namespace

bool gemm_tc_supported(const MatView& m, int64_t tokens) {
  if (m.dtype != DT_Q4_K && m.dtype != DT_Q8_0 && m.dtype != DT_Q5_0 && m.dtype != DT_Q5_1) return false;
  if (tokens < 16 || tokens > (1 << 24) || m.rows <= 0 || m.rows > (1 << 30)) return false;
  if (m.cols % BK != 0 || m.cols <= 0 || m.cols > (1 << 30)) return false;
  return ((uintptr_t)m.w & 15) == 0;
}

size_t gemm_tc_scratch_bytes(const MatView& m, int64_t tokens) { return (size_t)tokens * (size_t)m.cols * 2; }

cudaError_t launch_gemm_tc(const MatView& m, const float* x, float* y, int64_t tokens, void* scratch,
                           cudaStream_t stream, int* err_flag, uint64_t* launches) {
  __nv_bfloat16* xb = (__nv_bfloat16*)scratch;
  const int64_t n = tokens * m.cols;
  int64_t blocks = (n / 4 + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  if (blocks < 1) blocks = 1;
  to_bf16_kernel<<<(unsigned)blocks, 256, 0, stream>>>(x, xb, n);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  if (launches) ++*launches;
  switch (m.dtype) {
    case DT_Q4_K: e = launch_dt<DT_Q4_K>(m, xb, y, (int)tokens, stream, err_flag); break;
    case DT_Q8_0: e = launch_dt<DT_Q8_0>(m, xb, y, (int)tokens, stream, err_flag); break;
    case DT_Q5_0: e = launch_dt<DT_Q5_0>(m, xb, y, (int)tokens, stream, err_flag); break;
    case DT_Q5_1: e = launch_dt<DT_Q5_1>(m, xb, y, (int)tokens, stream, err_flag); break;
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
static __device__ __align__(256) unsigned char g_static_scratch[GEMM_STATIC_SCRATCH_BYTES];

size_t gemm_tc_static_scratch_limit() { return GEMM_STATIC_SCRATCH_BYTES; }

cudaError_t launch_gemm_tc_static(int device, const MatView& m, const float* x, float* y, int64_t tokens,
                                  cudaStream_t stream, int* err_flag, uint64_t* launches) {
  // In host code `g_static_scratch` is only a handle for the symbol, not a device address:
  // the address is looked up once per device, with that device current.
  static void* addr[64] = {nullptr};
  if (device < 0 || device >= 64) return cudaErrorInvalidDevice;
  if (!addr[device]) {
    void* p = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(&p, g_static_scratch);
    if (e != cudaSuccess) return e;
    addr[device] = p;
  }
  return launch_gemm_tc(m, x, y, tokens, addr[device], stream, err_flag, launches);
}

}  // namespace llr
