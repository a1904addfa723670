// Seeded synthetic packed weights, generated on the device.
//
// Bit-identical to llama_rust_b200/synth.py (the host generator the parity
// tests use), so a benchmark matrix and a test matrix with the same seed are
// the same bytes.  Everything is integer or correctly-rounded IEEE arithmetic:
//  * the stream is SplitMix64 (langtax/src/sample.rs:306-312) used as a
//    counter generator, word i = mix(seed + (i+1)*0x9E3779B97F4A7C15);
//  * quant bits are the raw bytes of the stream (Q8_0 codes are byte % 255 - 127
//    so that they are uniform in [-127, 127]);
//  * a "normal" n is Irwin-Hall: the twelve 16-bit fields of three words are
//    summed as integers, n = (S - 393210) / 65536 in binary64;
//  * block scales are |n| * 0.01 rounded to binary32 and then truncated to
//    binary16 the way the reference's f32_to_f16 does (langtax/src/fp16.rs:36-62).
#include "llr_formats.cuh"
#include "llr_kernels.cuh"

namespace llr {
namespace {

__host__ __device__ inline uint64_t sm64(uint64_t seed, uint64_t i) {
  uint64_t z = seed + (i + 1) * 0x9E3779B97F4A7C15ull;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}

__device__ inline double normal3(uint64_t seed, uint64_t i) {
  uint32_t s = 0;
#pragma unroll
  for (int k = 0; k < 3; ++k) {
    const uint64_t w = sm64(seed, i + k);
    s += (uint32_t)(w & 0xffff) + (uint32_t)((w >> 16) & 0xffff) + (uint32_t)((w >> 32) & 0xffff) +
         (uint32_t)(w >> 48);
  }
  return ((double)s - 393210.0) / 65536.0;
}

// truncating binary32 -> binary16 of the reference (fp16.rs:36-62)
__device__ inline uint16_t f32_to_f16_trunc(float f) {
  const uint32_t b = __float_as_uint(f);
  const uint16_t sign = (uint16_t)((b >> 16) & 0x8000u);
  const int biased = (int)((b >> 23) & 0xffu);
  const int exp = biased - 127 + 15;
  const uint32_t man = (b >> 13) & 0x3ffu;
  if (exp >= 31) return (uint16_t)(sign | 0x7c00u);
  if (exp > 0) return (uint16_t)(sign | (exp << 10) | man);
  if (biased == 0) return sign;
  const int shift = 1 - exp;
  if (shift > 11) return sign;
  return (uint16_t)(sign | (((0x400u | man) >> shift) & 0x3ffu));
}

__device__ inline uint16_t scale16(uint64_t seed, uint64_t i) {
  return f32_to_f16_trunc((float)(fabs(normal3(seed, i)) * 0.01));
}

__device__ inline void put_words(uint8_t* dst, uint64_t seed, uint64_t i0, int nbytes) {
  for (int k = 0; k < nbytes; ++k) dst[k] = (uint8_t)(sm64(seed, i0 + (k >> 3)) >> (8 * (k & 7)));
}

__device__ inline void put16(uint8_t* dst, uint16_t v) {
  dst[0] = (uint8_t)v;
  dst[1] = (uint8_t)(v >> 8);
}

__host__ __device__ constexpr int words_per_block(int dt) {
  return dt == DT_Q8_0 ? 7 : dt == DT_Q4_0 ? 5 : dt == DT_Q5_0 ? 6 : dt == DT_Q5_1 ? 9 : dt == DT_Q4_1 ? 8
         : dt == DT_Q4_K ? 24 : dt == DT_Q5_K ? 28 : dt == DT_Q6_K ? 29 : 3;
}

template <int DT>
__global__ void synth_kernel(uint8_t* __restrict__ w, int64_t n_blocks, uint64_t seed) {
  constexpr int WPB = words_per_block(DT);
  constexpr int BB = block_bytes(DT);
  for (int64_t b = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; b < n_blocks;
       b += (int64_t)gridDim.x * blockDim.x) {
    uint8_t* o = w + b * BB;
    const uint64_t i0 = (uint64_t)b * WPB;
    if constexpr (DT == DT_Q8_0) {
      for (int k = 0; k < 32; ++k) {
        const uint32_t byte = (uint32_t)(sm64(seed, i0 + (k >> 3)) >> (8 * (k & 7))) & 255u;
        o[2 + k] = (uint8_t)(int8_t)((int)(byte % 255u) - 127);
      }
      put16(o, scale16(seed, i0 + 4));
    } else if constexpr (DT == DT_Q4_0) {
      put_words(o + 2, seed, i0, 16);
      put16(o, scale16(seed, i0 + 2));
    } else if constexpr (DT == DT_Q5_0) {
      put_words(o + 2, seed, i0, 4);
      put_words(o + 6, seed, i0 + 1, 16);
      put16(o, scale16(seed, i0 + 3));
    } else if constexpr (DT == DT_Q5_1) {
      put_words(o + 4, seed, i0, 4);
      put_words(o + 8, seed, i0 + 1, 16);
      put16(o, scale16(seed, i0 + 3));
      put16(o + 2, scale16(seed, i0 + 6));
    } else if constexpr (DT == DT_Q4_1) {
      put_words(o + 4, seed, i0, 16);
      put16(o, scale16(seed, i0 + 2));
      put16(o + 2, scale16(seed, i0 + 5));
    } else if constexpr (DT == DT_Q5_K) {
      put_words(o + 48, seed, i0, 128);
      put_words(o + 16, seed, i0 + 16, 32);
      put_words(o + 4, seed, i0 + 20, 12);
      put16(o, scale16(seed, i0 + 22));
      put16(o + 2, scale16(seed, i0 + 25));
    } else if constexpr (DT == DT_Q4_K) {
      put_words(o + 16, seed, i0, 128);
      put_words(o + 4, seed, i0 + 16, 12);
      put16(o, scale16(seed, i0 + 18));
      put16(o + 2, scale16(seed, i0 + 21));
    } else if constexpr (DT == DT_Q6_K) {
      put_words(o, seed, i0, 128);
      put_words(o + 128, seed, i0 + 16, 64);
      put_words(o + 192, seed, i0 + 24, 16);
      put16(o + 208, scale16(seed, i0 + 26));
    } else {
      const float v = (float)(normal3(seed, i0) * 0.02);
      if constexpr (DT == DT_F32) {
        const uint32_t u = __float_as_uint(v);
        o[0] = (uint8_t)u; o[1] = (uint8_t)(u >> 8); o[2] = (uint8_t)(u >> 16); o[3] = (uint8_t)(u >> 24);
      } else if constexpr (DT == DT_F16) {
        put16(o, f32_to_f16_trunc(v));
      } else {
        const uint32_t u = __float_as_uint(v);  // bf16 round-to-nearest-even (fp16.rs:142-151)
        put16(o, (uint16_t)((u + 0x7fffu + ((u >> 16) & 1u)) >> 16));
      }
    }
  }
}

}  // namespace

cudaError_t launch_synth(int dtype, int64_t rows, int64_t cols, uint64_t seed, uint8_t* w,
                         cudaStream_t stream, uint64_t* launches) {
  const int be = block_elems(dtype);
  if (be == 0) return cudaErrorInvalidValue;
  const int64_t n_blocks = rows * (cols / be);
  if (n_blocks <= 0) return cudaSuccess;
  int64_t blocks = (n_blocks + 255) / 256;
  if (blocks > 148 * 64) blocks = 148 * 64;
  switch (dtype) {
#define LLR_SYNTH_CASE(D) case D: synth_kernel<D><<<(unsigned)blocks, 256, 0, stream>>>(w, n_blocks, seed); break;
    LLR_SYNTH_CASE(DT_F16) LLR_SYNTH_CASE(DT_BF16) LLR_SYNTH_CASE(DT_F32) LLR_SYNTH_CASE(DT_Q5_0)
    LLR_SYNTH_CASE(DT_Q5_1) LLR_SYNTH_CASE(DT_Q4_0) LLR_SYNTH_CASE(DT_Q8_0) LLR_SYNTH_CASE(DT_Q4_K)
    LLR_SYNTH_CASE(DT_Q6_K) LLR_SYNTH_CASE(DT_Q4_1) LLR_SYNTH_CASE(DT_Q5_K)
#undef LLR_SYNTH_CASE
    default: return cudaErrorInvalidValue;
  }
  if (launches) ++*launches;
  return cudaGetLastError();
}

}  // namespace llr
