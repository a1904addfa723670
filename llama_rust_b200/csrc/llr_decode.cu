// Element-wise and attention kernels of the device-resident Llama walk: what stands between the matrix
// products of Llama::forward_layers (langtax/src/decode.rs:2737-3097) -- rmsnorm_inplace :11498, rope :11578
// (adjacent-pair rotation), store_kv :12059, attend_query :11126 with grouped-query heads, silu :11826,
// the residual adds -- and the greedy argmax of sample.rs:293.  The host walk of the reference runs these on
// the CPU between two executor calls; here a decode step never leaves the device.
//
// Arithmetic follows the reference's formulas; sums that the reference adds sequentially (sum of squares,
// attention scores, softmax denominator, weighted values) are added in a fixed tree / block order here, so
// results are reproducible from run to run and differ from the CPU walk in the last bits only.
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdlib>
#include <math_constants.h>

#include "llr_kernels.cuh"

namespace llr {
namespace {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(~0u, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(~0u, v, o));
  return v;
}
// block-wide sum / max through shared memory (blockDim.x a multiple of 32, at most 1024); every thread gets the result
__device__ __forceinline__ float block_sum(float v, float* sh) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) sh[warp] = v;
  __syncthreads();
  float t = 0.f;
  for (int w = 0; w < nw; ++w) t += sh[w];  // fixed order
  return t;
}

__device__ __forceinline__ int row_position(const RowMap& r, int t) { return r.row_pos ? r.row_pos[t] : *r.pos_dev + t; }
__device__ __forceinline__ int row_sequence(const RowMap& r, int t) { return r.row_seq ? r.row_seq[t] : 0; }
// first float of the head vector of (sequence, layer, kv head, position) in a paged cache
__device__ __forceinline__ int64_t kv_offset(const KvView& kv, int seq, int layer, int head, int pos, int n_head_kv, int hd) {
  const int b = kv.table[(int64_t)seq * kv.max_blocks + pos / kv.block_tokens];
  return ((((int64_t)b * kv.n_layer + layer) * n_head_kv + head) * kv.block_tokens + pos % kv.block_tokens) * hd;
}

// The element-wise kernels of the walk are launched with programmatic stream serialization: a kernel may be placed on
// the SMs while its predecessor still runs, so its launch latency overlaps the predecessor's execution.  Each kernel
// therefore waits for its predecessor (and everything before it) before it reads anything, and lets its successor be
// placed right away; the matrix kernels that follow use that to prefetch weights.
__device__ __forceinline__ void pdl_enter() {
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

// one block per activation row; a row of up to 4096 values stays in registers between the two passes
constexpr int NORM_THREADS = 1024;
__global__ void __launch_bounds__(NORM_THREADS)
rmsnorm_kernel(float* __restrict__ x, const float* __restrict__ add, const float* __restrict__ w, float* __restrict__ y,
               int n, float eps) {
  pdl_enter();
  __shared__ float sh[32];
  float* xr = x + (int64_t)blockIdx.x * n;
  const float* ar = add ? add + (int64_t)blockIdx.x * n : nullptr;
  float* yr = y + (int64_t)blockIdx.x * n;
  const bool in_regs = n <= 4 * NORM_THREADS && n % 4 == 0;
  float4 keep = make_float4(0.f, 0.f, 0.f, 0.f);
  float ss = 0.f;
  if (in_regs) {
    const int i = 4 * threadIdx.x;
    if (i < n) {
      keep = *(const float4*)(xr + i);
      if (ar) {  // proj + residual (decode.rs:2938, :3050), written back: the new residual stream
        const float4 a = *(const float4*)(ar + i);
        keep.x = __fadd_rn(a.x, keep.x); keep.y = __fadd_rn(a.y, keep.y); keep.z = __fadd_rn(a.z, keep.z); keep.w = __fadd_rn(a.w, keep.w);
        *(float4*)(xr + i) = keep;
      }
      ss = fmaf(keep.x, keep.x, fmaf(keep.y, keep.y, fmaf(keep.z, keep.z, keep.w * keep.w)));
    }
  } else {
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
      float v = xr[i];
      if (ar) { v = __fadd_rn(ar[i], v); xr[i] = v; }
      ss = fmaf(v, v, ss);
    }
  }
  ss = block_sum(ss, sh);
  const float rms = sqrtf(__fadd_rn(__fdiv_rn(ss, (float)(n <= 65535 ? n : 1)), eps));
  const float inv = rms > 0.f ? __fdiv_rn(1.0f, rms) : 0.f;
  if (in_regs) {
    const int i = 4 * threadIdx.x;
    if (i < n) {
      float4 o = make_float4(__fmul_rn(keep.x, inv), __fmul_rn(keep.y, inv), __fmul_rn(keep.z, inv), __fmul_rn(keep.w, inv));
      if (w) {
        const float4 ww = *(const float4*)(w + i);
        o.x = __fmul_rn(o.x, ww.x); o.y = __fmul_rn(o.y, ww.y); o.z = __fmul_rn(o.z, ww.z); o.w = __fmul_rn(o.w, ww.w);
      }
      *(float4*)(yr + i) = o;
    }
  } else {
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
      const float t = __fmul_rn(xr[i], inv);
      yr[i] = w ? __fmul_rn(t, w[i]) : t;
    }
  }
}

// One block per token: the cosine and sine of every pair's angle once (all heads of a token turn by the same
// angles), then the rotation of every q and k head, then the k and v rows into the cache.
__global__ void __launch_bounds__(256)
rope_store_kernel(float* __restrict__ q, float* __restrict__ k, const float* __restrict__ v, KvView kv, RowMap rows, int layer,
                  WalkShape w) {
  pdl_enter();
  __shared__ float s_cos[128], s_sin[128];  // head_dim <= 256
  const int t = blockIdx.x;
  const int pos = row_position(rows, t);
  const int hd = w.head_dim, half = hd / 2;
  const float theta_scale = w.theta_scale;  // base^(-2/n_rot), computed once on the host in f32 as the reference does
  for (int p = threadIdx.x; p < half; p += blockDim.x) {
    float theta = (float)(pos <= 65535 ? pos : 65535);
    for (int i = 0; i < p; ++i) theta *= theta_scale;  // the reference advances theta multiplicatively in f32
    s_cos[p] = cosf(theta);
    s_sin[p] = sinf(theta);
  }
  __syncthreads();
  float* qrow = q + (int64_t)t * w.n_head * hd;
  float* krow = k + (int64_t)t * w.n_head_kv * hd;
  for (int idx = threadIdx.x; idx < (w.n_head + w.n_head_kv) * half; idx += blockDim.x) {
    const int h = idx / half, p = idx % half;
    float* vec = h < w.n_head ? qrow + h * hd : krow + (h - w.n_head) * hd;
    const float c = s_cos[p], s = s_sin[p];
    const float2 ab = *(const float2*)(vec + 2 * p);
    *(float2*)(vec + 2 * p) = make_float2(__fsub_rn(__fmul_rn(ab.x, c), __fmul_rn(ab.y, s)), __fadd_rn(__fmul_rn(ab.x, s), __fmul_rn(ab.y, c)));
  }
  __syncthreads();  // the rotated keys are read back below by other threads of the block
  // store_kv (decode.rs:12059) into the row's sequence, paged
  const int sid = row_sequence(rows, t);
  const float* vrow = v + (int64_t)t * w.n_head_kv * hd;
  for (int idx = threadIdx.x; idx < w.n_head_kv * hd; idx += blockDim.x) {
    const int hk = idx / hd, i = idx % hd;
    const int64_t off = kv_offset(kv, sid, layer, hk, pos, w.n_head_kv, hd);
    kv.k[off + i] = krow[idx];
    kv.v[off + i] = vrow[idx];
  }
}

// Attention of one row over one slice of positions.  A block handles the query heads that share a kv head and
// writes, per query head, the slice's maximum score, the sum of exp(score - max) and the exp-weighted sum of value
// rows; attention_combine_kernel merges the slices (the usual two-pass softmax, rearranged so that K and V are read
// once per kv head and by many SMs).  Slices have a fixed length in positions (attention_chunk), whatever the batch: a
// row's result depends on its own sequence only, never on what shares its batch.
// `KV` says where the key and value rows of a position lie: in the paged cache (one row per block: decode steps) or
// in a shared-memory tile that a block fills once for many rows of a prompt chunk.  The arithmetic is this one
// function either way, so both kernels give the same bits.
constexpr int ATT_THREADS = 256;
constexpr int ATT_MAX_GQA = 8;
constexpr int ATT_ROWS = 16;       // rows per block of the tiled kernel
constexpr int ATT_TILE_CHUNK = 128; // longest slice the tiled kernel stages (2 x 128 x head_dim floats: contexts up to 4096 positions)

struct KvGlobal {
  const KvView& kv;
  int sid, layer, hkv, n_head_kv, hd;
  __device__ __forceinline__ const float* k(int s) const { return kv.k + kv_offset(kv, sid, layer, hkv, s, n_head_kv, hd); }
  __device__ __forceinline__ const float* v(int s) const { return kv.v + kv_offset(kv, sid, layer, hkv, s, n_head_kv, hd); }
};
struct KvTile {
  const float* kt;
  const float* vt;
  int s0, hd;
  __device__ __forceinline__ const float* k(int s) const { return kt + (s - s0) * hd; }
  __device__ __forceinline__ const float* v(int s) const { return vt + (s - s0) * hd; }
};

// sq: the row's query heads of this kv head [gqa][hd] in shared memory (filled and synchronized by the caller);
// sc: [max(gqa * max_chunk, P * gqa * hd)] floats of shared memory; out: the slice's record of this row.
// Ends with the block's threads past their last read of sq and sc only after the caller's next __syncthreads().
template <typename KV>
__device__ __forceinline__ void attend_slice(const KV& src, const float* sq, float* sc, float* out, int s0, int s1, int max_chunk,
                                             int hd, int gqa) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = ATT_THREADS / 32;
  const float scale = 1.0f / sqrtf((float)hd);
  // scores: one warp per position, all query heads of the group against one read of the K row.  Four positions are in
  // flight per warp (their K rows are fetched before any of them is used): the loop is bound by memory latency, not
  // by arithmetic.  Each position's sum is formed exactly as if it were alone: columns in ascending order per lane.
  constexpr int SP = 4;
  for (int sbase = s0 + warp; sbase < s1; sbase += nw * SP) {
    float acc[SP][ATT_MAX_GQA];
    const float* krow[SP];
#pragma unroll
    for (int j = 0; j < SP; ++j) {
      const int sj = sbase + j * nw;
      krow[j] = sj < s1 ? src.k(sj) : nullptr;
#pragma unroll
      for (int g = 0; g < ATT_MAX_GQA; ++g) acc[j][g] = 0.f;
    }
    for (int i0 = 0; i0 < hd; i0 += 128) {
      float kvv[SP][4];
#pragma unroll
      for (int j = 0; j < SP; ++j)
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int i = i0 + lane + 32 * u;
          kvv[j][u] = (krow[j] && i < hd) ? krow[j][i] : 0.f;
        }
#pragma unroll
      for (int j = 0; j < SP; ++j)
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int i = i0 + lane + 32 * u;
          if (krow[j] && i < hd) {
#pragma unroll
            for (int g = 0; g < ATT_MAX_GQA; ++g)
              if (g < gqa) acc[j][g] = fmaf(sq[g * hd + i], kvv[j][u], acc[j][g]);
          }
        }
    }
#pragma unroll
    for (int j = 0; j < SP; ++j) {
      const int sj = sbase + j * nw;
      if (sj < s1) {  // warp-uniform
#pragma unroll
        for (int g = 0; g < ATT_MAX_GQA; ++g)
          if (g < gqa) {
            const float d = warp_sum(acc[j][g]);
            if (lane == 0) sc[g * max_chunk + (sj - s0)] = __fmul_rn(d, scale);
          }
      }
    }
  }
  __syncthreads();
  // per query head: the slice's maximum and the sum of exp(score - max); one warp per head, lanes add in a fixed tree
  for (int g = warp; g < gqa; g += nw) {
    float m = -CUDART_INF_F;
    for (int s = lane; s < s1 - s0; s += 32) m = fmaxf(m, sc[g * max_chunk + s]);
    m = warp_max(m);
    float l = 0.f;
    for (int s = lane; s < s1 - s0; s += 32) {
      const float e = expf(sc[g * max_chunk + s] - m);
      sc[g * max_chunk + s] = e;
      l += e;
    }
    l = warp_sum(l);
    if (lane == 0) { out[g * (hd + 2) + hd] = m; out[g * (hd + 2) + hd + 1] = l; }
  }
  __syncthreads();
  // weighted values: thread (i, grp) owns dimension i for every P-th run of eight positions of the slice
  // (P = ATT_THREADS / hd thread groups); the groups' sums are added in group order through shared memory
  const int P = ATT_THREADS / hd > 0 ? ATT_THREADS / hd : 1;
  float acc[ATT_MAX_GQA];
#pragma unroll
  for (int g = 0; g < ATT_MAX_GQA; ++g) acc[g] = 0.f;
  const int i = threadIdx.x % hd, grp = threadIdx.x / hd;
  if (grp < P) {
    // runs of eight positions go to the groups in turn: the split does not depend on the KV block size.  The eight
    // value rows of a run are fetched before the first is used; the sums are formed in ascending position order.
    for (int sb = s0 + 8 * grp; sb < s1; sb += 8 * P) {
      float vv[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) vv[j] = sb + j < s1 ? src.v(sb + j)[i] : 0.f;
#pragma unroll
      for (int j = 0; j < 8; ++j)
        if (sb + j < s1) {
#pragma unroll
          for (int g = 0; g < ATT_MAX_GQA; ++g)
            if (g < gqa) acc[g] = fmaf(sc[g * max_chunk + (sb + j - s0)], vv[j], acc[g]);
        }
    }
  }
  __syncthreads();  // the scores are no longer needed: their space takes the groups' partial sums
  float* vsum = sc;  // [P][gqa][hd]
  if (grp < P)
#pragma unroll
    for (int g = 0; g < ATT_MAX_GQA; ++g)
      if (g < gqa) vsum[(grp * gqa + g) * hd + i] = acc[g];
  __syncthreads();
  for (int idx = threadIdx.x; idx < gqa * hd; idx += ATT_THREADS) {
    float v = 0.f;
    for (int p = 0; p < P; ++p) v += vsum[p * gqa * hd + idx];
    out[(idx / hd) * (hd + 2) + idx % hd] = v;
  }
}

// The rotation of rope_store_kernel on n_vec vectors of hd floats in shared memory: one thread per pair
__device__ __forceinline__ void rope_in_place(float* vecs, int n_vec, int hd, int pos, float theta_scale) {
  const int half = hd / 2;
  for (int idx = threadIdx.x; idx < n_vec * half; idx += blockDim.x) {
    float* vec = vecs + (idx / half) * hd;
    const int p = idx % half;
    float theta = (float)(pos <= 65535 ? pos : 65535);
    for (int i = 0; i < p; ++i) theta *= theta_scale;
    const float c = cosf(theta), s = sinf(theta);
    const float a = vec[2 * p], b = vec[2 * p + 1];
    vec[2 * p] = __fsub_rn(__fmul_rn(a, c), __fmul_rn(b, s));
    vec[2 * p + 1] = __fadd_rn(__fmul_rn(a, s), __fmul_rn(b, c));
  }
}

// grid (kv head, position slice, token): one row per block, K and V straight from the paged cache (decode steps).
// With k_new / v_new (a single decode token) the kernel also does what rope_store_kernel does for that token: q is
// rotated as it is loaded, and the block whose slice holds the token's position rotates the new key, writes it and
// the new value into the cache and then reads them back like any other position: one launch less per layer.
__global__ void __launch_bounds__(ATT_THREADS)
attention_partial_kernel(const float* __restrict__ q, KvView kv, float* __restrict__ part, RowMap rows, int layer, int chunk,
                         WalkShape w, const float* __restrict__ k_new, const float* __restrict__ v_new) {
  pdl_enter();
  extern __shared__ float sm[];  // q[gqa][hd] | scores[gqa][chunk] or sums[P][gqa][hd]
  const int hkv = blockIdx.x, split = blockIdx.y, t = blockIdx.z;
  const int hd = w.head_dim, gqa = w.n_head / w.n_head_kv;
  const int seq = row_position(rows, t) + 1;  // positions this row attends to
  const int sid = row_sequence(rows, t);
  const int n_split = (int)gridDim.y;
  const int s0 = split * chunk, s1 = min(seq, s0 + chunk);
  if (s0 >= seq) return;  // this row's sequence ends before the slice
  float* sq = sm;
  float* sc = sq + gqa * hd;
  for (int i = threadIdx.x; i < gqa * hd; i += ATT_THREADS)
    sq[i] = q[((int64_t)t * w.n_head + hkv * gqa) * hd + i];
  if (k_new) {
    const bool mine = s1 == seq;  // the slice that holds the token's own position
    if (mine)
      for (int i = threadIdx.x; i < hd; i += ATT_THREADS) sc[i] = k_new[((int64_t)t * w.n_head_kv + hkv) * hd + i];
    __syncthreads();
    rope_in_place(sq, gqa, hd, seq - 1, w.theta_scale);
    if (mine) {
      rope_in_place(sc, 1, hd, seq - 1, w.theta_scale);
      __syncthreads();
      const int64_t off = kv_offset(kv, sid, layer, hkv, seq - 1, w.n_head_kv, hd);
      for (int i = threadIdx.x; i < hd; i += ATT_THREADS) {
        kv.k[off + i] = sc[i];
        kv.v[off + i] = v_new[((int64_t)t * w.n_head_kv + hkv) * hd + i];
      }
    }
  }
  __syncthreads();
  float* out = part + (((int64_t)t * w.n_head_kv + hkv) * n_split + split) * gqa * (hd + 2);
  attend_slice(KvGlobal{kv, sid, layer, hkv, w.n_head_kv, hd}, sq, sc, out, s0, s1, chunk, hd, gqa);
}

// The same slice of one row done by ONE warp, every elementary sum formed in the order attend_slice forms it (a
// position's score: lanes over the columns in ascending order, then the shuffle tree; a head's softmax: lanes over the
// positions; a dimension's weighted sum: per group of runs of eight positions in ascending order, then the groups in
// order), so the bits are the same.  GQA query heads per kv head and P = ATT_THREADS / head_dim groups are template
// parameters: nothing is predicated, and the loop over the value rows goes over the positions once, each position's
// weights and value row loaded once for all the dimensions and heads a lane owns (the loop is bound by shared-memory
// loads).  sq [GQA][hd] and sc [GQA][max_chunk] are this warp's.
template <int GQA, int P, typename KV>
__device__ __forceinline__ void attend_slice_warp(const KV& src, const float* sq, float* sc, float* out, int s0, int s1, int max_chunk) {
  constexpr int HD = ATT_THREADS / P, ND = HD / 32;
  const int lane = threadIdx.x & 31;
  const float scale = 1.0f / sqrtf((float)HD);
  constexpr int SP = 4;
  for (int sbase = s0; sbase < s1; sbase += SP) {
    float acc[SP][GQA];
    float kvv[SP][ND];
#pragma unroll
    for (int j = 0; j < SP; ++j) {
      const bool live = sbase + j < s1;
      const float* krow = src.k(live ? sbase + j : s0);
#pragma unroll
      for (int u = 0; u < ND; ++u) kvv[j][u] = live ? krow[lane + 32 * u] : 0.f;
#pragma unroll
      for (int g = 0; g < GQA; ++g) acc[j][g] = 0.f;
    }
#pragma unroll
    for (int u = 0; u < ND; ++u)
#pragma unroll
      for (int g = 0; g < GQA; ++g) {
        const float qv = sq[g * HD + lane + 32 * u];
#pragma unroll
        for (int j = 0; j < SP; ++j) acc[j][g] = fmaf(qv, kvv[j][u], acc[j][g]);
      }
#pragma unroll
    for (int j = 0; j < SP; ++j)
      if (sbase + j < s1) {
#pragma unroll
        for (int g = 0; g < GQA; ++g) {
          const float d = warp_sum(acc[j][g]);
          if (lane == 0) sc[g * max_chunk + (sbase + j - s0)] = __fmul_rn(d, scale);
        }
      }
  }
  __syncwarp();
#pragma unroll
  for (int g = 0; g < GQA; ++g) {
    float m = -CUDART_INF_F;
    for (int s = lane; s < s1 - s0; s += 32) m = fmaxf(m, sc[g * max_chunk + s]);
    m = warp_max(m);
    float l = 0.f;
    for (int s = lane; s < s1 - s0; s += 32) {
      const float e = expf(sc[g * max_chunk + s] - m);
      sc[g * max_chunk + s] = e;
      l += e;
    }
    l = warp_sum(l);
    if (lane == 0) { out[g * (HD + 2) + HD] = m; out[g * (HD + 2) + HD + 1] = l; }
  }
  __syncwarp();
  float acc[ND][P][GQA];
#pragma unroll
  for (int k = 0; k < ND; ++k)
#pragma unroll
    for (int grp = 0; grp < P; ++grp)
#pragma unroll
      for (int g = 0; g < GQA; ++g) acc[k][grp][g] = 0.f;
  for (int rb = 0; s0 + 8 * rb < s1; rb += P) {
#pragma unroll
    for (int grp = 0; grp < P; ++grp) {
      const int sb = s0 + 8 * (rb + grp);
#pragma unroll
      for (int j = 0; j < 8; ++j)
        if (sb + j < s1) {
          float e[GQA], v[ND];
          const float* vrow = src.v(sb + j);
#pragma unroll
          for (int g = 0; g < GQA; ++g) e[g] = sc[g * max_chunk + (sb + j - s0)];
#pragma unroll
          for (int k = 0; k < ND; ++k) v[k] = vrow[lane + 32 * k];
#pragma unroll
          for (int k = 0; k < ND; ++k)
#pragma unroll
            for (int g = 0; g < GQA; ++g) acc[k][grp][g] = fmaf(e[g], v[k], acc[k][grp][g]);
        }
    }
  }
#pragma unroll
  for (int k = 0; k < ND; ++k)
#pragma unroll
    for (int g = 0; g < GQA; ++g) {
      float total = 0.f;
#pragma unroll
      for (int grp = 0; grp < P; ++grp) total += acc[k][grp][g];
      out[g * (HD + 2) + lane + 32 * k] = total;
    }
}

// grid (kv head, position slice, group of ATT_ROWS rows): the rows of a prompt chunk share the slice's key and value
// rows, which the block stages in shared memory once per run of rows of one sequence; each warp then takes rows of
// its own, with no block-wide barrier between rows.
template <int GQA, int P>
__global__ void __launch_bounds__(ATT_THREADS, 3)
attention_tile_kernel(const float* __restrict__ q, KvView kv, float* __restrict__ part, RowMap rows, int layer, int chunk,
                      WalkShape w, int tokens) {
  pdl_enter();
  extern __shared__ float sm[];  // k tile [chunk][hd] | v tile [chunk][hd] | per warp: q[gqa][hd], scores[gqa][chunk]
  constexpr int hd = ATT_THREADS / P, gqa = GQA;
  const int hkv = blockIdx.x, split = blockIdx.y;
  const int n_split = (int)gridDim.y;
  const int s0 = split * chunk;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = ATT_THREADS / 32;
  float* kt = sm;
  float* vt = kt + chunk * hd;
  float* sq = vt + chunk * hd + warp * gqa * hd;
  float* sc = vt + chunk * hd + nw * gqa * hd + warp * gqa * chunk;
  // the last rows first: in a prompt chunk they attend to the most slices, the blocks of the first rows (which leave at once for
  // the slices beyond them) then fill the tail
  const int t_begin = ((int)gridDim.z - 1 - (int)blockIdx.z) * ATT_ROWS, t_end = min(tokens, t_begin + ATT_ROWS);
  // sequence and position of the group's rows, fetched in one go (the runs below are found in shared memory)
  __shared__ int s_seq[ATT_ROWS], s_pos[ATT_ROWS];
  if (threadIdx.x < ATT_ROWS && t_begin + (int)threadIdx.x < t_end) {
    s_seq[threadIdx.x] = row_sequence(rows, t_begin + threadIdx.x);
    s_pos[threadIdx.x] = row_position(rows, t_begin + threadIdx.x);
  }
  __syncthreads();
  for (int t = t_begin; t < t_end;) {  // runs of rows of one sequence; everything here is block-uniform
    const int sid = s_seq[t - t_begin];
    int u = t, need = 0;
    for (; u < t_end && s_seq[u - t_begin] == sid; ++u) need = max(need, min(s_pos[u - t_begin] + 1, s0 + chunk) - s0);
    if (need > 0) {
      // positions [s0, s0 + need) lie in blocks the sequence owns: a row's position is below its reserved length
      __syncthreads();  // the previous run's readers are done with the tile
      constexpr int vec = hd / 4;
      for (int idx = threadIdx.x; idx < need * vec; idx += ATT_THREADS) {
        const int p = idx / vec, c = idx % vec;
        const int64_t off = kv_offset(kv, sid, layer, hkv, s0 + p, w.n_head_kv, hd);
        ((float4*)(kt + p * hd))[c] = ((const float4*)(kv.k + off))[c];
        ((float4*)(vt + p * hd))[c] = ((const float4*)(kv.v + off))[c];
      }
      __syncthreads();
      for (int r = t + warp; r < u; r += nw) {
        const int seq = s_pos[r - t_begin] + 1;
        if (s0 >= seq) continue;
        const int s1 = min(seq, s0 + chunk);
        for (int i = lane; i < gqa * hd; i += 32) sq[i] = q[((int64_t)r * w.n_head + hkv * gqa) * hd + i];
        __syncwarp();
        float* out = part + (((int64_t)r * w.n_head_kv + hkv) * n_split + split) * gqa * (hd + 2);
        attend_slice_warp<GQA, P>(KvTile{kt, vt, s0, hd}, sq, sc, out, s0, s1, chunk);
        __syncwarp();
      }
    }
    t = u;
  }
}

// ---- prompt chunks of one sequence on the tensor cores -----------------------------------------------------------
// Same partial records as the tiled kernel above, for rows of ONE sequence at consecutive positions
// (llr_session_prefill).  A block holds 16 RT rows and one kv head and walks the slices blockIdx.y, blockIdx.y +
// gridDim.y, ... of CH = 8 NT positions; a warp takes one query head of the group and sixteen of the rows.  Queries, keys, values and the
// exponentials are rounded to binary16 when they are staged in shared memory (values transposed, so that two
// consecutive positions of a dimension share a word); scores and weighted sums are m16n8k16 MMAs with f32
// accumulation, maxima, exponentials and their sums are f32.  This is the attention of the 16-bit tensor-core path:
// the automatic path uses it from 64 rows on, next to the 16-bit chunk GEMM and with the same kind of tolerance; the
// f32-faithful path never does.
__device__ __forceinline__ uint32_t pack_h2(float lo, float hi) {
  const __half2 h = __floats2half2_rn(lo, hi);
  return *(const uint32_t*)&h;
}
__device__ __forceinline__ void mma_f16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

template <int GQA, int HD, int NT, int RT>
__global__ void __launch_bounds__(32 * GQA * RT)
attention_tile_mma_kernel(const float* __restrict__ q, KvView kv, float* __restrict__ part, RowMap rows, int layer, WalkShape w, int tokens,
                          int n_split) {
  pdl_enter();
  // strides in 32-bit words (two binary16 each); + 4 words spreads the fragment reads of eight rows over all banks
  constexpr int CH = 8 * NT, KW = HD / 2 + 4, VW = CH / 2 + 4, QW = HD / 2 + 4, PW = CH / 2 + 4, NW = GQA * RT, NTHR = 32 * NW;
  extern __shared__ uint32_t smw[];  // k [CH][KW] | v transposed [HD][VW] | per warp: q [16][QW] | per warp: exponentials [16][PW]
  uint32_t* kt = smw;
  uint32_t* vt = kt + CH * KW;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, t = lane & 3;
  uint32_t* qw = vt + HD * VW + warp * 16 * QW;
  uint32_t* pw = vt + HD * VW + NW * 16 * QW + warp * 16 * PW;
  const int hkv = blockIdx.x, head = warp % GQA;  // a warp: one query head of the group, sixteen of the block's 16 RT rows
  // the last rows first: they attend to the most positions, and the short blocks of the first rows then fill the tail
  const int b_begin = ((int)gridDim.z - 1 - (int)blockIdx.z) * (16 * RT), b_rows = min(tokens - b_begin, 16 * RT);
  const int last_pos = row_position(rows, b_begin) + b_rows - 1;  // of the block: the slices it walks
  if ((int)blockIdx.y * CH > last_pos) return;
  const int t_begin = b_begin + 16 * (warp / GQA), n_rows = max(0, min(tokens - t_begin, 16));
  const int p0 = row_position(rows, b_begin) + 16 * (warp / GQA);  // row r of the warp stands at position p0 + r
  const int sid = row_sequence(rows, b_begin);
  constexpr int vec = HD / 4;
  for (int idx = lane; idx < 16 * vec; idx += 32) {  // this warp's head of the group's rows; rows past the end are zero
    const int r = idx / vec, c = idx % vec;
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (r < n_rows) v = ((const float4*)(q + ((int64_t)(t_begin + r) * w.n_head + hkv * GQA + head) * HD))[c];
    *(uint2*)(qw + r * QW + 2 * c) = make_uint2(pack_h2(v.x, v.y), pack_h2(v.z, v.w));
  }
  const float scale = 1.0f / sqrtf((float)HD);
  // The slices a block walks are merged as they come (running maximum, rescaled sums): one record per row, head and
  // blockIdx.y, at slice index blockIdx.y, instead of one per slice.
  float run_m0 = -CUDART_INF_F, run_m1 = -CUDART_INF_F, run_l0 = 0.f, run_l1 = 0.f;
  float o[HD / 8][4];
#pragma unroll
  for (int nd = 0; nd < HD / 8; ++nd)
#pragma unroll
    for (int i = 0; i < 4; ++i) o[nd][i] = 0.f;
  for (int split = blockIdx.y; split * CH <= last_pos; split += (int)gridDim.y) {
    const int s0 = split * CH;
    // ---- stage the slice: positions no row of the group attends to are zero (their exponentials are zero as well)
    for (int idx = threadIdx.x; idx < CH * vec; idx += NTHR) {
      const int p = idx % CH, c = idx / CH;  // consecutive threads take consecutive positions: the transposed stores of v spread over the banks
      float4 kk = make_float4(0.f, 0.f, 0.f, 0.f), vv = kk;
      if (s0 + p <= last_pos) {
        const int64_t off = kv_offset(kv, sid, layer, hkv, s0 + p, w.n_head_kv, HD);
        kk = ((const float4*)(kv.k + off))[c];
        vv = ((const float4*)(kv.v + off))[c];
      }
      *(uint2*)(kt + p * KW + 2 * c) = make_uint2(pack_h2(kk.x, kk.y), pack_h2(kk.z, kk.w));
      __half* vh = (__half*)vt;
      vh[(4 * c + 0) * (2 * VW) + p] = __float2half_rn(vv.x);
      vh[(4 * c + 1) * (2 * VW) + p] = __float2half_rn(vv.y);
      vh[(4 * c + 2) * (2 * VW) + p] = __float2half_rn(vv.z);
      vh[(4 * c + 3) * (2 * VW) + p] = __float2half_rn(vv.w);
    }
    __syncthreads();
    if (p0 + n_rows - 1 >= s0) {  // warp-uniform: some row of this warp attends to the slice
    // ---- scores: rows g and g + 8 of the group against the slice's positions 8 nt + 2t, + 1
    float sc[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int i = 0; i < 4; ++i) sc[nt][i] = 0.f;
#pragma unroll
    for (int k0 = 0; k0 < HD / 2; k0 += 8) {  // in words: 16 dimensions per step
      const uint32_t a[4] = {qw[g * QW + k0 + t], qw[(g + 8) * QW + k0 + t], qw[g * QW + k0 + t + 4], qw[(g + 8) * QW + k0 + t + 4]};
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        const uint32_t* kr = kt + (8 * nt + g) * KW + k0 + t;
        mma_f16(sc[nt], a, kr[0], kr[4]);
      }
    }
    // ---- scale, causal mask, maximum, exponentials (rounded to binary16, as the MMA below reads them) and their sum
    const int lim0 = p0 + g - s0, lim1 = p0 + g + 8 - s0;  // last slice column rows g / g + 8 attend to
    float m0 = -CUDART_INF_F, m1 = -CUDART_INF_F;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const int col = 8 * nt + 2 * t + j;
        sc[nt][j] = (g < n_rows && col <= lim0) ? __fmul_rn(sc[nt][j], scale) : -CUDART_INF_F;
        sc[nt][2 + j] = (g + 8 < n_rows && col <= lim1) ? __fmul_rn(sc[nt][2 + j], scale) : -CUDART_INF_F;
        m0 = fmaxf(m0, sc[nt][j]);
        m1 = fmaxf(m1, sc[nt][2 + j]);
      }
    m0 = fmaxf(m0, __shfl_xor_sync(~0u, m0, 1)); m0 = fmaxf(m0, __shfl_xor_sync(~0u, m0, 2));
    m1 = fmaxf(m1, __shfl_xor_sync(~0u, m1, 1)); m1 = fmaxf(m1, __shfl_xor_sync(~0u, m1, 2));
    // what the earlier slices left is rescaled to the new maximum (a row that has attended to nothing yet keeps zeros)
    m0 = fmaxf(m0, run_m0);
    m1 = fmaxf(m1, run_m1);
    const float a0 = run_m0 == -CUDART_INF_F ? 0.f : expf(run_m0 - m0), a1 = run_m1 == -CUDART_INF_F ? 0.f : expf(run_m1 - m1);
    run_m0 = m0;
    run_m1 = m1;
#pragma unroll
    for (int nd = 0; nd < HD / 8; ++nd) { o[nd][0] *= a0; o[nd][1] *= a0; o[nd][2] *= a1; o[nd][3] *= a1; }
    float l0 = 0.f, l1 = 0.f;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      float e[4];
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        e[j] = sc[nt][j] == -CUDART_INF_F ? 0.f : expf(sc[nt][j] - m0);
        e[2 + j] = sc[nt][2 + j] == -CUDART_INF_F ? 0.f : expf(sc[nt][2 + j] - m1);
      }
      const __half2 h0 = __floats2half2_rn(e[0], e[1]), h1 = __floats2half2_rn(e[2], e[3]);
      l0 += __low2float(h0) + __high2float(h0);  // the sum of what the weighted sum below uses
      l1 += __low2float(h1) + __high2float(h1);
      pw[g * PW + 4 * nt + t] = *(const uint32_t*)&h0;
      pw[(g + 8) * PW + 4 * nt + t] = *(const uint32_t*)&h1;
    }
    l0 += __shfl_xor_sync(~0u, l0, 1); l0 += __shfl_xor_sync(~0u, l0, 2);
    l1 += __shfl_xor_sync(~0u, l1, 1); l1 += __shfl_xor_sync(~0u, l1, 2);
    run_l0 = fmaf(run_l0, a0, l0);
    run_l1 = fmaf(run_l1, a1, l1);
    __syncwarp();
    // ---- weighted value rows: dimensions 8 nd + 2t, + 1 of rows g and g + 8, added to the rescaled sums
#pragma unroll
    for (int k0 = 0; k0 < CH / 2; k0 += 8) {  // in words: 16 positions per step
      const uint32_t a[4] = {pw[g * PW + k0 + t], pw[(g + 8) * PW + k0 + t], pw[g * PW + k0 + t + 4], pw[(g + 8) * PW + k0 + t + 4]};
#pragma unroll
      for (int nd = 0; nd < HD / 8; ++nd) {
        const uint32_t* vr = vt + (8 * nd + g) * VW + k0 + t;
        mma_f16(o[nd], a, vr[0], vr[4]);
      }
    }
    }
    __syncthreads();  // every warp is done with the slice before the next one is staged
  }
  // ---- one record per row: HD sums, the maximum, the sum of exponentials.  A row whose position lies before this
  // block's first slice has none, and the merge does not look for one: it reads min(slices of the row, gridDim.y) records.
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int r = g + 8 * half;
    if (r >= n_rows || p0 + r < (int)blockIdx.y * CH) continue;
    float* out = part + ((((int64_t)(t_begin + r) * w.n_head_kv + hkv) * n_split + blockIdx.y) * GQA + head) * (HD + 2);
#pragma unroll
    for (int nd = 0; nd < HD / 8; ++nd) *(float2*)(out + 8 * nd + 2 * t) = make_float2(o[nd][2 * half], o[nd][2 * half + 1]);
    if (t == 0) { out[HD] = half ? run_m1 : run_m0; out[HD + 1] = half ? run_l1 : run_l0; }
  }
}

// grid (query heads / 4, token), one warp per query head: merges the position slices (at most 32).  Lane sp turns
// slice sp's maximum into the weight exp(m_slice - m); the denominator is the shuffle-tree sum of the weighted slice
// sums; then every lane adds its dimensions over the slices in ascending order, the weights coming by shuffle.
__global__ void __launch_bounds__(128)
attention_combine_kernel(const float* __restrict__ part, float* __restrict__ out, RowMap rows, int chunk, WalkShape w, int heads_per_block,
                         int max_records, int record_chunk) {
  pdl_enter();
  // heads_per_block 4: one warp per head (many rows: fewer, fuller blocks); 1: the four warps share a head's
  // dimensions (a decode step has few blocks to fill the device with)
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int hq = heads_per_block == 4 ? blockIdx.x * 4 + warp : blockIdx.x, t = blockIdx.y;
  if (hq >= w.n_head) return;
  const int d0 = heads_per_block == 4 ? lane : lane + 32 * warp, dstep = heads_per_block == 4 ? 32 : 128;
  const int hd = w.head_dim, gqa = w.n_head / w.n_head_kv;
  const int hkv = hq / gqa, g = hq % gqa;
  const int seq = row_position(rows, t) + 1;
  // chunk: positions per slice of the f32 kernels, which fixes the room a row's records take.  The tensor-core kernel
  // walks slices of record_chunk positions of its own and leaves one record per walked run of slices, at the first
  // max_records indices.
  const int n_split = (w.n_ctx + chunk - 1) / chunk, used = min(min(n_split, (seq + record_chunk - 1) / record_chunk), max_records);
  const float* base = part + ((int64_t)t * w.n_head_kv + hkv) * n_split * gqa * (hd + 2) + g * (hd + 2);
  const int64_t stride = (int64_t)gqa * (hd + 2);
  const float ms = lane < used ? base[lane * stride + hd] : -CUDART_INF_F;
  const float m = warp_max(ms);
  const float e = lane < used ? expf(ms - m) : 0.f;
  const float l = warp_sum(lane < used ? base[lane * stride + hd + 1] * e : 0.f);
  float acc[8];  // head_dim <= 256: up to eight dimensions per lane, all in flight at once
#pragma unroll
  for (int k = 0; k < 8; ++k) acc[k] = 0.f;
  for (int sp0 = 0; sp0 < used; sp0 += 4) {  // four slices' records are fetched before the first is used
    float v[4][8];
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int k = 0; k < 8; ++k) v[j][k] = (sp0 + j < used && d0 + dstep * k < hd) ? base[(sp0 + j) * stride + d0 + dstep * k] : 0.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float es = __shfl_sync(0xffffffffu, e, (sp0 + j) & 31);
      if (sp0 + j < used) {
#pragma unroll
        for (int k = 0; k < 8; ++k)
          if (d0 + dstep * k < hd) acc[k] = fmaf(v[j][k], es, acc[k]);
      }
    }
  }
#pragma unroll
  for (int k = 0; k < 8; ++k)
    if (d0 + dstep * k < hd) out[((int64_t)t * w.n_head + hq) * hd + d0 + dstep * k] = l > 0.f ? __fdiv_rn(acc[k], l) : 0.f;
}

__device__ __forceinline__ float swiglu_of(float a, float b) { return __fmul_rn(__fdiv_rn(a, 1.0f + expf(-a)), b); }  // silu(gate) * up (decode.rs:11826, :2984)
__global__ void swiglu_kernel(float* __restrict__ g, const float* __restrict__ u, int64_t n) {
  pdl_enter();
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) g[i] = swiglu_of(g[i], u[i]);
}
// the same, four elements per thread and step (n4 = n / 4; g and u 16-byte aligned)
__global__ void swiglu4_kernel(float4* __restrict__ g, const float4* __restrict__ u, int64_t n4) {
  pdl_enter();
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (int64_t)gridDim.x * blockDim.x) {
    const float4 a = g[i], b = u[i];
    g[i] = make_float4(swiglu_of(a.x, b.x), swiglu_of(a.y, b.y), swiglu_of(a.z, b.z), swiglu_of(a.w, b.w));
  }
}
__global__ void add_kernel(float* __restrict__ x, const float* __restrict__ y, int64_t n) {
  pdl_enter();
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
    x[i] = __fadd_rn(y[i], x[i]);
}

// one block: index of the first strict maximum (sample.rs:293: `v > best` scanning upwards, so ties go to the
// lower index), its margin over the largest other value, and the position counter advanced for the next step
__global__ void __launch_bounds__(1024)
argmax_kernel(const float* __restrict__ logits, int n, int* __restrict__ out_id, float* __restrict__ out_margin,
              int* __restrict__ pos_dev, int advance, int* __restrict__ count_dev) {
  pdl_enter();
  // with count_dev: out_id[0] is the slot the next step reads its token from, and the token and its margin are also
  // appended at out_id[1 + *count_dev] / out_margin[*count_dev]: every step of a generation is then the same launch
  const int slot = count_dev ? *count_dev : 0;
  logits += (int64_t)blockIdx.x * n;  // one block per row of logits (a single row unless launch_argmax_rows)
  out_id += blockIdx.x;
  if (out_margin) out_margin += blockIdx.x;
  __shared__ float sv[32];
  __shared__ int si[32];
  __shared__ int s_best;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  if (n > 0) {
    float best = -CUDART_INF_F;
    int bi = 0x7fffffff;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
      const float v = logits[i];
      if (v > best) { best = v; bi = i; }  // ascending i per thread: the first of equal values stays
    }
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(~0u, best, o);
      const int oi = __shfl_xor_sync(~0u, bi, o);
      if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; }
    }
    if (lane == 0) { sv[warp] = best; si[warp] = bi; }
    __syncthreads();
    if (warp == 0) {
      best = lane < nw ? sv[lane] : -CUDART_INF_F;
      bi = lane < nw ? si[lane] : 0x7fffffff;
      for (int o = 16; o > 0; o >>= 1) {
        const float ob = __shfl_xor_sync(~0u, best, o);
        const int oi = __shfl_xor_sync(~0u, bi, o);
        if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; }
      }
      if (lane == 0) s_best = bi == 0x7fffffff ? 0 : bi;  // all NaN or -inf: index 0, as the reference's scan leaves it
    }
    __syncthreads();
    const int win = s_best;
    if (out_margin) {
      float second = -CUDART_INF_F;
      for (int i = threadIdx.x; i < n; i += blockDim.x)
        if (i != win) second = fmaxf(second, logits[i]);
      second = warp_max(second);
      __syncthreads();
      if (lane == 0) sv[warp] = second;
      __syncthreads();
      if (threadIdx.x == 0) {
        float m = -CUDART_INF_F;
        for (int w = 0; w < nw; ++w) m = fmaxf(m, sv[w]);
        out_margin[slot] = logits[win] - m;
      }
    }
    if (threadIdx.x == 0) {
      out_id[0] = win;
      if (count_dev) { out_id[1 + slot] = win; *count_dev = slot + 1; }
    }
  }
  if (threadIdx.x == 0 && pos_dev) *pos_dev += advance;
}

// Two-stage argmax of one long row (a vocabulary): ARG_BLOCKS blocks each reduce a contiguous range to (best value, its
// first index, largest other value of the range); one block merges the ranges in ascending order, so the first of equal
// maxima still wins (sample.rs:293), and applies the bookkeeping of argmax_kernel.
constexpr int ARG_BLOCKS = 128;
__global__ void __launch_bounds__(256)
argmax_part_kernel(const float* __restrict__ logits, int n, float* __restrict__ pbest, int* __restrict__ pidx, float* __restrict__ psecond) {
  pdl_enter();
  __shared__ float sv[8], s2[8];
  __shared__ int si[8];
  const int per = (n + gridDim.x - 1) / gridDim.x;
  const int lo = blockIdx.x * per, hi = min(n, lo + per);
  float best = -CUDART_INF_F, second = -CUDART_INF_F;
  int bi = 0x7fffffff;
  for (int i = lo + threadIdx.x; i < hi; i += blockDim.x) {
    const float v = logits[i];
    if (v > best) { second = best; best = v; bi = i; }
    else second = fmaxf(second, v);
  }
  // merge (best, index, second) of two disjoint sets: the larger best wins, ties to the lower index; the loser's best
  // and both seconds compete for second place
  auto merge = [](float& b, int& i, float& s, float ob, int oi, float os) {
    const bool other = ob > b || (ob == b && oi < i);
    const float loser = other ? b : ob;
    s = fmaxf(fmaxf(s, os), loser);
    if (other) { b = ob; i = oi; }
  };
  for (int o = 16; o > 0; o >>= 1) {
    const float ob = __shfl_xor_sync(~0u, best, o), os = __shfl_xor_sync(~0u, second, o);
    const int oi = __shfl_xor_sync(~0u, bi, o);
    merge(best, bi, second, ob, oi, os);
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) { sv[warp] = best; si[warp] = bi; s2[warp] = second; }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < (int)(blockDim.x >> 5); ++w) merge(best, bi, second, sv[w], si[w], s2[w]);
    pbest[blockIdx.x] = best; pidx[blockIdx.x] = bi; psecond[blockIdx.x] = second;
  }
}
__global__ void __launch_bounds__(ARG_BLOCKS)
argmax_merge_kernel(const float* __restrict__ pbest, const int* __restrict__ pidx, const float* __restrict__ psecond, int parts,
                    int* __restrict__ out_id, float* __restrict__ out_margin, int* __restrict__ pos_dev, int advance,
                    int* __restrict__ count_dev) {
  pdl_enter();
  if (threadIdx.x != 0) return;  // a hundred-odd triples: one thread, ascending order
  float best = -CUDART_INF_F, second = -CUDART_INF_F;
  int bi = 0x7fffffff;
  for (int p = 0; p < parts; ++p) {
    const float ob = pbest[p], os = psecond[p];
    const int oi = pidx[p];
    const bool other = ob > best || (ob == best && oi < bi);
    const float loser = other ? best : ob;
    second = fmaxf(fmaxf(second, os), loser);
    if (other) { best = ob; bi = oi; }
  }
  const int win = bi == 0x7fffffff ? 0 : bi;
  const int slot = count_dev ? *count_dev : 0;
  out_id[0] = win;
  if (out_margin) out_margin[slot] = best - second;
  if (count_dev) { out_id[1 + slot] = win; *count_dev = slot + 1; }
  if (pos_dev) *pos_dev += advance;
}

// positions per attention slice: 32, or a thirty-second of the context when that is longer
int attention_chunk(const WalkShape& w) {
  const int c = (w.n_ctx + 31) / 32;
  return c > 32 ? c : 32;
}
int attention_splits(const WalkShape& w) {
  const int c = attention_chunk(w);
  return (w.n_ctx + c - 1) / c;
}

// LLR_WALK_PDL=0 launches these kernels in plain stream order
bool walk_pdl() {
  static const bool on = [] { const char* v = std::getenv("LLR_WALK_PDL"); return !(v && v[0] == '0'); }();
  return on;
}
template <typename... P, typename... A>
cudaError_t launch_walk(void (*kern)(P...), dim3 grid, dim3 block, size_t smem, cudaStream_t s, A... args) {
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr.val.programmaticStreamSerializationAllowed = 1;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cfg.attrs = &attr;
  cfg.numAttrs = walk_pdl() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kern, static_cast<P>(args)...);
}

}  // namespace

cudaError_t launch_rmsnorm(float* x, const float* add, const float* w, float* y, int tokens, int n, float eps,
                           cudaStream_t s, uint64_t* launches) {
  if (tokens <= 0) return cudaSuccess;
  if (launches) ++*launches;
  return launch_walk(rmsnorm_kernel, dim3(tokens), dim3(NORM_THREADS), 0, s, x, add, w, y, n, eps);
}

cudaError_t launch_rope_store(float* q, float* k, const float* v, const KvView& kv, const RowMap& rows, int tokens, int layer,
                              const WalkShape& w, cudaStream_t s, uint64_t* launches) {
  if (tokens <= 0) return cudaSuccess;
  if (launches) ++*launches;
  return launch_walk(rope_store_kernel, dim3(tokens), dim3(256), 0, s, q, k, v, kv, rows, layer, w);
}

size_t attention_scratch_floats(int tokens, const WalkShape& w) {
  return (size_t)tokens * w.n_head_kv * attention_splits(w) * (w.n_head / w.n_head_kv) * (w.head_dim + 2);
}

cudaError_t launch_attention(const float* q, const KvView& kv, float* out, float* scratch, const RowMap& rows, int tokens,
                             int layer, const WalkShape& w, cudaStream_t s, uint64_t* launches, const float* k_new, const float* v_new,
                             bool tensor_cores, bool one_sequence) {
  if (tokens <= 0) return cudaSuccess;
  const int gqa = w.n_head / w.n_head_kv;
  if (gqa < 1 || gqa > ATT_MAX_GQA || w.n_head % w.n_head_kv != 0 || w.head_dim > ATT_THREADS) return cudaErrorInvalidValue;
  const int splits = attention_splits(w);
  const int max_chunk = attention_chunk(w);
  const size_t groups = ATT_THREADS / w.head_dim > 0 ? ATT_THREADS / w.head_dim : 1;
  const size_t score_floats = (size_t)gqa * max_chunk > groups * gqa * w.head_dim ? (size_t)gqa * max_chunk : groups * gqa * w.head_dim;
  const size_t smem = ((size_t)gqa * w.head_dim + score_floats + 32) * sizeof(float);
  if (smem > 200 * 1024) return cudaErrorInvalidValue;
  static PerDevice configured;  // largest size the kernel has been allowed on this device
  std::atomic<int>& allowed = configured.here();
  if (smem > 48 * 1024 && (int)smem > allowed.load(std::memory_order_relaxed)) {
    cudaError_t e = cudaFuncSetAttribute(attention_partial_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    allowed.store((int)smem, std::memory_order_relaxed);
  }
  if (launches) *launches += 2;
  cudaError_t e;
  // prompt chunks: rows of a group share the slice's keys and values through a shared-memory tile
  const size_t tile_smem = (2 * (size_t)max_chunk * w.head_dim + (ATT_THREADS / 32) * ((size_t)gqa * w.head_dim + (size_t)gqa * max_chunk)) * sizeof(float);
  void (*tile)(const float*, KvView, float*, RowMap, int, int, WalkShape, int) = nullptr;
#define LLR_TILE(G, PP) if (gqa == G && w.head_dim == ATT_THREADS / PP) tile = attention_tile_kernel<G, PP>;
  LLR_TILE(1, 1) LLR_TILE(2, 1) LLR_TILE(4, 1) LLR_TILE(1, 2) LLR_TILE(2, 2) LLR_TILE(4, 2) LLR_TILE(8, 2)
  LLR_TILE(1, 4) LLR_TILE(2, 4) LLR_TILE(4, 4) LLR_TILE(8, 4)
#undef LLR_TILE
  // a prompt chunk of one sequence at consecutive positions, when the caller allows 16-bit operands: tensor cores
  void (*mma)(const float*, KvView, float*, RowMap, int, WalkShape, int, int) = nullptr;
  size_t mma_smem = 0;
  int mma_rt = 1;
  // its slices are its own (64 positions; 32 when the context is short): the records it leaves do not depend on max_chunk
  const int mma_chunk = w.n_ctx > 1024 ? 64 : 32;
  if (tensor_cores && (one_sequence || (!rows.row_pos && !rows.row_seq)) && tokens >= 64 && (w.head_dim == 64 || w.head_dim == 128)) {
#define LLR_MMA(G, H, N) if (gqa == G && w.head_dim == H && mma_chunk == 8 * N) mma = attention_tile_mma_kernel<G, H, N, (G <= 4 ? 4 : 2)>;
    LLR_MMA(1, 64, 4) LLR_MMA(2, 64, 4) LLR_MMA(4, 64, 4) LLR_MMA(8, 64, 4) LLR_MMA(1, 64, 8) LLR_MMA(2, 64, 8) LLR_MMA(4, 64, 8) LLR_MMA(8, 64, 8)
    LLR_MMA(1, 128, 4) LLR_MMA(2, 128, 4) LLR_MMA(4, 128, 4) LLR_MMA(8, 128, 4) LLR_MMA(1, 128, 8) LLR_MMA(2, 128, 8) LLR_MMA(4, 128, 8) LLR_MMA(8, 128, 8)
#undef LLR_MMA
    mma_rt = gqa <= 4 ? 4 : 2;  // sixteen-row tiles per block
    mma_smem = ((size_t)mma_chunk * (w.head_dim / 2 + 4) + (size_t)w.head_dim * (mma_chunk / 2 + 4) +
                (size_t)gqa * mma_rt * 16 * (w.head_dim / 2 + 4 + mma_chunk / 2 + 4)) * sizeof(uint32_t);
  }
  int max_records = splits, record_chunk = max_chunk;
  if (mma && mma_smem <= 200 * 1024) {
    const int mma_splits = (w.n_ctx + mma_chunk - 1) / mma_chunk;
    max_records = std::min(std::min(mma_splits, splits), 4);
    record_chunk = mma_chunk;
    if (mma_smem > 48 * 1024) {
      e = cudaFuncSetAttribute((const void*)mma, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)mma_smem);
      if (e != cudaSuccess) return e;
    }
    e = launch_walk(mma, dim3(w.n_head_kv, max_records, (tokens + 16 * mma_rt - 1) / (16 * mma_rt)), dim3(32 * gqa * mma_rt), mma_smem,
                    s, q, kv, scratch, rows, layer, w, tokens, splits);
  } else if (tile && tokens >= 4 && max_chunk <= ATT_TILE_CHUNK && tile_smem <= 200 * 1024) {
    if (tile_smem > 48 * 1024) {
      e = cudaFuncSetAttribute((const void*)tile, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)tile_smem);
      if (e != cudaSuccess) return e;
    }
    e = launch_walk(tile, dim3(w.n_head_kv, splits, (tokens + ATT_ROWS - 1) / ATT_ROWS), dim3(ATT_THREADS), tile_smem, s, q, kv, scratch,
                    rows, layer, max_chunk, w, tokens);
  } else {
    e = launch_walk(attention_partial_kernel, dim3(w.n_head_kv, splits, tokens), dim3(ATT_THREADS), smem, s, q, kv, scratch, rows, layer,
                    max_chunk, w, tokens == 1 ? k_new : (const float*)nullptr, tokens == 1 ? v_new : (const float*)nullptr);
  }
  if (e != cudaSuccess) return e;
  return launch_walk(attention_combine_kernel, dim3(tokens >= 16 ? (w.n_head + 3) / 4 : w.n_head, tokens), dim3(128), 0, s, (const float*)scratch, out, rows,
                     max_chunk, w, tokens >= 16 ? 4 : 1, max_records, record_chunk);
}

cudaError_t launch_swiglu(float* g, const float* u, int64_t n, cudaStream_t s, uint64_t* launches) {
  if (n <= 0) return cudaSuccess;
  int64_t blocks = (n + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  if (launches) ++*launches;
  if (n % 4 == 0 && (((uintptr_t)g | (uintptr_t)u) & 15) == 0) {
    int64_t b4 = (n / 4 + 255) / 256;
    if (b4 > 148 * 8) b4 = 148 * 8;
    return launch_walk(swiglu4_kernel, dim3((unsigned)b4), dim3(256), 0, s, (float4*)g, (const float4*)u, n / 4);
  }
  return launch_walk(swiglu_kernel, dim3((unsigned)blocks), dim3(256), 0, s, g, u, n);
}

cudaError_t launch_add(float* x, const float* y, int64_t n, cudaStream_t s, uint64_t* launches) {
  if (n <= 0) return cudaSuccess;
  int64_t blocks = (n + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  if (launches) ++*launches;
  return launch_walk(add_kernel, dim3((unsigned)blocks), dim3(256), 0, s, x, y, n);
}

cudaError_t launch_argmax_rows(const float* logits, int n_rows, int n, int* out_id, float* out_margin, cudaStream_t s,
                               uint64_t* launches) {
  if (n_rows <= 0) return cudaSuccess;
  if (launches) ++*launches;
  return launch_walk(argmax_kernel, dim3(n_rows), dim3(1024), 0, s, logits, n, out_id, out_margin, (int*)nullptr, 0, (int*)nullptr);
}

cudaError_t launch_argmax_advance(const float* logits, int n, int* out_id, float* out_margin, int* pos_dev, int advance,
                                  int* count_dev, float* part, cudaStream_t s, uint64_t* launches) {
  if (n >= 16384 && part) {  // a vocabulary: spread the scan over the device (part: 3 * ARG_BLOCKS words of scratch)
    if (launches) *launches += 2;
    cudaError_t e = launch_walk(argmax_part_kernel, dim3(ARG_BLOCKS), dim3(256), 0, s, logits, n, part, (int*)(part + ARG_BLOCKS), part + 2 * ARG_BLOCKS);
    if (e != cudaSuccess) return e;
    return launch_walk(argmax_merge_kernel, dim3(1), dim3(ARG_BLOCKS), 0, s, (const float*)part, (const int*)(part + ARG_BLOCKS),
                       (const float*)(part + 2 * ARG_BLOCKS), (int)ARG_BLOCKS, out_id, out_margin, pos_dev, advance, count_dev);
  }
  if (launches) ++*launches;
  return launch_walk(argmax_kernel, dim3(1), dim3(1024), 0, s, logits, n, out_id, out_margin, pos_dev, advance, count_dev);
}

}  // namespace llr
