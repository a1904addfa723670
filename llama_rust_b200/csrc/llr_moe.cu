// Routed-expert FFN layer: the small kernels around the expert matrix products.
//
// Follows langtax/src/decode.rs: grouped_one_expert :10062 gathers the rows routed to an
// expert into a packed activation matrix, swiglu_expert_gemm :10148 runs gate and up
// products, silu(g) * u (silu_inplace :11826), the down product, and
// scatter_expert_rows :10263 adds y * w into the layer output.  The output of a token is
// accumulated over its experts in ascending expert id, starting from zero, which fixes
// the f32 rounding order exactly as the reference's `for e in 0..n_expert` loop does.
#include "llr_kernels.cuh"

namespace llr {
namespace {

__global__ void gather_rows_kernel(const float* __restrict__ x, const int* __restrict__ tok_of_row,
                                   float* __restrict__ packed, int n_rows, int n_embd) {
  const int row = blockIdx.x;
  if (row >= n_rows) return;
  const float4* src = (const float4*)(x + (int64_t)tok_of_row[row] * n_embd);
  float4* dst = (float4*)(packed + (int64_t)row * n_embd);
  for (int i = threadIdx.x; i < n_embd / 4; i += blockDim.x) dst[i] = src[i];
}

// Router logits for an F32 router (ffn_gate_inp, decode.rs:9977): a matrix with a handful of rows
// against every token.  One CTA per token, one warp per expert (striding when there are more
// experts than warps), f32 FMA over float4 loads, warp-shuffle reduction.  The general decode
// kernels are built for thousands of rows and leave the GPU idle on eight.
__global__ void router_logits_kernel(const float* __restrict__ w, const float* __restrict__ x, float* __restrict__ logits,
                                     int n_expert, int n_embd) {
  const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarp = blockDim.x >> 5;
  const float4* xr = (const float4*)(x + (int64_t)t * n_embd);
  for (int e = warp; e < n_expert; e += nwarp) {
    const float4* wr = (const float4*)(w + (int64_t)e * n_embd);
    float acc = 0.0f;
    for (int i = lane; i < n_embd / 4; i += 32) {
      const float4 a = __ldg(wr + i), b = xr[i];
      acc = fmaf(a.x, b.x, acc); acc = fmaf(a.y, b.y, acc); acc = fmaf(a.z, b.z, acc); acc = fmaf(a.w, b.w, acc);
    }
#pragma unroll
    for (int o = 16; o; o >>= 1) acc += __shfl_xor_sync(~0u, acc, o);
    if (lane == 0) logits[(int64_t)t * n_expert + e] = acc;
  }
}

__global__ void silu_mul_kernel(float* __restrict__ g, const float* __restrict__ u, int64_t n) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    const float v = g[i];
    g[i] = (v / (1.0f + expf(-v))) * u[i];
  }
}

// the same, four elements per thread and pass (both arrays 16-byte aligned, n4 = n / 4)
__global__ void silu_mul4_kernel(float4* __restrict__ g, const float4* __restrict__ u, int64_t n4) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (int64_t)gridDim.x * blockDim.x) {
    float4 v = g[i];
    const float4 w = __ldg(u + i);
    v.x = (v.x / (1.0f + expf(-v.x))) * w.x;
    v.y = (v.y / (1.0f + expf(-v.y))) * w.y;
    v.z = (v.z / (1.0f + expf(-v.z))) * w.z;
    v.w = (v.w / (1.0f + expf(-v.w))) * w.w;
    g[i] = v;
  }
}

// rows_of_tok[t*n_used + j]: packed row of token t's j-th selection, selections ordered by
// ascending expert id; w_of_tok the matching router weights.
__global__ void scatter_combine_kernel(const float* __restrict__ y, const int* __restrict__ rows_of_tok,
                                       const float* __restrict__ w_of_tok, float* __restrict__ out,
                                       int tokens, int n_used, int n_embd) {
  const int t = blockIdx.x;
  if (t >= tokens) return;
  for (int c = threadIdx.x; c < n_embd; c += blockDim.x) {
    float acc = 0.0f;
    for (int j = 0; j < n_used; ++j) {
      const float term = __fmul_rn(y[(int64_t)rows_of_tok[t * n_used + j] * n_embd + c], w_of_tok[t * n_used + j]);
      acc = __fadd_rn(acc, term);
    }
    out[(int64_t)t * n_embd + c] = acc;
  }
}

// Routing of one token per thread, in place on its row of router logits, exactly the reference's sequence
// (route_softmax_tokens decode.rs:9969: softmax :12021 with a sequential sum, topk_into :11363 with ties to the
// lower id, fill_router_weights :11392 with the 2^-14 clamp :321).  ids / wts: n_used per token, in top-k order.
__global__ void route_kernel(float* __restrict__ logits, int tokens, int n_expert, int n_used, int norm_w,
                             int* __restrict__ ids, float* __restrict__ wts) {
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= tokens) return;
  float* row = logits + (int64_t)t * n_expert;
  float mx = -INFINITY;
  for (int i = 0; i < n_expert; ++i) mx = fmaxf(mx, row[i]);
  float sum = 0.0f;
  for (int i = 0; i < n_expert; ++i) { const float e = expf(row[i] - mx); row[i] = e; sum = __fadd_rn(sum, e); }
  if (sum > 0.0f) for (int i = 0; i < n_expert; ++i) row[i] = __fdiv_rn(row[i], sum);
  float wsum = 0.0f;
  for (int j = 0; j < n_used; ++j) {
    int best = -1;
    float bv = 0.0f;
    for (int i = 0; i < n_expert; ++i) {
      const float v = row[i];
      if (v == -1.0f) continue;  // taken (probabilities are never negative)
      if (best < 0 || v > bv) { best = i; bv = v; }
    }
    ids[t * n_used + j] = best;
    wts[t * n_used + j] = bv;
    wsum = __fadd_rn(wsum, bv);
    row[best] = -1.0f;
  }
  if (norm_w) {
    if (wsum < 1.0f / 16384.0f) wsum = 1.0f / 16384.0f;
    for (int j = 0; j < n_used; ++j) wts[t * n_used + j] = __fdiv_rn(wts[t * n_used + j], wsum);
  }
}

// Packed row order of the grouped FFN (grouped_routed_ffn decode.rs:10006): experts ascending, tokens ascending
// inside an expert.  One block; deterministic (prefix sums, no atomics).  first_row[e] = first packed row of expert e
// (n_expert + 1 entries), tok_of_row[r] = token of packed row r, rows_of_tok / w_of_tok[t*n_used + slot] = row and router
// weight of token t's slot-th expert in ascending expert id (the accumulation order of scatter_expert_rows :10263);
// the weight of an expert that is not resident here (local[e] == 0) is zero.  fill: tokens ints of scratch.
__global__ void __launch_bounds__(1024)
bucket_kernel(const int* __restrict__ ids, const float* __restrict__ wts, const unsigned char* __restrict__ local, int tokens,
              int n_expert, int n_used, int* __restrict__ first_row, int* __restrict__ tok_of_row, int* __restrict__ rows_of_tok,
              float* __restrict__ w_of_tok, int* __restrict__ fill) {
  __shared__ int warp_tot[32];
  __shared__ int s_base;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int t = threadIdx.x; t < tokens; t += blockDim.x) fill[t] = 0;
  if (threadIdx.x == 0) s_base = 0;
  __syncthreads();
  for (int e = 0; e < n_expert; ++e) {
    if (threadIdx.x == 0) first_row[e] = s_base;
    for (int t0 = 0; t0 < tokens; t0 += blockDim.x) {
      const int t = t0 + threadIdx.x;
      int slot_j = -1;
      if (t < tokens)
        for (int j = 0; j < n_used; ++j)
          if (ids[t * n_used + j] == e) { slot_j = j; break; }
      const unsigned mask = __ballot_sync(~0u, slot_j >= 0);
      if (lane == 0) warp_tot[warp] = __popc(mask);
      __syncthreads();
      int before = 0;
      for (int w = 0; w < warp; ++w) before += warp_tot[w];
      int total = 0;
      for (int w = 0; w < (int)(blockDim.x >> 5); ++w) total += warp_tot[w];
      const int base = s_base;
      if (slot_j >= 0) {
        const int r = base + before + __popc(mask & ((1u << lane) - 1u));
        tok_of_row[r] = t;
        const int slot = fill[t]++;
        rows_of_tok[t * n_used + slot] = r;
        w_of_tok[t * n_used + slot] = local[e] ? wts[t * n_used + slot_j] : 0.0f;
      }
      __syncthreads();
      if (threadIdx.x == 0) s_base = base + total;
      __syncthreads();
    }
  }
  if (threadIdx.x == 0) first_row[n_expert] = s_base;
}

// One token's selection in ascending expert id (the order scatter_expert_rows :10263 adds in), for the products whose
// matrix is chosen on the device.  n_used <= 8; one thread.
__global__ void select_sorted_kernel(const int* __restrict__ ids, const float* __restrict__ wts, int n_used, int* __restrict__ sel,
                                     float* __restrict__ selw) {
  asm volatile("griddepcontrol.wait;" ::: "memory");
  if (threadIdx.x != 0) return;
  int id[8];
  float w[8];
  for (int j = 0; j < n_used; ++j) { id[j] = ids[j]; w[j] = wts[j]; }
  for (int a = 1; a < n_used; ++a)  // insertion sort: ids of one token are distinct
    for (int b = a; b > 0 && id[b - 1] > id[b]; --b) {
      const int ti = id[b]; id[b] = id[b - 1]; id[b - 1] = ti;
      const float tw = w[b]; w[b] = w[b - 1]; w[b - 1] = tw;
    }
  for (int j = 0; j < n_used; ++j) { sel[j] = id[j]; selw[j] = w[j]; }
}

// out[c] = sum over the selected experts, in the order given, of y[j][c] * w[j]: product rounded, then added, from zero
// (what scatter_combine_kernel does for a packed batch)
__global__ void combine_one_kernel(const float* __restrict__ y, const float* __restrict__ selw, float* __restrict__ out, int n_used,
                                   int n_embd) {
  asm volatile("griddepcontrol.wait;" ::: "memory");
  for (int c = blockIdx.x * blockDim.x + threadIdx.x; c < n_embd; c += gridDim.x * blockDim.x) {
    float acc = 0.0f;
    for (int j = 0; j < n_used; ++j) acc = __fadd_rn(acc, __fmul_rn(y[(int64_t)j * n_embd + c], selw[j]));
    out[c] = acc;
  }
}

}  // namespace

cudaError_t launch_select_sorted(const int* ids, const float* wts, int n_used, int* sel, float* selw, cudaStream_t s, uint64_t* launches) {
  if (n_used < 1 || n_used > 8) return cudaErrorInvalidValue;
  select_sorted_kernel<<<1, 32, 0, s>>>(ids, wts, n_used, sel, selw);
  if (launches) ++*launches;
  return cudaGetLastError();
}

cudaError_t launch_combine_one(const float* y, const float* selw, float* out, int n_used, int n_embd, cudaStream_t s, uint64_t* launches) {
  combine_one_kernel<<<(n_embd + 255) / 256, 256, 0, s>>>(y, selw, out, n_used, n_embd);
  if (launches) ++*launches;
  return cudaGetLastError();
}

cudaError_t launch_route(float* logits, int tokens, int n_expert, int n_used, int norm_w, int* ids, float* wts,
                         cudaStream_t s, uint64_t* launches) {
  if (tokens <= 0) return cudaSuccess;
  route_kernel<<<(tokens + 127) / 128, 128, 0, s>>>(logits, tokens, n_expert, n_used, norm_w, ids, wts);
  if (launches) ++*launches;
  return cudaGetLastError();
}

cudaError_t launch_bucket(const int* ids, const float* wts, const unsigned char* local, int tokens, int n_expert, int n_used,
                          int* first_row, int* tok_of_row, int* rows_of_tok, float* w_of_tok, int* fill, cudaStream_t s,
                          uint64_t* launches) {
  if (tokens <= 0) return cudaSuccess;
  bucket_kernel<<<1, 1024, 0, s>>>(ids, wts, local, tokens, n_expert, n_used, first_row, tok_of_row, rows_of_tok, w_of_tok, fill);
  if (launches) ++*launches;
  return cudaGetLastError();
}

cudaError_t launch_gather_rows(const float* x, const int* tok_of_row, float* packed, int n_rows, int n_embd,
                               cudaStream_t s, uint64_t* launches) {
  if (n_rows <= 0) return cudaSuccess;
  gather_rows_kernel<<<n_rows, 256, 0, s>>>(x, tok_of_row, packed, n_rows, n_embd);
  if (launches) ++*launches;
  return cudaGetLastError();
}

cudaError_t launch_router_logits(const float* w, const float* x, float* logits, int tokens, int n_expert, int n_embd,
                                 cudaStream_t s, uint64_t* launches) {
  router_logits_kernel<<<(unsigned)tokens, 256, 0, s>>>(w, x, logits, n_expert, n_embd);
  if (launches) ++*launches;
  return cudaGetLastError();
}

cudaError_t launch_silu_mul(float* g, const float* u, int64_t n, cudaStream_t s, uint64_t* launches) {
  if (n <= 0) return cudaSuccess;
  if (n % 4 == 0 && (((uintptr_t)g | (uintptr_t)u) & 15) == 0) {
    int64_t blocks = (n / 4 + 255) / 256;
    if (blocks > 148 * 8) blocks = 148 * 8;
    silu_mul4_kernel<<<(unsigned)blocks, 256, 0, s>>>((float4*)g, (const float4*)u, n / 4);
  } else {
    int64_t blocks = (n + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    silu_mul_kernel<<<(unsigned)blocks, 256, 0, s>>>(g, u, n);
  }
  if (launches) ++*launches;
  return cudaGetLastError();
}

cudaError_t launch_scatter_combine(const float* y, const int* rows_of_tok, const float* w_of_tok, float* out,
                                   int tokens, int n_used, int n_embd, cudaStream_t s, uint64_t* launches) {
  if (tokens <= 0) return cudaSuccess;
  scatter_combine_kernel<<<tokens, 256, 0, s>>>(y, rows_of_tok, w_of_tok, out, tokens, n_used, n_embd);
  if (launches) ++*launches;
  return cudaGetLastError();
}

}  // namespace llr
