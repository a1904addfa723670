// Expert parallelism: the exchange of routed rows between ranks as peer stores.
//
// Experts are striped over the ranks (expert e on rank e % G, expertvm/src/place.rs:71-75) and the tokens
// are sharded too.  Every rank routes its own tokens and buckets the routed rows by expert in token order
// (the packed order of grouped_routed_ffn, langtax/src/decode.rs:10006); then
//   dispatch: each packed row is stored straight into the owner's receive area (its own arena for experts
//             that live here), together with its packed row number; the CTA that finishes last stores the
//             per-expert counts and raises one flag per owner;
//   serve:    the owner waits (bounded) for every sender's flag, gathers what arrived into the packed order
//             of its experts (sender ascending, position ascending: the global token order when the tokens
//             are sharded in rank order), runs the expert products, and stores every result row into the
//             sender's return area at the row number that came with it; one flag per sender;
//   combine:  the sender waits (bounded) for every owner's flag; its return area is then exactly the packed
//             result matrix of the single-device layer, and scatter_expert_rows (decode.rs:10263) runs on it.
// No collective call and no host hop carries rows; the host reads one small table of counts to size the
// expert launches, as the single-device layer does.
//
// Everything a peer writes lives in this rank's arena, twice (runs alternate between the halves): a sender
// cannot start run n+1 before it has every owner's return flag of run n, and an owner raises that flag only
// after it has read what run n delivered, so a half is never written while it is being read.
#include "llr_kernels.cuh"

namespace llr {
namespace {

__device__ __forceinline__ unsigned long long ld_acquire_sys(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(unsigned long long* p, unsigned long long v) {
  asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
// true for the CTA that completes the count (cumulative over runs: `target` is the total after this launch)
__device__ __forceinline__ bool last_cta(unsigned long long* counter, unsigned long long target) {
  unsigned long long old;
  asm volatile("atom.acq_rel.gpu.global.add.u64 %0, [%1], %2;" : "=l"(old) : "l"(counter), "l"(1ull) : "memory");
  return old + 1 == target;
}
__device__ __forceinline__ void copy_row(float* dst, const float* src, int n_embd) {
  const float4* s = (const float4*)src;
  float4* d = (float4*)dst;
  for (int i = threadIdx.x; i < n_embd / 4; i += blockDim.x) d[i] = s[i];
}
// largest k with first[k] <= r (first is ascending, first[0] = 0, r < first[n])
__device__ __forceinline__ int segment_of(const int* first, int n, int r) {
  int lo = 0, hi = n;
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (first[mid] <= r) lo = mid; else hi = mid;
  }
  return lo;
}

// One CTA per packed row of this rank's routed rows.
__global__ void __launch_bounds__(256)
ep_dispatch_kernel(const float* __restrict__ x, const int* __restrict__ tok_of_row, const int* __restrict__ first_row,
                   EpPeers peers, EpLayout L, int parity, unsigned long long epoch, unsigned long long done_target) {
  const int r = blockIdx.x;
  const int e = segment_of(first_row, L.n_expert, r);
  const int owner = e % L.world, le = e / L.world, i = r - first_row[e];
  char* base = peers.arena[owner];
  const size_t slot = ((size_t)le * L.world + L.rank) * L.t_max + i;
  copy_row((float*)(base + L.recv_off[parity]) + slot * L.n_embd, x + (size_t)tok_of_row[r] * L.n_embd, L.n_embd);
  if (threadIdx.x == 0) ((int*)(base + L.tag_off[parity]))[slot] = r;
  __syncthreads();  // every thread's peer stores are issued before the count
  if (threadIdx.x == 0) {
    EpHeader* mine = (EpHeader*)peers.arena[L.rank];
    if (last_cta(&mine->done_dispatch, done_target)) {  // acquires every CTA's release: their stores are ordered before ours
      for (int ex = 0; ex < L.n_expert; ++ex)
        ((int*)(peers.arena[ex % L.world] + L.cnt_off[parity]))[(ex / L.world) * L.world + L.rank] = first_row[ex + 1] - first_row[ex];
      for (int p = 0; p < L.world; ++p) st_release_sys(&((EpHeader*)peers.arena[p])->flag_in[L.rank], epoch);
    }
  }
}

// Thread s waits until flags[s] has reached `epoch`; a wait that runs out records an error and ends.
__global__ void ep_wait_kernel(const unsigned long long* __restrict__ flags, int world, unsigned long long epoch, int poll_limit,
                               int* __restrict__ err) {
  const int s = threadIdx.x;
  if (s >= world) return;
  for (int polls = 0; ld_acquire_sys(flags + s) < epoch; ++polls) {
    if (polls >= poll_limit) { report_error(err, 2); return; }
    __nanosleep(polls < 8 ? 64 : 256);
  }
}

// One CTA per gathered row q: segment k = local expert * world + sender, rows of a segment in arrival position order.
__global__ void __launch_bounds__(256)
ep_gather_kernel(const char* __restrict__ arena, EpLayout L, int parity, const int* __restrict__ seg_first, int n_seg,
                 float* __restrict__ rows, int* __restrict__ ret_src, int* __restrict__ ret_tag) {
  const int q = blockIdx.x;
  const int k = segment_of(seg_first, n_seg, q);
  const size_t slot = (size_t)k * L.t_max + (q - seg_first[k]);
  copy_row(rows + (size_t)q * L.n_embd, (const float*)(arena + L.recv_off[parity]) + slot * L.n_embd, L.n_embd);
  if (threadIdx.x == 0) {
    ret_src[q] = k % L.world;
    ret_tag[q] = ((const int*)(arena + L.tag_off[parity]))[slot];
  }
}

// One CTA per result row; with no rows (n_rows == 0, one CTA) only the flags are raised.
__global__ void __launch_bounds__(256)
ep_return_kernel(const float* __restrict__ y, const int* __restrict__ ret_src, const int* __restrict__ ret_tag, int n_rows,
                 EpPeers peers, EpLayout L, int parity, unsigned long long epoch, unsigned long long done_target) {
  bool last = n_rows == 0;
  if (n_rows > 0) {
    const int q = blockIdx.x;
    copy_row((float*)(peers.arena[ret_src[q]] + L.back_off[parity]) + (size_t)ret_tag[q] * L.n_embd, y + (size_t)q * L.n_embd, L.n_embd);
    __syncthreads();
    if (threadIdx.x == 0) last = last_cta(&((EpHeader*)peers.arena[L.rank])->done_return, done_target);
  }
  if (threadIdx.x == 0 && last)
    for (int p = 0; p < L.world; ++p) st_release_sys(&((EpHeader*)peers.arena[p])->flag_back[L.rank], epoch);
}

}  // namespace

EpLayout ep_layout(int n_expert, int n_used, int n_embd, int world, int rank, int t_max) {
  EpLayout L;
  L.n_expert = n_expert; L.n_used = n_used; L.n_embd = n_embd; L.world = world; L.rank = rank; L.t_max = t_max;
  L.e_loc = (n_expert + world - 1) / world;
  auto up = [](size_t v) { return (v + 255) & ~(size_t)255; };
  size_t at = up(sizeof(EpHeader));
  const size_t slots = (size_t)L.e_loc * world * t_max;
  for (int p = 0; p < 2; ++p) {
    L.cnt_off[p] = at;  at = up(at + (size_t)L.e_loc * world * 4);
    L.tag_off[p] = at;  at = up(at + slots * 4);
    L.recv_off[p] = at; at = up(at + slots * n_embd * 4);
    L.back_off[p] = at; at = up(at + (size_t)t_max * n_used * n_embd * 4);
  }
  L.total = at;
  return L;
}

cudaError_t launch_ep_dispatch(const float* x, const int* tok_of_row, const int* first_row, int n_rows, const EpPeers& peers,
                               const EpLayout& L, int parity, unsigned long long epoch, unsigned long long done_target,
                               cudaStream_t s, uint64_t* launches) {
  ep_dispatch_kernel<<<(unsigned)n_rows, 256, 0, s>>>(x, tok_of_row, first_row, peers, L, parity, epoch, done_target);
  if (launches) ++*launches;
  return cudaGetLastError();
}

cudaError_t launch_ep_wait(const unsigned long long* flags, int world, unsigned long long epoch, int poll_limit, int* err,
                           cudaStream_t s, uint64_t* launches) {
  ep_wait_kernel<<<1, 32, 0, s>>>(flags, world, epoch, poll_limit, err);
  if (launches) ++*launches;
  return cudaGetLastError();
}

cudaError_t launch_ep_gather(const char* arena, const EpLayout& L, int parity, const int* seg_first, int n_seg, int n_rows,
                             float* rows, int* ret_src, int* ret_tag, cudaStream_t s, uint64_t* launches) {
  if (n_rows <= 0) return cudaSuccess;
  ep_gather_kernel<<<(unsigned)n_rows, 256, 0, s>>>(arena, L, parity, seg_first, n_seg, rows, ret_src, ret_tag);
  if (launches) ++*launches;
  return cudaGetLastError();
}

cudaError_t launch_ep_return(const float* y, const int* ret_src, const int* ret_tag, int n_rows, const EpPeers& peers,
                             const EpLayout& L, int parity, unsigned long long epoch, unsigned long long done_target,
                             cudaStream_t s, uint64_t* launches) {
  ep_return_kernel<<<(unsigned)(n_rows > 0 ? n_rows : 1), 256, 0, s>>>(y, ret_src, ret_tag, n_rows, peers, L, parity, epoch, done_target);
  if (launches) ++*launches;
  return cudaGetLastError();
}

}  // namespace llr
