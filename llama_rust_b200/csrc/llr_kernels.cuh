// Internal launch interface between the executor (llr_exec.cu) and the kernels.
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

#include <atomic>
#include <string>
#include <vector>

namespace llr {

// One-time setup of a kernel, per device: function attributes and occupancy belong to a device's context, and executors
// of several devices (and threads) may share a process.  here() is the current device's slot; 0 means not set up yet
// (two threads that both find 0 do the same setup and store the same value).
struct PerDevice {
  std::atomic<int> slot[64];
  std::atomic<int>& here() {
    int d = 0;
    cudaGetDevice(&d);
    return slot[d & 63];
  }
};

// A resident packed matrix as the kernels see it.  `w` is 256-byte aligned and
// the allocation is padded so that 16-byte windows around any row are readable.
// Error word of an executor: one int in mapped pinned host memory.  A kernel whose bounded wait
// ran out stores a non-zero code with a plain store (any writer wins); the host reads the word
// after synchronizing, with no copy on the path.
#ifdef __CUDACC__
__device__ __forceinline__ void report_error(int* err, int code) { *(volatile int*)err = code; }
#endif

struct MatView {
  const uint8_t* w;
  int dtype;
  int64_t rows, cols;
  int64_t row_bytes;
  int f16_ok = -1;  // tensor-core GEMM operand choice: 1 binary16 (weights fit its range), 0 bfloat16, -1 not examined (bfloat16)
};

enum GemvPath : int { PATH_AUTO = 0, PATH_GENERIC = 1, PATH_STAGED = 2, PATH_MMA = 3, PATH_TC = 4 };
constexpr int64_t TC_MIN_TOKENS = 64;  // from here on AUTO prefers the bf16 tcgen05 GEMM

// y[t*rows + r] = sum_c W[r,c] * x[t*cols + c] for t < tokens.  Any shape the
// entry points accept.  `launches` is incremented by the kernels launched.
// `err_flag` is a device int that kernels with bounded waits set to non-zero when a wait ran out.
// `scratch` (gemm_tc_scratch_bytes, or null) lets the tensor-core GEMM stage bf16 activations.
cudaError_t launch_matmul(const MatView& m, const float* x, float* y, int64_t tokens,
                          cudaStream_t stream, int path, int sm_count, int* err_flag,
                          void* scratch, uint64_t* launches);
bool matmul_wants_tc(const MatView& m, int64_t tokens, int path);

// Always-available reference kernel: one warp per row, byte loads, any alignment.
cudaError_t launch_gemv_generic(const MatView& m, const float* x, float* y, int64_t tokens,
                                cudaStream_t stream, uint64_t* launches);

// Shared-memory staged decode GEMV (tokens <= 8 per pass); see llr_gemv_staged.cu.
bool gemv_staged_supported(const MatView& m);
cudaError_t launch_gemv_staged(const MatView& m, const float* x, float* y, int64_t tokens,
                               cudaStream_t stream, int sm_count, uint64_t* launches);

// Streaming decode GEMV for the element formats F32 / F16 / BF16 (tokens <= 8 per pass); see llr_gemv_rows.cu.
bool gemv_rows_supported(const MatView& m);
cudaError_t launch_gemv_rows(const MatView& m, const float* x, float* y, int64_t tokens, cudaStream_t stream, int sm_count,
                             uint64_t* launches);

// Integer tensor-core decode GEMV for Q4_K / Q6_K / Q8_0 (tokens <= 8 per pass); see
// llr_gemv_stream.cu.  Launched with programmatic stream serialization.
bool gemv_mma_supported(const MatView& m);
cudaError_t launch_gemv_mma(const MatView& m, const float* x, float* y, int64_t tokens,
                            cudaStream_t stream, int sm_count, int* err_flag, uint64_t* launches);
// Result delivery to the host by the kernel itself (host-pointer calls with at most 8 activation
// rows): the reducer also stores each finished value at y + y_delta bytes, a device alias of
// mapped pinned host memory, and the CTA that finishes last stores `ticket` into *done (mapped
// pinned as well) after a system-scope fence.  The host polls *done instead of enqueuing a
// device-to-host copy and synchronizing the stream.  count is a zeroed device word.
struct HostOut {
  long long y_delta;
  int* done;
  unsigned int* count;
  int ticket;
};
// One product with ONE activation row whose matrix a kernel earlier in the stream chooses: the weights are addressed
// through maps_dev[*sel_dev], an array (device memory) of GEMV_MAP_BYTES-byte tensor maps that gemv_mma_encode_map filled
// for matrices of one shape and format (`shape`: any of them).  No host round trip between the choice and the product.
constexpr int GEMV_MAP_BYTES = 128;
cudaError_t gemv_mma_encode_map(const MatView& m, void* map_out);
cudaError_t launch_gemv_mma_select(const MatView& shape, const void* maps_dev, const int* sel_dev, const float* x, float* y,
                                   cudaStream_t stream, int sm_count, int* err_flag, uint64_t* launches);
bool gemv_mma_hostout_ok(const MatView& m, int64_t tokens);
cudaError_t launch_gemv_mma_hostout(const MatView& m, const float* x, float* y, int64_t tokens, const HostOut& ho,
                                    cudaStream_t stream, int sm_count, int* err_flag, uint64_t* launches);

// One matrix product of a program (llr_gemv_stream.cu).  The caller fills the first block and the
// operation fields; tile_begin / n_tiles and everything about tagged buffers are filled in by
// program_create.
//
// Tagged buffers.  A result that a later entry of the same program reads is also written as 8-byte
// pairs {f32 bits, tag}, tag = tag_base of the run + producing phase.  A consumer loads pairs and
// spins (bounded) until every tag is the expected one: the value is its own arrival signal, so no
// counter, fence or poll separates a phase from the next.
enum XOp : int {
  XOP_NONE = 0,     // x as it is
  XOP_RMSNORM = 1,  // x * (1 / sqrt(mean(x^2) + eps)) * x2[c]   (x2: norm weights, plain f32, may be null)
  XOP_SWIGLU = 2,   // silu(x) * x2[c]                            (x2: the `up` vector)
};
struct ProgEntry {
  const uint8_t* w;
  const float* x;     // input, plain f32 (ignored by the kernel when xt is set)
  float* y;           // result, plain f32 (this rank's slice)
  int64_t row_bytes;
  int rows, cols, dtype, tokens;
  int tile_begin, n_tiles;
  int64_t y_ld;  // floats between consecutive activation rows of y (0: rows); larger when y is a slice of a wider vector
  // ---- 64 bytes
  const void* xt;     // tagged input (pairs), or null
  const void* x2;     // second operand of x_op: plain f32, or pairs when x2_phase >= 0
  const void* resid;  // added to the finished result, indexed like y: plain f32, or pairs when resid_phase >= 0; may be null
  void* yt;           // tagged copy of the result (this rank's slice), or null when no entry reads it
  int x_op;
  float eps;
  int x_phase, x2_phase, resid_phase;  // phase that writes the tagged source (-1: plain memory, ready at launch)
  int sel_slot, map_base;  // select programs (program_set_select): the matrix is maps[map_base + sel[sel_slot]]
  int pad;
};
static_assert(sizeof(ProgEntry) == 128, "entries are copied as sixteen 8-byte words");
// Row-sharded programs across GPUs: where the other ranks keep their copies of the results
// and of the phase counters.  peer address = local address + delta[g] bytes (arenas have one layout).
struct PeerTable {
  int n_peers;  // other ranks (world size - 1), at most 7
  int pad;
  unsigned long long* counters[7];
  long long y_delta[7];
};
// wait_prev: bit 0 = wait for the previous phase's counter, bit 1 = publish this phase's counter,
// bit 2 (phase 0 of a sharded program) = wait for the end of the previous run on every rank.
struct ProgPhase { int first_entry, n_entries, n_tiles, wait_prev; };
struct Program;
bool prog_entry_supported(const MatView& m);
// Placement of a sharded program's buffers: the arena is header | result area of result_bytes |
// tagged area of 2 * result_bytes; the pair of the float at result offset o lies at tagged offset 2 o.
struct ShardInfo {
  unsigned long long* counters;  // arena header
  PeerTable peers;
  char* arena;
  size_t result_bytes;
  int world, rank;
};
// phase_of[i] is non-decreasing.  strict_phases: an input that is not an earlier entry's result makes
// its phase wait until the previous phase is completely written (counter per phase); otherwise such
// inputs are read as they are at launch.
cudaError_t program_create(const std::vector<ProgEntry>& entries, const std::vector<int>& phase_of,
                           int sm_count, bool strict_phases, const ShardInfo* shard, Program** out, std::string* msg);
void program_destroy(Program* p);
// Turns a one-phase, one-token program without operations into a select program: entry E then reads its weights through
// maps_dev[E.map_base + sel_dev[E.sel_slot]] (tensor maps of gemv_mma_encode_map, matrices shaped like E) instead of
// E.w.  The table is read on the device when the launch runs, after the kernels before it in the stream.
cudaError_t program_set_select(Program* p, const void* maps_dev, const int* sel_dev);
// poll_limit: iterations a device-side wait for another CTA's or rank's data may take before it gives up
cudaError_t program_run(Program* p, cudaStream_t stream, int* err_flag, int poll_limit, uint64_t* launches);
int program_phases(const Program* p);
int program_entries(const Program* p);
int program_counter_phases(const Program* p);
int program_grid(const Program* p);  // phases that synchronise through a counter

// dequant -> shared memory -> tcgen05/TMEM chunk GEMM (bf16 operands, f32 accumulate) for
// Q4_K / Q8_0 / Q5_0 / Q5_1 with many activation rows; see llr_gemm_tc.cu.
bool gemm_tc_supported(const MatView& m, int64_t tokens);
// Examines the block headers of a matrix the GEMM can take: writes the bit pattern of the largest
// possible |weight| to *out_dev (device); weight_bound_allows_f16 turns that into the operand choice.
cudaError_t launch_weight_bound(const MatView& m, unsigned int* out_dev, cudaStream_t stream, uint64_t* launches);
bool weight_bound_allows_f16(unsigned int bound_bits);
// Grouped launch: several products of one dtype in one grid (routed experts).  x16 / xscale are
// the group's activations as tc_convert_activations left them; desc_dev is device scratch of
// gemm_tc_group_desc_bytes(n) bytes, 64-byte aligned.
struct GemmGroupSpec {
  MatView m;
  const void* x16;
  const float* xscale;
  float* y;
  int tokens;
};
size_t gemm_tc_group_desc_bytes(int n_groups);
cudaError_t tc_convert_activations(const float* x, int64_t n_rows, int cols, bool f16, void* out16, float* xscale,
                                   cudaStream_t stream, uint64_t* launches);
// Routed-expert layer: 16-bit operand row r from row src_row[r] of x (cols a multiple of 4, rows
// 16-byte aligned).
cudaError_t tc_convert_expert_rows(const float* x, const int* src_row, int64_t n_rows, int cols, bool f16,
                                   void* out16, float* xscale, cudaStream_t stream, uint64_t* launches);
cudaError_t launch_gemm_tc_grouped(const GemmGroupSpec* specs, int n_groups, bool f16, void* desc_dev,
                                   cudaStream_t stream, int* err_flag, uint64_t* launches);
size_t gemm_tc_scratch_bytes(const MatView& m, int64_t tokens);
cudaError_t launch_gemm_tc(const MatView& m, const float* x, float* y, int64_t tokens, void* scratch, size_t scratch_bytes,
                           cudaStream_t stream, int* err_flag, uint64_t* launches);

// Same kernels with the staging buffer in a file-scope __device__ array (no allocation).
constexpr size_t GEMM_STATIC_SCRATCH_BYTES = 32u << 20;
size_t gemm_tc_static_scratch_limit();
cudaError_t launch_gemm_tc_static(int device, const MatView& m, const float* x, float* y, int64_t tokens,
                                  cudaStream_t stream, int* err_flag, uint64_t* launches);

// Routed-expert FFN glue (llr_moe.cu)
cudaError_t launch_gather_rows(const float* x, const int* tok_of_row, float* packed, int n_rows, int n_embd,
                               cudaStream_t s, uint64_t* launches);
cudaError_t launch_silu_mul(float* g, const float* u, int64_t n, cudaStream_t s, uint64_t* launches);
// logits[t*n_expert + e] = dot(w[e], x[t]) for an F32 router matrix (n_embd % 4 == 0, 16-byte aligned)
cudaError_t launch_router_logits(const float* w, const float* x, float* logits, int tokens, int n_expert, int n_embd,
                                 cudaStream_t s, uint64_t* launches);
// Routing on the device: softmax / top-k / weights per token in place on the logits, then the packed row order
cudaError_t launch_route(float* logits, int tokens, int n_expert, int n_used, int norm_w, int* ids, float* wts,
                         cudaStream_t s, uint64_t* launches);
cudaError_t launch_bucket(const int* ids, const float* wts, const unsigned char* local, int tokens, int n_expert, int n_used,
                          int* first_row, int* tok_of_row, int* rows_of_tok, float* w_of_tok, int* fill, cudaStream_t s,
                          uint64_t* launches);
cudaError_t launch_scatter_combine(const float* y, const int* rows_of_tok, const float* w_of_tok, float* out,
                                   int tokens, int n_used, int n_embd, cudaStream_t s, uint64_t* launches);
// One token without a host round trip: its selection sorted by expert id (n_used <= 8), and the combine of its experts' rows
cudaError_t launch_select_sorted(const int* ids, const float* wts, int n_used, int* sel, float* selw, cudaStream_t s, uint64_t* launches);
cudaError_t launch_combine_one(const float* y, const float* selw, float* out, int n_used, int n_embd, cudaStream_t s, uint64_t* launches);

// Expert parallelism over peer stores (llr_moe_ep.cu).  An arena starts with an EpHeader, then twice (runs
// alternate): counts [local expert][sender], packed row numbers and rows [local expert][sender][t_max], and the
// return area [t_max * n_used] rows.
constexpr int EP_MAX_WORLD = 8;
struct EpHeader {
  unsigned long long flag_in[EP_MAX_WORLD];    // [sender]: last run whose rows from that sender are complete here
  unsigned long long flag_back[EP_MAX_WORLD];  // [owner]: last run whose results from that owner are complete here
  unsigned long long done_dispatch, done_return;  // this rank's CTAs, counted over all runs
};
struct EpPeers { char* arena[EP_MAX_WORLD]; };  // every rank's arena as mapped here (entry `rank`: this rank's own)
struct EpLayout {
  int n_expert, n_used, n_embd, world, rank, t_max, e_loc;
  size_t cnt_off[2], tag_off[2], recv_off[2], back_off[2], total;
};
EpLayout ep_layout(int n_expert, int n_used, int n_embd, int world, int rank, int t_max);
cudaError_t launch_ep_dispatch(const float* x, const int* tok_of_row, const int* first_row, int n_rows, const EpPeers& peers,
                               const EpLayout& L, int parity, unsigned long long epoch, unsigned long long done_target,
                               cudaStream_t s, uint64_t* launches);
cudaError_t launch_ep_wait(const unsigned long long* flags, int world, unsigned long long epoch, int poll_limit, int* err,
                           cudaStream_t s, uint64_t* launches);
cudaError_t launch_ep_gather(const char* arena, const EpLayout& L, int parity, const int* seg_first, int n_seg, int n_rows,
                             float* rows, int* ret_src, int* ret_tag, cudaStream_t s, uint64_t* launches);
cudaError_t launch_ep_return(const float* y, const int* ret_src, const int* ret_tag, int n_rows, const EpPeers& peers,
                             const EpLayout& L, int parity, unsigned long long epoch, unsigned long long done_target,
                             cudaStream_t s, uint64_t* launches);

// out[(r-row0)*cols + c] = dequantized W[r,c], bit-exact with the reference.
cudaError_t launch_dequant(const MatView& m, int64_t row0, int64_t n_rows, float* out,
                           cudaStream_t stream, uint64_t* launches);

// out[i*cols + c] = dequantized W[ids[i], c] with ids in device memory (token embeddings)
cudaError_t launch_dequant_indexed(const MatView& m, const int* ids_dev, int64_t n, float* out,
                                   cudaStream_t stream, uint64_t* launches);

// ---- element-wise and attention kernels of the device-resident Llama walk (llr_decode.cu) ----
struct WalkShape { int n_embd, n_head, n_head_kv, head_dim, n_ff, n_ctx; float rms_eps, rope_base, theta_scale; };
// y[t] = (x[t] * 1/sqrt(mean(x[t]^2) + eps)) * w; with `add` non-null first x[t] += add[t] (written back: the new
// residual stream).  w may be null (all ones).
cudaError_t launch_rmsnorm(float* x, const float* add, const float* w, float* y, int tokens, int n, float eps,
                           cudaStream_t s, uint64_t* launches);
// Paged KV cache as the kernels see it (langtax/src/kv_page.rs:395-437: a head vector of block b lies at
// (((b * n_layers + layer) * n_head_kv + head) * block_tokens + t % block_tokens) * head_dim, b = table[t / block_tokens]).
// table holds max_blocks entries per sequence.
struct KvView {
  float* k;
  float* v;
  const int* table;
  int block_tokens, max_blocks, n_layer;
};
// Where the rows of a batch stand: row t belongs to sequence row_seq[t] at position row_pos[t]; with null arrays all
// rows belong to sequence 0 at positions *pos_dev + t (the position counter lives in device memory so that a captured
// or pre-enqueued step sees the current value).
struct RowMap {
  const int* pos_dev;
  const int* row_pos;
  const int* row_seq;
};
// RoPE (adjacent pairs) on q and k at each row's position, then k and v into the cache.
cudaError_t launch_rope_store(float* q, float* k, const float* v, const KvView& kv, const RowMap& rows, int tokens, int layer,
                              const WalkShape& w, cudaStream_t s, uint64_t* launches);
// out[t][hq] = softmax(q[t][hq] . K[0..pos(t)] / sqrt(hd)) V over row t's own sequence, grouped-query heads; scratch holds
// the partial results of the position splits (attention_scratch_floats)
size_t attention_scratch_floats(int tokens, const WalkShape& w);
cudaError_t launch_attention(const float* q, const KvView& kv, float* out, float* scratch, const RowMap& rows, int tokens,
                             int layer, const WalkShape& w, cudaStream_t s, uint64_t* launches,
                             const float* k_new = nullptr, const float* v_new = nullptr,  // k_new / v_new: one decode token whose rotation and cache store the attention kernel does itself
                             bool tensor_cores = false,  // a prompt chunk of one sequence may run as binary16 MMAs with f32 accumulation (the tolerance of the 16-bit chunk GEMM)
                             bool one_sequence = false);  // the caller vouches that the rows are one sequence at consecutive positions (rows given per row)
cudaError_t launch_swiglu(float* g, const float* u, int64_t n, cudaStream_t s, uint64_t* launches);
cudaError_t launch_add(float* x, const float* y, int64_t n, cudaStream_t s, uint64_t* launches);
// first index of the strict maximum of logits[0..n) -> *out_id (device; n == 0: no argmax), and *pos_dev += advance
// With count_dev the token also goes to out_id[1 + *count_dev], its margin to out_margin[*count_dev], and the
// count grows by one (a generation loop whose steps are identical launches).
// part: 384 words of device scratch (a long row is scanned by many blocks), or null
cudaError_t launch_argmax_advance(const float* logits, int n, int* out_id, float* out_margin, int* pos_dev, int advance,
                                  int* count_dev, float* part, cudaStream_t s, uint64_t* launches);
// one argmax per row of logits[n_rows][n] -> out_id[row], out_margin[row] (optional)
cudaError_t launch_argmax_rows(const float* logits, int n_rows, int n, int* out_id, float* out_margin, cudaStream_t s,
                               uint64_t* launches);

// *flag_dev = 1 when the two device byte ranges differ (both 16-byte aligned), else 0
cudaError_t launch_bytes_differ(const void* a, const void* b, size_t n, int* flag_dev, cudaStream_t stream, uint64_t* launches);

// Seeded synthetic packed blocks (see llama_rust_b200/synth.py for the recipe).
cudaError_t launch_synth(int dtype, int64_t rows, int64_t cols, uint64_t seed, uint8_t* w,
                         cudaStream_t stream, uint64_t* launches);

}  // namespace llr
