/* llama_rust_b200 — C ABI of the B200 (sm_100a) quantized matrix executor.
 *
 * Drop-in boundary for the matrix-executor seam of mingley/llama-rust: the
 * entry points below are what the crate's FFI for this path binds in place of
 * the `llama_native_cuda` crate (native-cuda/src/gpu.rs) and of
 * `native_gpu::matmul` (langtax/src/native_gpu.rs:124).  Plain pointers and
 * sizes only; every function returns an int status, 0 = ok.
 *
 * Conventions shared by all entry points (reference behaviour in brackets):
 *  - dtype tags are the reference's `GemmKind as u8` [langtax/src/quant.rs:6645]:
 *    F16=0 BF16=1 F32=2 Q4_1=5 Q5_0=6 Q5_1=7 Q4_0=12 Q8_0=13 Q4_K=17 Q5_K=18 Q6_K=19.  Any
 *    other tag is LLR_ERR_DTYPE; there is no CPU fallback [README.md:29-31].
 *  - activations and results are token-major f32: x[t*cols + c], y[t*rows + r]
 *    [quant.rs:6264-6267].
 *  - weights are GGUF packed blocks, rows contiguous without padding; they stay
 *    packed in device memory and are never expanded to f32.
 *  - all validation happens before any device work; a failing call leaves the
 *    output buffer untouched and the executor usable
 *    [langtax/tests/native_cuda_parity.rs:410-431, native-cuda/src/main.rs:48-66].
 *  - an executor is not thread-safe: one per inference thread
 *    [native_gpu.rs:114-116].  Host-pointer calls are synchronous: the output
 *    is valid on return.
 */
#ifndef LLAMA_RUST_B200_H
#define LLAMA_RUST_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define LLR_DTYPE_F16 0
#define LLR_DTYPE_BF16 1
#define LLR_DTYPE_F32 2
#define LLR_DTYPE_Q4_1 5
#define LLR_DTYPE_Q5_0 6
#define LLR_DTYPE_Q5_1 7
#define LLR_DTYPE_Q4_0 12
#define LLR_DTYPE_Q8_0 13
#define LLR_DTYPE_Q4_K 17
#define LLR_DTYPE_Q5_K 18
#define LLR_DTYPE_Q6_K 19

#define LLR_OK 0
#define LLR_ERR_INVALID 1   /* bad shape / length / null pointer  [QuantError::Size, ::NativeCuda] */
#define LLR_ERR_UNALIGNED 2 /* cols not a multiple of the block   [QuantError::UnalignedCols]      */
#define LLR_ERR_DTYPE 3     /* unsupported dtype tag                                               */
#define LLR_ERR_OVERFLOW 4  /* a size product overflows           ["... shape overflow"]           */
#define LLR_ERR_FOREIGN 5   /* matrix belongs to another executor [gpu.rs:286-288]                 */
#define LLR_ERR_CUDA 6      /* CUDA runtime failure; see llr_exec_last_error                       */
#define LLR_ERR_OOM 7       /* device allocation failed after dropping cached weights              */
#define LLR_ERR_CONFIG 8    /* malformed LLAMA_CUDA_CACHE_BYTES   [native_gpu.rs:20-32]            */
/* GGUF parse errors [GgufError, langtax/src/gguf.rs:338-370] */
#define LLR_GGUF_MAGIC 20        /* "not a GGUF file"                 */
#define LLR_GGUF_VERSION 21      /* "unsupported GGUF version {v}"    */
#define LLR_GGUF_TRUNCATED 22    /* "truncated GGUF"                  */
#define LLR_GGUF_UTF8 23         /* "non-utf8 GGUF string"            */
#define LLR_GGUF_TYPE 24         /* "unsupported ggml type {t}"       */
#define LLR_GGUF_REMOVED_TYPE 25 /* "ggml-removed type {t}"           */
#define LLR_GGUF_KV_TYPE 26      /* "unsupported GGUF kv type {t}"    */
#define LLR_GGUF_SHAPE 27        /* "invalid GGUF tensor shape"       */

typedef struct llr_exec llr_exec;     /* opaque executor: device, stream, scratch, residency */
typedef struct llr_matrix llr_matrix; /* opaque resident packed matrix, tied to its executor  */

typedef struct llr_counters {
  uint64_t launches;       /* kernels launched by this executor                     */
  uint64_t uploads;        /* packed matrices copied host -> device                 */
  uint64_t upload_bytes;
  uint64_t resident_bytes; /* packed bytes held by the residency cache              */
  uint64_t cache_limit;    /* residency budget in bytes (0 = residency disabled)    */
  uint64_t cache_hits;
  uint64_t cache_misses;
  uint64_t evictions;
  uint64_t h2d_bytes;      /* activation bytes copied host -> device                */
  uint64_t d2h_bytes;      /* result bytes copied device -> host                    */
} llr_counters;

/* Replaces CudaGemv::new(device_ordinal) [native-cuda/src/gpu.rs:148]. */
int llr_exec_create(int device, llr_exec** out);
int llr_exec_destroy(llr_exec* exec);

/* Replaces CudaGemv::memory_info [gpu.rs:164]: free and total device bytes. */
int llr_exec_mem_info(llr_exec* exec, size_t* free_bytes, size_t* total_bytes);

/* Message of the last failing call on this executor ("" if none).  With a null
 * executor: the last failure of llr_exec_create on the calling thread.
 * Replaces the String of Result<_, String> [gpu.rs] / QuantError::NativeCuda
 * [quant.rs:4157]. */
const char* llr_exec_last_error(const llr_exec* exec);

int llr_exec_counters(const llr_exec* exec, llr_counters* out);

/* Diagnostic knob: which decode kernel serves the call.  0 = pick automatically
 * (integer tensor-core kernel where the format and shape allow, else the
 * staged kernel, else the shape-agnostic one), 1 = the shape-agnostic byte-load
 * kernel, 2 = the shared-memory staged FMA kernel (falls back to 1 for shapes
 * it cannot take), 3 = the integer tensor-core kernel for any number of
 * activation rows (f32-faithful), 4 = the tcgen05 GEMM whenever it can take
 * the call.  Automatic choice: up to 63 activation rows as 3, from 64 rows the
 * tcgen05 GEMM for every block-quantized format (16-bit operands, binary16 when
 * the weights' range allows, else bfloat16: relative L2 error of a result up to
 * 4e-3 against the f32 row kernels, 3e-4 typical with binary16).
 * Also read once from the environment variable LLR_GEMV_PATH
 * (generic|staged|mma|tc) when the executor is created. */
int llr_exec_set_path(llr_exec* exec, int path);

/* Packed bytes of one row of `cols` columns.  Replaces the <t>_row_bytes
 * family [quant.rs:4210-4218 and siblings]. */
int llr_row_bytes(uint8_t dtype, size_t cols, size_t* out);

/* Copy a packed matrix to the device and keep it resident.  Replaces
 * CudaGemv::upload [gpu.rs:264], which took F32-expanded weights; this one
 * takes the GGUF bytes as they are.  rows and cols must be positive and
 * packed_len == rows * row_bytes(dtype, cols). */
int llr_matrix_upload(llr_exec* exec, uint8_t dtype, size_t rows, size_t cols,
                      const void* packed, size_t packed_len, llr_matrix** out);
/* Same, from packed bytes already in device memory (device-to-device copy). */
int llr_matrix_upload_device(llr_exec* exec, uint8_t dtype, size_t rows, size_t cols,
                             const void* packed_dev, size_t packed_len, llr_matrix** out);
int llr_matrix_free(llr_matrix* matrix);
int llr_matrix_info(const llr_matrix* matrix, uint8_t* dtype, size_t* rows, size_t* cols,
                    size_t* packed_bytes);

/* y[rows] = W x.  Replaces CudaGemv::gemv_resident [gpu.rs:280].  Host
 * pointers; x_len must equal cols and y_len rows. */
int llr_gemv_resident(llr_exec* exec, const llr_matrix* matrix, const float* x, size_t x_len,
                      float* y, size_t y_len);

/* y[t*rows + r] for `tokens` activation rows in one call.  Replaces
 * CudaGemv::gemm_resident [gpu.rs:351].  tokens == 0 is an error.
 * Host-pointer calls return with y valid.  Every error detected before the
 * launch (all shape and handle errors) leaves y untouched, as in the reference.
 * For up to 8 activation rows on the streaming decode kernel, the kernel stores
 * the result straight into y when y is pinned host memory (into a pinned staging
 * buffer otherwise) and raises a completion word this call polls, instead of a
 * device-to-host copy and a stream synchronize; if a device-side bounded wait
 * runs out (status LLR_ERR_CUDA) a pinned y may then hold partial results.
 * LLR_HOST_DELIVERY=0 in the environment selects the copy path always. */
int llr_gemm_resident(llr_exec* exec, const llr_matrix* matrix, size_t tokens, const float* x,
                      size_t x_len, float* y, size_t y_len);

/* The call the crate makes for every f32-activation matrix product.  Replaces
 * native_gpu::matmul [langtax/src/native_gpu.rs:124-214] together with the
 * validation of native_matmul [quant.rs:6683-6758]; the `expand` closure of
 * the reference is never needed.  Weights are looked up in a device residency
 * cache keyed by (dtype, rows, cols, length, 128-bit content hash), so the
 * same bytes at another address hit and changed bytes at the same address miss
 * [native_cuda_parity.rs:181-187].  The reference compares every byte on a hit
 * [native_gpu.rs:96-98]; here two different matrices with equal shape, length and
 * fingerprint would be taken for one (no such pair is known; the hash is not
 * cryptographic).  LLAMA_CUDA_CACHE_VERIFY=1 compares all bytes on the device on
 * every hit and restores the exact guarantee at the price of an upload per call.  The budget is LLAMA_CUDA_CACHE_BYTES
 * ("auto" or unset: free - max(free/4, 512 MiB); a decimal byte count; 0
 * disables residency but not execution) [native_gpu.rs:5-9, 34-40] and counts
 * packed bytes only.  rows == 0 is a successful no-op [quant.rs:6743]. */
int llr_matmul(llr_exec* exec, uint8_t dtype, size_t rows, size_t cols, size_t tokens,
               const void* packed, size_t packed_len, const float* x, size_t x_len, float* y,
               size_t y_len);

/* llr_matmul for weights the caller can name: (key_hi, key_lo) is a stable identity of the packed bytes -- the blob
 * range QuantMat.start..end of an immutable model file [langtax/src/decode.rs:476-485], or (layer, expert, part) of an
 * expert store [ExpertKey, expertvm/src/store.rs:13-20] -- and replaces the content fingerprint: a hit reads nothing
 * but the key.  The caller guarantees that one key always names the same bytes.  Keyed and fingerprinted entries
 * share the budget and never match each other. */
int llr_matmul_keyed(llr_exec* exec, uint64_t key_hi, uint64_t key_lo, uint8_t dtype, size_t rows, size_t cols,
                     size_t tokens, const void* packed, size_t packed_len, const float* x, size_t x_len, float* y,
                     size_t y_len);
/* Keeps the resident matrix of a key out of eviction (pinned != 0) or releases it again (0)
 * [pin_hot / unpin_all of the expert store as Engine::pin_predicted uses them, langtax/src/engine.rs:916-950].
 * Pinned bytes still count against the budget. */
int llr_exec_pin_key(llr_exec* exec, uint64_t key_hi, uint64_t key_lo, int pinned);
/* Move an expert's weights to the device that computes, or leave them and ship activations: the byte-volume rule
 * of plan_placement [expertvm/src/planner.rs:332-349]; returns LLR_PLACE_*. */
#define LLR_PLACE_MOVE_WEIGHTS 0
#define LLR_PLACE_DISPATCH_ACTIVATIONS 1
int llr_plan_placement(uint64_t expert_bytes, uint64_t activation_bytes, uint64_t fan_in, uint64_t reuse,
                       uint64_t link_bps);

/* ---- model files ---------------------------------------------------------------------------------------------
 * GGUF v3 reader [load_gguf / parse_gguf, langtax/src/gguf.rs:700-806] and the step from a tensor's blob range to a
 * resident packed matrix [QuantMat, quant_mat, quant_mat_rows: langtax/src/decode.rs:476-485, :9612-9713].
 * llr_gguf_open maps the file read-only; llr_gguf_open_bytes parses an image the caller keeps alive.  Both return
 * the object even on a parse error (for llr_gguf_last_error); release it with llr_gguf_close. */
typedef struct llr_gguf llr_gguf;
typedef struct {
  const char* name;    /* valid until llr_gguf_close; name_len bytes of UTF-8 and a terminating NUL */
  int32_t ggml_type;   /* ggml type id as stored in the file                                      */
  int32_t dtype;       /* LLR_DTYPE_* of the executor, or -1 when it has no kernel for the type   */
  uint32_t n_dims;     /* 1..4                                                                    */
  uint64_t shape[4];   /* GGUF order, innermost (columns) first; unused entries are 1             */
  uint64_t start, end; /* byte range of the payload in the file [Tensor::blob_range, gguf.rs:435] */
  uint64_t name_len;   /* bytes of `name`: a name is any UTF-8 string, NUL bytes included [read_string, gguf.rs:903] */
} llr_gguf_tensor;
int llr_gguf_open(const char* path, llr_gguf** out);
int llr_gguf_open_bytes(const void* bytes, size_t len, llr_gguf** out);
void llr_gguf_close(llr_gguf* g);
const char* llr_gguf_last_error(const llr_gguf* g);
int llr_gguf_info(const llr_gguf* g, size_t* n_tensors, size_t* alignment, size_t* file_bytes);
int llr_gguf_tensor_at(const llr_gguf* g, size_t index, llr_gguf_tensor* out); /* file order [Gguf::tensors] */
int llr_gguf_find(const llr_gguf* g, const char* name, llr_gguf_tensor* out);  /* first of that name [Gguf::tensor] */
/* (names are looked up as C strings: a tensor whose name holds a NUL byte is reached through llr_gguf_tensor_at only) */
/* Copies bytes [start, start + len) of the file image to out (small host-side tensors such as norm weights). */
int llr_gguf_read(const llr_gguf* g, uint64_t start, size_t len, void* out);
/* Typed metadata readers: LLR_ERR_INVALID when the key is absent or holds another type [gguf.rs:571-628]. */
int llr_gguf_kv_u32(const llr_gguf* g, const char* key, uint32_t* out);
int llr_gguf_kv_f32(const llr_gguf* g, const char* key, float* out);
int llr_gguf_kv_bool(const llr_gguf* g, const char* key, int* out);
int llr_gguf_kv_string(const llr_gguf* g, const char* key, const char** out, size_t* len);
int llr_gguf_kv_i32s(const llr_gguf* g, const char* key, int32_t* out, size_t cap, size_t* n);
int llr_gguf_kv_type(const llr_gguf* g, const char* key, int* type, int* elem_type, size_t* n_items);
/* Any scalar value as raw bits (integers extended to 64 bits, floats as their IEEE bits) with its gguf type. */
int llr_gguf_kv_bits(const llr_gguf* g, const char* key, uint64_t* bits, int* type);
/* Rows [first_row, first_row + n_rows) (n_rows 0: all rows) of part `part` (0 for a 2-D weight, the expert for a
 * 3-D *_exps tensor) as a resident matrix: the bytes go from the file image to the device packed. */
int llr_gguf_upload(llr_exec* exec, llr_gguf* g, const char* name, size_t part, size_t first_row, size_t n_rows,
                    llr_matrix** out);
/* The same range through llr_matmul_keyed, the key being (this open file, byte offset): the crate-facing product
 * for weights that live in a model file; after the first call nothing of the weights is read on the host. */
int llr_gguf_matmul(llr_exec* exec, llr_gguf* g, const char* name, size_t part, size_t first_row, size_t n_rows,
                    size_t tokens, const float* x, size_t x_len, float* y, size_t y_len);
/* The key llr_gguf_matmul uses for that range, e.g. for llr_exec_pin_key.  key_hi counts open files from 1;
 * callers that make keys of their own keep them apart by setting the top bit of key_hi. */
int llr_gguf_key(llr_gguf* g, const char* name, size_t part, size_t first_row, size_t n_rows, uint64_t* key_hi,
                 uint64_t* key_lo);

/* Device-pointer form of llr_gemm_resident: x_dev and y_dev are device
 * buffers of tokens*cols and tokens*rows floats; the work is enqueued on
 * `stream` (a cudaStream_t; null = the executor's own stream) and the call
 * returns without synchronizing.  An extension with no counterpart in the
 * reference, whose executor copies through host memory on every call
 * [gpu.rs:301-334]. */
int llr_matmul_device(llr_exec* exec, const llr_matrix* matrix, size_t tokens, const float* x_dev,
                      float* y_dev, void* stream);
/* Chunk GEMM that allocates nothing.  No counterpart in the reference.
 *
 * For callers that must not touch the device allocator while they run: a serving
 * loop whose KV pool and weights already fill the GPU, so a growing scratch
 * buffer could fail or evict; code inside a region where the implicit device
 * synchronization of cudaMalloc/cudaFree is not acceptable; hosts that hand this
 * library a fixed memory budget up front.  Same tensor-core GEMM as the
 * automatic path takes from 64 activation rows on (every block-quantized format;
 * cols % 256 == 0, Q6_K cols % 2048 == 0; tokens >= 16; 16-bit operands -- binary16 when the matrix's
 * weights fit its range, else bfloat16 -- with f32 accumulation), but the
 * 16-bit copy of the activations is staged in a fixed 32 MiB array built into the
 * library (every GPU that loads the library holds it until the process exits)
 * instead of an executor buffer.  x_dev / y_dev are device buffers of
 * tokens*cols and tokens*rows floats, x_dev 16-byte aligned; the work is
 * enqueued on `stream` (null = the executor's stream) without synchronizing.
 * Limit: tokens * cols * 2 bytes <= 32 MiB, larger calls are rejected with
 * LLR_ERR_INVALID and a message; nothing else is tried.
 * A long row that llr_matmul_device would cut along K into slices (partial sums in
 * executor scratch) is computed in one piece here when the slices do not fit
 * the fixed array: the result then differs from llr_matmul_device's in summation
 * order only.
 * The first call on a device looks up the array's device address
 * (cudaGetSymbolAddress); make that first call outside any stream capture.
 * The call itself performs no cudaMalloc, cudaFree or other allocating call.
 * All calls share the one array and it keeps the last call's contents: each
 * call overwrites the part it uses before reading it, so nothing has to be
 * cleared, but two calls that overlap on the GPU (different streams, or
 * another executor) race on it; order them. */
int llr_gemm_device_noalloc(llr_exec* exec, const llr_matrix* matrix, size_t tokens,
                            const float* x_dev, float* y_dev, void* stream);

/* Block the calling thread until the executor's own stream is idle; reports
 * LLR_ERR_CUDA if a kernel's bounded device-side wait gave up since the last check. */
int llr_exec_synchronize(llr_exec* exec);

/* ---- programs: many decode products in one persistent launch -----------------
 * An extension with no counterpart in the reference, which launches and
 * synchronizes once per product [gpu.rs:301-334]; it stands where the per-token
 * sequence of gemm_into calls of Llama::forward_layers stands
 * [langtax/src/decode.rs:2737-3097].  A program is a fixed list of products over
 * resident matrices with device activation / result buffers.  Entries with the
 * same `phase` value are independent of each other; `phase` must be
 * non-decreasing along the list.  Supported: Q4_K, Q6_K (cols % 2048 == 0) and
 * Q8_0 matrices with cols % 256 == 0, tokens 1..8, buffers 16-byte aligned.
 * One launch (cooperative: the whole grid is resident) runs the list;
 * llr_program_run returns without synchronizing.  Two runs of the same program
 * must not overlap on the device.
 *
 * How a later entry gets an earlier entry's result: when an input pointer
 * (x_dev, and for llr_program_op also x2_dev of SwiGLU and resid_dev) is exactly
 * the y_dev of an earlier-phase entry with the same `tokens` and as many rows as
 * the reader has columns (one token: any 16-byte aligned part of that result will
 * do), the result travels inside the launch as 8-byte pairs {value, tag of run
 * and phase} in scratch the program owns: the reader spins (bounded) on the pairs
 * it needs, so nothing else separates the two phases.  y_dev still receives the
 * plain floats.
 * llr_program_create keeps strict phases on top: a phase with an input that is
 * NOT such a result starts only after every product of the previous phase has
 * been written (a counter per phase), so that x may alias earlier results in any
 * other way.  llr_program_create_ops does not: inputs that are not results of
 * the program are read as they are when the launch starts and must not be
 * written during it. */
typedef struct llr_program llr_program;
typedef struct llr_program_entry {
  const llr_matrix* matrix;
  const float* x_dev; /* tokens * cols floats */
  float* y_dev;       /* tokens * rows floats */
  uint32_t tokens;
  uint32_t phase;
} llr_program_entry;
int llr_program_create(llr_exec* exec, const llr_program_entry* entries, size_t n_entries,
                       llr_program** out);
int llr_program_run(llr_exec* exec, llr_program* program, void* stream);
int llr_program_free(llr_program* program);
/* entries, phases, phases that synchronise through a counter, CTAs of the launch (any pointer may be null) */
int llr_program_info(const llr_program* program, uint32_t* entries, uint32_t* phases, uint32_t* counter_phases,
                     uint32_t* ctas);

/* Products with the element-wise step that precedes them in the model and the
 * residual add that follows, so that a chain of products needs no other kernel
 * [the walk of decode.rs:2737-3097: rmsnorm_inplace :11498 before q/k/v, gate/up
 * and the output matrix; silu(gate) * up :2972-2996 before ffn_down; `+ residual`
 * after attn_output and ffn_down].
 *   LLR_XOP_NONE     y = W x
 *   LLR_XOP_RMSNORM  y = W ((x * 1/sqrt(mean(x^2) + eps)) * x2), x2 = cols norm weights
 *                    (plain device floats, NULL = all ones); the sum of squares is added
 *                    in a fixed tree order, not sequentially as the reference does
 *   LLR_XOP_SWIGLU   y = W (silu(x) * x2), x2 = tokens * cols floats (the `up` result)
 * resid_dev (optional, tokens * y_ld floats, indexed like the full-width result):
 * y += resid.  y_ld = floats between consecutive activation rows of y (0: rows). */
#define LLR_XOP_NONE 0
#define LLR_XOP_RMSNORM 1
#define LLR_XOP_SWIGLU 2
typedef struct llr_program_op {
  const llr_matrix* matrix;
  const float* x_dev;
  const float* x2_dev;
  const float* resid_dev;
  float* y_dev;
  uint64_t y_ld;
  uint32_t tokens, phase;
  uint32_t x_op;
  float eps;
} llr_program_op;
/* shard == NULL: one GPU.  Otherwise this rank's part of a row-sharded program, see below. */
typedef struct llr_program_shard {
  void* arena;
  size_t arena_bytes;
  uint32_t world, rank;
  void* const* peer_arenas;
} llr_program_shard;
int llr_program_create_ops(llr_exec* exec, const llr_program_op* ops, size_t n_ops,
                           const llr_program_shard* shard, llr_program** out);

/* Bound of the device-side waits of programs on data another CTA or rank produces, in
 * polls of roughly 0.1-0.3 us (default 2^20).  When a wait runs out the kernel records it,
 * every later wait of that launch returns at once, the launch finishes, and
 * llr_exec_synchronize reports LLR_ERR_CUDA; the executor stays usable [the reference's
 * executor stays usable after an error: native-cuda/src/main.rs:48-66]. */
int llr_exec_set_wait_limit(llr_exec* exec, uint32_t polls);

/* ---- row-sharded programs across GPUs -------------------------------------------
 * No counterpart in the reference (it runs on one device).  One process per GPU; rank g
 * holds rows [g*rows/G, (g+1)*rows/G) of every matrix as its own resident matrix and a
 * full-width copy of every result vector.  A sharded program is a program whose reducer
 * also stores each finished value, plain and tagged, into the same place of every other
 * rank's buffers (peer stores over NVLink), so the all-gather of result slices is part of
 * the launch: no collective call between products, and a reader spins on its own GPU's
 * copy of the pairs.  All ranks must create the same program (same entries, phases and
 * shard shapes) before any rank runs it, and run it the same number of times.  After a run,
 * a rank's plain results are complete once every rank has synchronized its stream.
 * A device-side wait is bounded (llr_exec_set_wait_limit): ranks must start a run within
 * that bound of each other (default about 0.2 s) or the run fails with LLR_ERR_CUDA.
 *
 * Buffers the peers write live in one arena per rank: llr_shared_alloc returns zeroed
 * device memory and a 64-byte handle another process opens with llr_shared_open (CUDA
 * IPC).  An arena is: LLR_ARENA_HEADER_BYTES that belong to the library | a result area
 * of R bytes | 2 R bytes for the tagged copies, R = ((arena_bytes - header) / 3) rounded
 * down to a multiple of 256.  Result buffers lie in the result area, at the same offsets on
 * every rank.  y_dev of an entry points at this rank's slice inside its own arena;
 * y_ld is the full row count (world * shard rows for a result that later entries read).
 * peer_arenas[g] is rank g's arena as opened here (the entry of this rank itself is
 * ignored).  world is 2..8; at most 4095 phases.  Arenas may be reused by a later
 * program once no rank is running the earlier one. */
#define LLR_ARENA_HEADER_BYTES 65536
typedef struct llr_ipc_handle { unsigned char bytes[64]; } llr_ipc_handle;
int llr_shared_alloc(llr_exec* exec, size_t bytes, void** dev, llr_ipc_handle* handle);
int llr_shared_open(llr_exec* exec, const llr_ipc_handle* handle, void** dev);
int llr_shared_close(llr_exec* exec, void* dev);
int llr_shared_free(llr_exec* exec, void* dev);
/* Strict phases, as llr_program_create; y_ld[i] as llr_program_op.y_ld (NULL: shard rows). */
int llr_program_create_sharded(llr_exec* exec, const llr_program_entry* entries, const uint64_t* y_ld,
                               size_t n_entries, void* arena, size_t arena_bytes, uint32_t world,
                               uint32_t rank, void* const* peer_arenas, llr_program** out);

/* ---- routed-expert FFN layer ----------------------------------------------------
 * One mixture-of-experts FFN layer as the reference runs it [langtax/src/decode.rs:
 * softmax_routed_layer :9938 -> route_softmax_tokens :9969 (router product, softmax,
 * top-k with ties to the lower id, weights optionally divided by max(sum, 2^-14))
 * -> grouped_routed_ffn :10006 (experts in ascending id: gather rows, gate and up
 * products, silu(g)*u, down product) -> scatter_expert_rows :10263 (out[t] += y*w)].
 * Everything runs on the device (the routing in the reference's order of operations:
 * sequential softmax sum, ties to the lower id); only the per-expert row counts visit
 * the host, which sizes the expert launches with them.  router: n_expert x n_embd; gate[e], up[e]: n_ff x n_embd; down[e]:
 * n_embd x n_ff (the ExpertParts of expertvm/src/store.rs:13-20, resident).
 * x: tokens*n_embd floats, out: tokens*n_embd floats (host).  sel_ids / sel_w
 * (tokens*n_used each, may be null) receive the routing decision.
 * Experts striped over GPUs (expert e on rank e % G, expertvm/src/place.rs:71-75): an
 * expert whose gate, up and down entries are all NULL is resident elsewhere; it takes part
 * in the routing, and its rows contribute zero to `out`, which is then this rank's partial
 * sum.  With two experts per token the sum of the ranks' partial outputs is bit-identical
 * to the single-device result (at most two non-zero terms per element). */
typedef struct llr_moe_layer {
  uint32_t n_expert, n_used, norm_w;
  const llr_matrix* router;
  const llr_matrix* const* gate;
  const llr_matrix* const* up;
  const llr_matrix* const* down;
} llr_moe_layer;
int llr_moe_ffn(llr_exec* exec, const llr_moe_layer* layer, size_t tokens, const float* x, size_t x_len,
                float* out, size_t out_len, int32_t* sel_ids, float* sel_w);
/* The two device-pointer halves of the layer, for expert parallelism with an exchange of routed rows between
 * ranks [an all-to-all of token rows; expertvm/src/place.rs:71-75 gives the owner of an expert]:
 * llr_moe_route_device: router product, softmax, top-k and router weights for `tokens` rows at x_dev;
 *   ids_dev / w_dev receive tokens * n_used entries in top-k order (only layer->router, n_expert, n_used and
 *   norm_w are read).  Enqueued on the executor's stream, no synchronization.
 * llr_moe_experts_device: gate/up products, silu(g)*u and the down product over packed rows that are already
 *   grouped by expert in ascending expert id: counts[e] rows for expert e (host array of n_expert entries;
 *   experts that are not resident here must have count 0), rows_dev and y_dev sum(counts) x n_embd floats.
 *   The caller multiplies by the router weights and adds a token's rows in ascending expert id. */
int llr_moe_route_device(llr_exec* exec, const llr_moe_layer* layer, size_t tokens, const float* x_dev,
                         int32_t* ids_dev, float* w_dev);
int llr_moe_experts_device(llr_exec* exec, const llr_moe_layer* layer, const uint32_t* counts,
                           const float* rows_dev, float* y_dev);

/* Expert parallelism with the exchange inside the library: experts striped over the ranks (expert e on rank
 * e % world, expertvm/src/place.rs:71-75), tokens sharded over the ranks, routed rows and their results moved
 * between GPUs by peer stores from the kernels that gather and scatter them [the all-to-all of token
 * rows; grouped_routed_ffn decode.rs:10006, scatter_expert_rows :10263].  One process per GPU (or several
 * executors of one process); no collective call, no host hop for rows; one small device-to-host copy of row counts
 * per run sizes the expert launches.
 *   arena: llr_moe_ep_arena_bytes(...) bytes of zeroed device memory per rank that the peers can write
 *   (llr_shared_alloc / llr_shared_open); peer_arenas[g] is rank g's arena as mapped in this process (the entry of
 *   this rank itself is ignored; may be NULL when world is 1).  layer: as llr_moe_ffn, with NULL gate/up/down for
 *   every expert e with e % world != rank.  max_tokens bounds the tokens of this rank per run.
 * A run is three calls, which llr_moe_ep_run makes in order:
 *   llr_moe_ep_dispatch  routes this rank's tokens (x_dev: tokens x n_embd floats on the device) and stores each
 *                        routed row into its expert's owner; enqueued, no synchronization;
 *   llr_moe_ep_serve     waits on the device, bounded by llr_exec_set_wait_limit, until every rank's rows for this
 *                        rank's experts have arrived, runs the experts on them and stores the results back into the
 *                        senders; synchronizes the stream once (row counts);
 *   llr_moe_ep_combine   waits (bounded) for the results of every owner and adds a token's rows times their router
 *                        weights in ascending expert id into out_dev; ids_dev / w_dev (tokens * n_used, may be NULL)
 *                        receive the routing decision; enqueued, no synchronization (llr_exec_synchronize ends the run).
 * Every rank makes the same sequence of runs (a rank with no tokens of its own still passes at least one).  Ranks must
 * reach a wait within the wait limit of each other, else the run fails with LLR_ERR_CUDA and the layer object has to be
 * re-created on every rank, on zeroed arenas: runs are counted from the creation of the layer, in the object and in the
 * arena alike, so an arena that served a layer before is refused (LLR_ERR_INVALID) until it has been zeroed again.  Several ranks driven from ONE thread (executors on one or several GPUs) call dispatch
 * on every rank first, then serve on every rank, then combine: no wait then ever spins.  With the f32-faithful
 * kernels (llr_exec_set_path(exec, 3)) the output is bit-identical to llr_moe_ffn on the same tokens. */
typedef struct llr_moe_ep llr_moe_ep;
size_t llr_moe_ep_arena_bytes(uint32_t n_expert, uint32_t n_used, size_t n_embd, uint32_t world, size_t max_tokens);
int llr_moe_ep_create(llr_exec* exec, const llr_moe_layer* layer, uint32_t world, uint32_t rank, size_t max_tokens,
                      void* arena, size_t arena_bytes, void* const* peer_arenas, llr_moe_ep** out);
int llr_moe_ep_dispatch(llr_moe_ep* ep, size_t tokens, const float* x_dev);
int llr_moe_ep_serve(llr_moe_ep* ep);
int llr_moe_ep_combine(llr_moe_ep* ep, float* out_dev, int32_t* ids_dev, float* w_dev);
int llr_moe_ep_run(llr_moe_ep* ep, size_t tokens, const float* x_dev, float* out_dev, int32_t* ids_dev, float* w_dev);
int llr_moe_ep_free(llr_moe_ep* ep);

/* ---- device-resident Llama walk ------------------------------------------------------
 * The per-token walk of the plain llama architecture with everything on the device
 * [langtax/src/decode.rs: Llama::forward_layers :2737-3097 -- rmsnorm_inplace :11498, the
 * q/k/v products, rope :11578 (adjacent-pair rotation), store_kv :12059 into a dense
 * [layer][kv_head][position][head_dim] f32 cache, attend_query :11126 with grouped-query
 * heads, attn_output, residual, rmsnorm, silu(gate)*up :2972-2996, ffn_down, residual; last
 * token's logits :3058-3079; greedy argmax sample.rs:293].  It stands where
 * Session::{prefill, decode} stand: the reference runs the element-wise steps on the host
 * between two executor calls (225 host round trips per token); here a generated token
 * never leaves the device, llr_session_decode enqueues all steps and synchronizes once.
 * Matrix products go through the executor's kernels (llr_exec_set_path applies); on the
 * automatic path a prompt chunk of 64 rows and more also runs its attention on the tensor
 * cores with binary16 operands and f32 accumulation (the tolerance of the 16-bit chunk GEMM;
 * llr_exec_set_path(exec, 3) keeps f32 arithmetic throughout).
 * Sums the reference adds sequentially (sum of squares, scores, softmax denominator) are
 * added in a fixed tree order: logits agree with the host walk to rounding, not bit for bit.
 * Norm weights are host f32 vectors of n_embd (NULL: all ones).  output == NULL: tied to
 * token_embd [decode.rs:2069-2072].  The model's matrices must outlive the session. */
typedef struct llr_llama_config {
  uint32_t n_layer, n_embd, n_head, n_head_kv, head_dim, n_ff, n_vocab, n_ctx;
  float rms_eps;   /* llama.attention.layer_norm_rms_epsilon, default 1e-5 [decode.rs:1958] */
  float rope_base; /* llama.rope.freq_base, default 10000 [decode.rs:2053] */
} llr_llama_config;
typedef struct llr_llama_layer {
  const llr_matrix *attn_q, *attn_k, *attn_v, *attn_output, *ffn_gate, *ffn_up, *ffn_down;
  const float *attn_norm, *ffn_norm;
  /* architecture=llama with routed experts [llama_moe_into decode.rs:10366: softmax over all experts, top-k, SwiGLU
   * experts, weights normalised with the 2^-14 clamp, no shared expert]: n_expert > 0 replaces the dense FFN of this
   * layer by the routed layer of llr_moe_ffn (ffn_gate / ffn_up / ffn_down are then not read and may be NULL).
   * ffn_gate_inp: n_expert x n_embd; the three arrays hold n_expert matrices each (n_ff x n_embd, n_ff x n_embd,
   * n_embd x n_ff; cfg.n_ff is the experts' width).  The arrays are copied at session creation.  For more than one row
   * the per-expert row counts of every such layer visit the host (one synchronization per layer); a step of one token
   * chooses its experts' products on the device (no host round trip, replayed from a graph like a dense step) when every
   * expert matrix is in a block-quantized format the streaming decode kernel takes and at most 8 experts are used. */
  uint32_t n_expert, n_expert_used;
  const llr_matrix* ffn_gate_inp;
  const llr_matrix* const* ffn_gate_exps;
  const llr_matrix* const* ffn_up_exps;
  const llr_matrix* const* ffn_down_exps;
} llr_llama_layer;
typedef struct llr_llama_model {
  llr_llama_config cfg;
  const llr_matrix* token_embd;
  const llr_matrix* output;
  const float* output_norm;
  const llr_llama_layer* layers; /* cfg.n_layer of them */
} llr_llama_model;
typedef struct llr_session llr_session;
/* One sequence, a KV pool that holds n_ctx positions. */
int llr_session_create(llr_exec* exec, const llr_llama_model* model, llr_session** out);
/* n_seq sequences over one paged KV pool [langtax/src/kv_page.rs:395-437]: kv_blocks blocks (0: enough for every sequence
 * to reach n_ctx) of block_tokens positions each; a sequence takes blocks from the pool as it grows and gives them back
 * when it is reset.  The single-sequence calls below act on sequence 0. */
int llr_session_create_paged(llr_exec* exec, const llr_llama_model* model, size_t n_seq, size_t kv_blocks,
                             size_t block_tokens, llr_session** out);
/* Appends n tokens at the session's position (in chunks of up to 512 rows through the batched
 * products) and leaves the logits of the last one in the session; last_logits (optional, host,
 * n_vocab floats) receives them. */
int llr_session_prefill(llr_session* session, const int32_t* tokens, size_t n, float* last_logits);
/* Greedy decode: n_gen times { token = argmax(logits); append token -> logits }.  out_ids receives
 * the n_gen tokens, out_margin (optional) each step's top-2 logit margin. */
int llr_session_decode(llr_session* session, size_t n_gen, int32_t* out_ids, float* out_margin);
/* Copies the current logits (n_vocab floats) to the host. */
int llr_session_logits(llr_session* session, float* logits, size_t n);
int llr_session_position(const llr_session* session, size_t* position);
int llr_session_reset(llr_session* session);
int llr_session_free(llr_session* session);
/* A ragged batch over several sequences in one pass [Engine::try_compute_batch langtax/src/engine.rs:1215-1274 ->
 * prefill_batch decode.rs:2579]: group g appends counts[g] tokens (tokens holds the groups one after the other) to
 * sequence seq_ids[g]; each sequence at most once per batch; at most 512 rows in all.  The groups are flattened in
 * ascending sequence id into one activation matrix, so every matrix product of the step runs once over all rows, while
 * attention and the KV cache go by each row's own sequence and position.  last_logits (optional, n_groups x n_vocab,
 * host) and next_ids (optional, n_groups, host) receive each group's last-row logits and their greedy argmax, in the
 * caller's group order.  A row's results do not depend on which other rows share its batch when the f32-faithful
 * products run (llr_exec_set_path(3)). */
int llr_session_batch(llr_session* session, size_t n_groups, const uint32_t* seq_ids, const uint32_t* counts,
                      const int32_t* tokens, float* last_logits, int32_t* next_ids);
int llr_session_seq_position(const llr_session* session, size_t seq, size_t* position);
int llr_session_seq_reset(llr_session* session, size_t seq);
/* Keeps the first n_keep positions of a sequence's cache and forgets the rest (their blocks return to the pool):
 * the device half of prompt reuse [KvCache::prompt keeps the longest common prefix and recomputes the remainder,
 * langtax/tests/native_cuda_parity.rs:243-256]. */
int llr_session_seq_truncate(llr_session* session, size_t seq, size_t n_keep);

/* Dequantize rows [row0, row0+n_rows) of a resident matrix to f32 on the
 * device and copy them to out (n_rows*cols floats, host).  Bit-exact
 * counterpart of dequant_<t>_row [quant.rs:7511, 7533, 7734, 7884, 7918, 8046,
 * 8083, 8783]. */
int llr_dequant_rows(llr_exec* exec, const llr_matrix* matrix, size_t row0, size_t n_rows,
                     float* out, size_t out_len);

/* Fill a resident matrix with seeded synthetic packed blocks on the device
 * (uniform quant bits from SplitMix64 [langtax/src/sample.rs:306-312], binary16
 * scales |n|*0.01 with n an exact-integer Irwin-Hall normal).  Benchmark
 * input generator; bit-identical to llama_rust_b200.synth on the host. */
int llr_matrix_synth(llr_exec* exec, uint8_t dtype, size_t rows, size_t cols, uint64_t seed,
                     llr_matrix** out);
/* Copy the packed bytes of a resident matrix back to the host. */
int llr_matrix_download(llr_exec* exec, const llr_matrix* matrix, void* out, size_t out_len);

#ifdef __cplusplus
}
#endif
#endif
