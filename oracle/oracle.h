/* CPU oracle for the quantized matrix-product path of mingley/llama-rust.
 *
 * TEST INFRASTRUCTURE ONLY.  This is a CPU restatement of the reference's
 * algorithm (block formats, binary16 decode, row dequantization, scalar and
 * AVX2 row dots, GEMV/GEMM entry points with their validation, the host-side
 * model walk) used as the checker for the CUDA path and as the timed CPU
 * baseline.  Nothing in the shipped library links or calls it.
 *
 * Parity is PINNED: the restatement reproduces the reference's own golden
 * output of langtax/q8_gemv.c (y_checksum=80e188057fa1eef0, README.md:276)
 * bit for bit, agrees with that file compiled unmodified (oracle/_ref), and
 * reproduces the reference's in-tree known-answer tests (tests/test_oracle_*).
 *
 * dtype tags are the reference's `GemmKind as u8` (langtax/src/quant.rs:6645):
 * F16=0 BF16=1 F32=2 Q4_1=5 Q5_0=6 Q5_1=7 Q4_0=12 Q8_0=13 Q4_K=17 Q5_K=18 Q6_K=19.
 */
#ifndef LLR_ORACLE_H
#define LLR_ORACLE_H
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
  ORC_F16 = 0, ORC_BF16 = 1, ORC_F32 = 2, ORC_Q4_1 = 5, ORC_Q5_0 = 6, ORC_Q5_1 = 7,
  ORC_Q4_0 = 12, ORC_Q8_0 = 13, ORC_Q4_K = 17, ORC_Q5_K = 18, ORC_Q6_K = 19
};

/* error codes (0 = ok) mirroring QuantError variants, quant.rs:4120-4160 */
enum {
  ORC_OK = 0,
  ORC_ERR_UNALIGNED_COLS = 1, /* QuantError::UnalignedCols */
  ORC_ERR_SIZE = 2,           /* QuantError::Size */
  ORC_ERR_DTYPE = 3,          /* tag outside the eleven above */
  ORC_ERR_OVERFLOW = 4
};

/* fp16.rs:4-62, 137-151 */
float    orc_f16_to_f32(uint16_t h);
uint16_t orc_f32_to_f16(float f);       /* truncating, subnormals kept */
float    orc_bf16_to_f32(uint16_t h);
uint16_t orc_f32_to_bf16(float f);      /* round to nearest even */

/* elements per block / bytes per block / bytes per row (quant.rs:86-163, 4210) */
int     orc_block_elems(int kind);
int     orc_block_bytes(int kind);
int64_t orc_row_bytes(int kind, int64_t n_cols); /* <0: -ORC_ERR_* */

/* packers (quant.rs:4342, 4594, 4639, 4680, 4852, 4977, 5712) */
void orc_pack_q8_0_block(float d, const int8_t qs[32], uint8_t out[34]);
void orc_pack_q4_0_from_i4(float d, const int8_t v[32], uint8_t out[18]);
void orc_pack_q5_0_block(float d, const uint8_t q5[32], uint8_t out[22]);
void orc_pack_q5_1_block(float d, float m, const uint8_t q5[32], uint8_t out[24]);
void orc_pack_q4_k_block(float d, float dmin, const uint8_t sc[8], const uint8_t mn[8],
                         const uint8_t q4[256], uint8_t out[144]);
void orc_pack_q6_k_block(float d, const int8_t sc[16], const int8_t q[256], uint8_t out[210]);
void orc_pack_q4_1_block(float d, float m, const uint8_t q4[32], uint8_t out[20]);            /* quant.rs:4611 */
void orc_pack_q5_k_block(float d, float dmin, const uint8_t sc[8], const uint8_t mn[8],
                         const uint8_t q5[256], uint8_t out[176]);                              /* quant.rs:5019 */
void orc_pack_f16(const float* v, int64_t n, uint8_t* out);
void orc_pack_bf16(const float* v, int64_t n, uint8_t* out);

/* dequant_<t>_row (quant.rs:7511-8853).  Returns ORC_* */
int orc_dequant_row(int kind, int64_t n_cols, const uint8_t* row, int64_t row_len,
                    float* y, int64_t y_len);
/* whole matrix, rows*n_cols floats */
int orc_dequant_matrix(int kind, int64_t n_rows, int64_t n_cols, const uint8_t* w,
                       int64_t w_len, float* y);

/* scalar vec_dot_<t>_f32_row (quant.rs:8963-10163): one sequential f32
 * accumulator in the reference's element order. */
float orc_dot_row_scalar(int kind, const uint8_t* row, int64_t row_len, const float* x,
                         int64_t x_len);
/* AVX2+FMA(+F16C) row dots (langtax/src/simd/x86.rs:208-775).  Falls back to
 * the scalar kernel when the CPU lacks the features, as simd/mod.rs:135-271. */
float orc_dot_row_simd(int kind, const uint8_t* row, int64_t row_len, const float* x,
                       int64_t x_len);
int orc_have_simd(void);

/* gemv_<t>_f32 / gemm_<t>_f32 (quant.rs:6144-6478, 6760-6888, 7176-7221).
 * simd: 0 scalar rows, 1 AVX2 rows.  threads: 0 = min(hw, rows, 10) as
 * pool.rs:70-79, 1 = sequential, n = exactly n (still <= rows).
 * y is token-major y[t*n_rows + r]; x is x[t*n_cols + c]. */
int orc_gemv(int kind, int64_t n_cols, const uint8_t* w, int64_t w_len, const float* x,
             int64_t x_len, float* y, int64_t y_len, int simd, int threads);
int orc_gemm(int kind, int64_t n_cols, int64_t n_tokens, const uint8_t* w, int64_t w_len,
             const float* x, int64_t x_len, float* y, int64_t y_len, int simd, int threads);

/* f64 dot of the f32-dequantized weights with x: the boundary oracle of
 * langtax/tests/native_cuda_parity.rs:124-148.  out is token-major doubles. */
int orc_gemm_f64(int kind, int64_t n_cols, int64_t n_tokens, const uint8_t* w, int64_t w_len,
                 const float* x, int64_t x_len, double* out, int64_t out_len);

/* Q8_0 x Q8_0 GEMV (quant.rs:6080, 8860; x86.rs:459): the kernel the
 * reference's published golden checksum belongs to. */
int orc_gemv_q8_0_q8_0(int64_t n_cols, const uint8_t* w, int64_t w_len, const uint8_t* xq,
                       int64_t xq_len, float* y, int64_t y_len, int simd);
/* demo_gguf data generator (langtax/src/main.rs:40-102, q8_gemv.c:143-161) */
void orc_demo_q8_0(int64_t n_cols, int64_t n_rows, uint8_t* w, uint8_t* xq);
/* FNV-1a over output bit patterns (q8_gemv.c:103-112) */
uint64_t orc_y_checksum(const float* y, int64_t n);

/* ---- host-side model walk (decode.rs) used for greedy-identity checks ---- */
void  orc_rmsnorm(float* x, const float* w, int64_t n, float eps);            /* :11498 */
void  orc_rope_norm(float* v, int64_t n_heads, int64_t head_dim, int64_t n_rot,
                    int64_t pos, float base);                                   /* :11578 */
void  orc_softmax(float* v, int64_t n);                                         /* :12021 */
float orc_silu(float v);                                                        /* :11826 */
int64_t orc_argmax(const float* v, int64_t n);                                  /* sample.rs:293 */
void  orc_topk(const float* p, int64_t n, int64_t k, int32_t* ids);            /* :11363 */

/* Routed-expert FFN layer (decode.rs:9938-10290): router GEMM, softmax, top-k (ties to the
 * lower id), optional weight normalisation with the 2^-14 clamp, then experts in ascending
 * order: gather rows, gate & up GEMM, silu(g)*u, down GEMM, out[t] += y * w. */
int orc_moe_ffn(int n_expert, int n_used, int norm_w, int router_kind, const uint8_t* router,
                int64_t router_len, int expert_kind, const uint8_t* const* gate,
                const uint8_t* const* up, const uint8_t* const* down, int64_t n_embd, int64_t n_ff,
                int64_t tokens, const float* x, float* out, int32_t* sel_ids, float* sel_w,
                int threads);

/* Dense Llama walk (decode.rs:2710-3097, plain llama architecture, norm weights all ones):
 * prefill of the whole prompt as one batch (LogitsKind::Last), then greedy decode.  Matrix
 * products go through `cb` when given (tensor_id = layer*7 + {0 q,1 k,2 v,3 o,4 gate,5 up,
 * 6 down}, n_layer*7 = output), else through the oracle's CPU kernels on tensors[]/kinds[].
 * Embedding rows come from `embd_cb` when given, else from dequant_<t>_row of token_embd.
 * out_margin[i] = top-1 minus top-2 logit at generated token i. */
typedef int (*orc_matmul_cb)(void* user, int tensor_id, int64_t n_tokens, const float* x, float* y);
typedef struct orc_llama_cfg {
  int32_t n_layer, n_embd, n_head, n_head_kv, head_dim, n_ff, n_vocab, n_ctx;
  float rms_eps, rope_base;
} orc_llama_cfg;
int orc_llama_generate(const orc_llama_cfg* c, orc_matmul_cb cb, void* user, const uint8_t* const* tensors,
                       const int* kinds, int embd_kind, const uint8_t* token_embd,
                       int (*embd_cb)(void* user, int32_t token, float* row), const int32_t* prompt,
                       int n_prompt, int n_gen, int32_t* out_ids, float* out_margin, float* last_logits,
                       int threads);

/* The same walk for architecture=llama with n_expert > 0 (llama_moe_into decode.rs:10366): every layer's dense FFN is
 * the routed-expert layer above with norm_w = 1.  router[layer]; gate / up / down[layer * n_expert + e]; the dense
 * ffn entries of tensors[] are not read.  moe == NULL: the dense walk. */
typedef struct orc_llama_moe {
  int32_t n_expert, n_used, router_kind, expert_kind;
  const uint8_t* const* router;
  const uint8_t* const* gate;
  const uint8_t* const* up;
  const uint8_t* const* down;
} orc_llama_moe;
int orc_llama_generate_moe(const orc_llama_cfg* c, const orc_llama_moe* moe, orc_matmul_cb cb, void* user,
                           const uint8_t* const* tensors, const int* kinds, int embd_kind, const uint8_t* token_embd,
                           int (*embd_cb)(void* user, int32_t token, float* row), const int32_t* prompt,
                           int n_prompt, int n_gen, int32_t* out_ids, float* out_margin, float* last_logits,
                           int threads);

#ifdef __cplusplus
}
#endif
#endif
