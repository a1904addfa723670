// CPU oracle, model-level pieces.  TEST INFRASTRUCTURE ONLY (see oracle.h).
//
// Restates the routed-expert FFN of langtax/src/decode.rs: router GEMM + per-token
// softmax / top-k / weight normalisation (softmax_select_tokens :9983-10003, topk_into
// :11363, fill_router_weights :11392, MOE_NORM_W_CLAMP :321), bucketing and the
// ascending-expert grouped FFN (grouped_routed_ffn :10006, grouped_one_expert :10062,
// swiglu_expert_gemm :10148, scatter_expert_rows :10263), with the matrix products done by
// the oracle's own gemm (AVX2 row kernels).  Compile with -ffp-contract=off.
#include <cmath>
#include <cstring>
#include <vector>

#include "oracle.h"

extern "C" {

// sel_ids / sel_w: tokens * n_used, in the reference's top-k order (descending weight,
// ties to the lower expert id).  out: tokens * n_embd.
int orc_moe_ffn(int n_expert, int n_used, int norm_w, int router_kind, const uint8_t* router,
                int64_t router_len, int expert_kind, const uint8_t* const* gate,
                const uint8_t* const* up, const uint8_t* const* down, int64_t n_embd, int64_t n_ff,
                int64_t tokens, const float* x, float* out, int32_t* sel_ids, float* sel_w,
                int threads) {
  const int64_t up_len = orc_row_bytes(expert_kind, n_embd) * n_ff;
  const int64_t down_len = orc_row_bytes(expert_kind, n_ff) * n_embd;
  if (up_len < 0 || down_len < 0 || n_used <= 0 || n_used > n_expert) return ORC_ERR_SIZE;
  std::vector<float> logits((size_t)(tokens * n_expert));
  int rc = orc_gemm(router_kind, n_embd, tokens, router, router_len, x, tokens * n_embd,
                    logits.data(), tokens * n_expert, 1, threads);
  if (rc) return rc;
  std::vector<std::vector<int64_t>> buckets((size_t)n_expert);
  for (int64_t t = 0; t < tokens; ++t) {
    float* row = logits.data() + t * n_expert;
    orc_softmax(row, n_expert);
    orc_topk(row, n_expert, n_used, sel_ids + t * n_used);
    float wsum = 0.0f;
    for (int j = 0; j < n_used; ++j) {
      sel_w[t * n_used + j] = row[sel_ids[t * n_used + j]];
      wsum += sel_w[t * n_used + j];
    }
    if (norm_w) {
      if (wsum < 1.0f / 16384.0f) wsum = 1.0f / 16384.0f;
      for (int j = 0; j < n_used; ++j) sel_w[t * n_used + j] /= wsum;
    }
    for (int j = 0; j < n_used; ++j) buckets[(size_t)sel_ids[t * n_used + j]].push_back(t);
  }
  std::memset(out, 0, sizeof(float) * (size_t)(tokens * n_embd));
  std::vector<float> pack, g, u, y;
  for (int e = 0; e < n_expert; ++e) {  // ascending expert id: fixes the f32 accumulation order
    const std::vector<int64_t>& toks = buckets[(size_t)e];
    const int64_t n = (int64_t)toks.size();
    if (n == 0) continue;
    pack.resize((size_t)(n * n_embd));
    for (int64_t i = 0; i < n; ++i)
      std::memcpy(pack.data() + i * n_embd, x + toks[(size_t)i] * n_embd, sizeof(float) * (size_t)n_embd);
    g.resize((size_t)(n * n_ff));
    u.resize((size_t)(n * n_ff));
    y.resize((size_t)(n * n_embd));
    if ((rc = orc_gemm(expert_kind, n_embd, n, gate[e], up_len, pack.data(), n * n_embd, g.data(), n * n_ff, 1, threads))) return rc;
    if ((rc = orc_gemm(expert_kind, n_embd, n, up[e], up_len, pack.data(), n * n_embd, u.data(), n * n_ff, 1, threads))) return rc;
    for (size_t i = 0; i < g.size(); ++i) {
      const float a = orc_silu(g[i]);
      g[i] = a * u[i];
    }
    if ((rc = orc_gemm(expert_kind, n_ff, n, down[e], down_len, g.data(), n * n_ff, y.data(), n * n_embd, 1, threads))) return rc;
    for (int64_t i = 0; i < n; ++i) {
      const int64_t t = toks[(size_t)i];
      float w = 0.0f;
      for (int j = 0; j < n_used; ++j)
        if (sel_ids[t * n_used + j] == e) { w = sel_w[t * n_used + j]; break; }
      float* dst = out + t * n_embd;
      const float* src = y.data() + i * n_embd;
      for (int64_t c = 0; c < n_embd; ++c) {
        const float term = src[c] * w;
        dst[c] += term;
      }
    }
  }
  return ORC_OK;
}

}  // extern "C"
