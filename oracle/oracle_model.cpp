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



// ---- dense Llama walk (langtax/src/decode.rs:2710-3097 for the plain llama architecture:
// RMSNorm :11498, q/k/v products, RoPE-NORM per head :11578, KV store :12059 in the dense
// layout [layer][kv_head][t][hd], GQA attention :11126, attn_output, residual, RMSNorm,
// SwiGLU FFN :2972-2996, residual; LogitsKind::Last :3058-3079; greedy argmax sample.rs:293).
// Every matrix product goes through `matmul`: either the oracle's own CPU kernels or a
// callback, so the very same host code can drive another executor and only the products
// differ between the two runs.

// tensors[layer*7 + {0 q,1 k,2 v,3 o,4 gate,5 up,6 down}], tensors[n_layer*7] = output;
// token_embd separately.  kinds[] parallel.  norms are all-ones F32 (attn_norm, ffn_norm,
// output_norm): the synthetic model of the greedy-identity tests has no trained norms.
static int walk_matmul(const orc_llama_cfg* c, orc_matmul_cb cb, void* user, const uint8_t* const* tensors,
                       const int* kinds, int id, int64_t rows, int64_t cols, int64_t n, const float* x,
                       float* y, int threads) {
  if (cb) return cb(user, id, n, x, y);
  (void)c;
  const int64_t len = orc_row_bytes(kinds[id], cols) * rows;
  return orc_gemm(kinds[id], cols, n, tensors[id], len, x, n * cols, y, n * rows, 1, threads);
}

int orc_llama_generate(const orc_llama_cfg* c, orc_matmul_cb cb, void* user, const uint8_t* const* tensors,
                       const int* kinds, int embd_kind, const uint8_t* token_embd,
                       int (*embd_cb)(void* user, int32_t token, float* row), const int32_t* prompt,
                       int n_prompt, int n_gen, int32_t* out_ids, float* out_margin, float* last_logits,
                       int threads) {
  return orc_llama_generate_moe(c, nullptr, cb, user, tensors, kinds, embd_kind, token_embd, embd_cb, prompt, n_prompt, n_gen,
                                out_ids, out_margin, last_logits, threads);
}

// The same walk with the dense FFN of every layer replaced by the routed experts of `moe` when it is given
// (llama_moe_into decode.rs:10366: architecture=llama with n_expert > 0, norm_w = true, no shared expert).
int orc_llama_generate_moe(const orc_llama_cfg* c, const orc_llama_moe* moe, orc_matmul_cb cb, void* user,
                           const uint8_t* const* tensors, const int* kinds, int embd_kind, const uint8_t* token_embd,
                           int (*embd_cb)(void* user, int32_t token, float* row), const int32_t* prompt,
                           int n_prompt, int n_gen, int32_t* out_ids, float* out_margin, float* last_logits,
                           int threads) {
  const int64_t E = c->n_embd, H = c->n_head, HKV = c->n_head_kv, HD = c->head_dim, FF = c->n_ff, V = c->n_vocab;
  const int64_t QW = H * HD, KVW = HKV * HD;
  if (n_prompt <= 0 || n_prompt + n_gen > c->n_ctx || H % HKV != 0) return ORC_ERR_SIZE;
  const int64_t nmax = n_prompt;
  std::vector<float> x((size_t)(nmax * E)), residual((size_t)(nmax * E)), q((size_t)(nmax * QW)), k((size_t)(nmax * KVW)),
      v((size_t)(nmax * KVW)), attn((size_t)(nmax * QW)), proj((size_t)(nmax * E)), gate((size_t)(nmax * FF)),
      up((size_t)(nmax * FF)), ffn((size_t)(nmax * E)), xn((size_t)E), logits((size_t)V), scores((size_t)c->n_ctx);
  std::vector<float> ones((size_t)E, 1.0f);
  std::vector<int32_t> sel_ids;
  std::vector<float> sel_w;
  std::vector<float> cache_k((size_t)c->n_layer * HKV * c->n_ctx * HD), cache_v(cache_k.size());
  auto kv_off = [&](int64_t layer, int64_t h, int64_t t) { return ((layer * HKV + h) * c->n_ctx + t) * HD; };
  const int64_t embd_rb = orc_row_bytes(embd_kind, E);

  int64_t pos0 = 0;
  std::vector<int32_t> toks(prompt, prompt + n_prompt);
  for (int step = 0; step <= n_gen; ++step) {
    const int64_t n = (int64_t)toks.size();
    for (int64_t t = 0; t < n; ++t) {
      int rc = embd_cb ? embd_cb(user, toks[(size_t)t], x.data() + t * E)
                       : orc_dequant_row(embd_kind, E, token_embd + (int64_t)toks[(size_t)t] * embd_rb, embd_rb,
                                         x.data() + t * E, E);
      if (rc) return rc;
    }
    for (int64_t li = 0; li < c->n_layer; ++li) {
      const int base = (int)li * 7;
      int rc;
      std::memcpy(residual.data(), x.data(), sizeof(float) * (size_t)(n * E));
      for (int64_t t = 0; t < n; ++t) orc_rmsnorm(x.data() + t * E, ones.data(), E, c->rms_eps);
      if ((rc = walk_matmul(c, cb, user, tensors, kinds, base + 0, QW, E, n, x.data(), q.data(), threads))) return rc;
      if ((rc = walk_matmul(c, cb, user, tensors, kinds, base + 1, KVW, E, n, x.data(), k.data(), threads))) return rc;
      if ((rc = walk_matmul(c, cb, user, tensors, kinds, base + 2, KVW, E, n, x.data(), v.data(), threads))) return rc;
      for (int64_t t = 0; t < n; ++t) {
        const int64_t p = pos0 + t;
        orc_rope_norm(k.data() + t * KVW, HKV, HD, HD, p, c->rope_base);
        for (int64_t h = 0; h < HKV; ++h) {
          std::memcpy(cache_k.data() + kv_off(li, h, p), k.data() + t * KVW + h * HD, sizeof(float) * (size_t)HD);
          std::memcpy(cache_v.data() + kv_off(li, h, p), v.data() + t * KVW + h * HD, sizeof(float) * (size_t)HD);
        }
      }
      const float score_scale = 1.0f / std::sqrt((float)(uint16_t)HD);
      const int64_t gqa = H / HKV;
      for (int64_t t = 0; t < n; ++t) {
        const int64_t p = pos0 + t, seq = p + 1;
        float* qt = q.data() + t * QW;
        orc_rope_norm(qt, H, HD, HD, p, c->rope_base);
        for (int64_t hq = 0; hq < H; ++hq) {
          const int64_t hkv = hq / gqa;
          const float* qv = qt + hq * HD;
          for (int64_t s = 0; s < seq; ++s) {
            const float* kv = cache_k.data() + kv_off(li, hkv, s);
            float dot = 0.0f;
            for (int64_t i = 0; i < HD; ++i) {
              const float pr = qv[i] * kv[i];
              dot += pr;
            }
            scores[(size_t)s] = dot * score_scale;
          }
          orc_softmax(scores.data(), seq);
          float* dst = attn.data() + t * QW + hq * HD;
          for (int64_t i = 0; i < HD; ++i) dst[i] = 0.0f;
          for (int64_t s = 0; s < seq; ++s) {
            const float* vv = cache_v.data() + kv_off(li, hkv, s);
            const float st = scores[(size_t)s];
            for (int64_t i = 0; i < HD; ++i) {
              const float pr = st * vv[i];
              dst[i] += pr;
            }
          }
        }
      }
      if ((rc = walk_matmul(c, cb, user, tensors, kinds, base + 3, E, QW, n, attn.data(), proj.data(), threads))) return rc;
      for (int64_t i = 0; i < n * E; ++i) x[(size_t)i] = proj[(size_t)i] + residual[(size_t)i];
      std::memcpy(residual.data(), x.data(), sizeof(float) * (size_t)(n * E));
      for (int64_t t = 0; t < n; ++t) orc_rmsnorm(x.data() + t * E, ones.data(), E, c->rms_eps);
      if (moe) {
        const int64_t NE = moe->n_expert;
        sel_ids.resize((size_t)(n * moe->n_used));
        sel_w.resize((size_t)(n * moe->n_used));
        if ((rc = orc_moe_ffn(moe->n_expert, moe->n_used, 1, moe->router_kind, moe->router[li], orc_row_bytes(moe->router_kind, E) * NE,
                              moe->expert_kind, moe->gate + li * NE, moe->up + li * NE, moe->down + li * NE, E, FF, n, x.data(),
                              ffn.data(), sel_ids.data(), sel_w.data(), threads)))
          return rc;
      } else {
      if ((rc = walk_matmul(c, cb, user, tensors, kinds, base + 4, FF, E, n, x.data(), gate.data(), threads))) return rc;
      if ((rc = walk_matmul(c, cb, user, tensors, kinds, base + 5, FF, E, n, x.data(), up.data(), threads))) return rc;
      for (int64_t i = 0; i < n * FF; ++i) {
        const float a = orc_silu(gate[(size_t)i]);
        gate[(size_t)i] = a * up[(size_t)i];
      }
      if ((rc = walk_matmul(c, cb, user, tensors, kinds, base + 6, E, FF, n, gate.data(), ffn.data(), threads))) return rc;
      }
      for (int64_t i = 0; i < n * E; ++i) x[(size_t)i] = ffn[(size_t)i] + residual[(size_t)i];
    }
    std::memcpy(xn.data(), x.data() + (n - 1) * E, sizeof(float) * (size_t)E);
    orc_rmsnorm(xn.data(), ones.data(), E, c->rms_eps);
    int rc = walk_matmul(c, cb, user, tensors, kinds, c->n_layer * 7, V, E, 1, xn.data(), logits.data(), threads);
    if (rc) return rc;
    if (step == n_gen) break;
    const int64_t best = orc_argmax(logits.data(), V);
    float second = -INFINITY;
    for (int64_t i = 0; i < V; ++i)
      if (i != best && logits[(size_t)i] > second) second = logits[(size_t)i];
    out_ids[step] = (int32_t)best;
    if (out_margin) out_margin[step] = logits[(size_t)best] - second;
    pos0 += n;
    toks.assign(1, (int32_t)best);
  }
  if (last_logits) std::memcpy(last_logits, logits.data(), sizeof(float) * (size_t)V);
  return ORC_OK;
}
}  // extern "C"
