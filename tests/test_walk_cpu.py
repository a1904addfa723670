"""The oracle's Llama walk with routed experts against its own dense walk (CPU only): with every expert equal to the dense
FFN and the router weights normalised (norm_w, llama_moe_into langtax/src/decode.rs:10366), a token's output is
w1*y + w2*y with w1 + w2 = 1, so the logits agree with the dense walk to rounding, whatever the router selects."""
import numpy as np

import llama_walk as lw
from helpers import F32, Q4_K, random_packed


def test_moe_walk_with_identical_experts_equals_the_dense_walk(orc):
    cfg = dict(n_layer=2, n_embd=256, n_head=4, n_head_kv=2, head_dim=64, n_ff=256, n_vocab=40)
    rng = np.random.default_rng(11)
    tl = lw.tensor_list(cfg)
    kinds = [Q4_K] * len(tl)
    weights = [lw.center_q4k(random_packed(rng, Q4_K, r, c)) for _, _, r, c in tl]
    embd = lw.center_q4k(random_packed(rng, Q4_K, cfg["n_vocab"], cfg["n_embd"]))
    n_expert = 4
    moe = dict(n_used=2, router_kind=F32, expert_kind=Q4_K,
               router=[(rng.standard_normal(n_expert * cfg["n_embd"]) * 0.5).astype(np.float32).view(np.uint8) for _ in range(2)],
               gate=[[weights[7 * li + 4]] * n_expert for li in range(2)], up=[[weights[7 * li + 5]] * n_expert for li in range(2)],
               down=[[weights[7 * li + 6]] * n_expert for li in range(2)])
    prompt = np.array([1, 7, 3, 20], np.int32)
    ids_d, _, logits_d = lw.run_cpu(cfg, 16, weights, embd, prompt, 3, want_logits=True, kinds=kinds)
    ids_m, _, logits_m = lw.run_cpu(cfg, 16, weights, embd, prompt, 3, want_logits=True, kinds=kinds, moe=moe)
    assert np.array_equal(ids_d, ids_m)
    scale = np.abs(logits_d).max()
    assert np.abs(logits_d - logits_m).max() <= 2e-5 * scale, (np.abs(logits_d - logits_m).max(), scale)
    # and the routed walk does depend on its experts: another expert set changes the logits
    moe["down"] = [[lw.center_q4k(random_packed(rng, Q4_K, cfg["n_embd"], cfg["n_ff"]))] * n_expert for _ in range(2)]
    logits_x = lw.run_cpu(cfg, 16, weights, embd, prompt, 0, want_logits=True, kinds=kinds, moe=moe)[2]
    assert np.abs(logits_x - lw.run_cpu(cfg, 16, weights, embd, prompt, 0, want_logits=True, kinds=kinds)[2]).max() > 1e-3 * scale
