"""Generates tests/golden/config3_golden.json: the greedy tokens of benchmark config 3 as the CPU
oracle (AVX2 restatement of the reference's row kernels + the reference's host walk) produces
them.  Llama-3-8B-shaped random-init model, Q4_K_M-style mix, weights from the seeded host
generator (bit-identical to the device generator), 512 uniform-random prompt ids, 128 greedy
tokens.  Takes several minutes and ~6 GB of RAM.

  python tests/golden/make_config3.py [recipe] [n_layer]
      recipe: plain (uniform bits in every field, as the configuration states; default) or
              centered (llama_walk.center_q4k applied to the Q4_K tensors: a model whose logits compete)
      n_layer < 32 for a quick trial
"""
import json
import os
import sys
import time

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
import llama_walk as lw  # noqa: E402
from llama_rust_b200 import synth  # noqa: E402

BASE_SEED, PROMPT_SEED, N_PROMPT, N_GEN = 3, 3003, 512, 128


def main():
    cfg = dict(lw.LLAMA3_8B)
    recipe = sys.argv[1] if len(sys.argv) > 1 else "plain"
    assert recipe in ("plain", "centered")
    if len(sys.argv) > 2:
        cfg["n_layer"] = int(sys.argv[2])
    tl = lw.tensor_list(cfg)
    t0 = time.time()
    if recipe == "centered":
        weights, embd = lw.centered_weights(cfg, BASE_SEED)
    else:
        weights = [synth.packed_matrix(dt, rows, cols, synth.tensor_seed(BASE_SEED, name)) for name, dt, rows, cols in tl]
        embd = synth.packed_matrix(lw.Q4_K, cfg["n_vocab"], cfg["n_embd"], synth.tensor_seed(BASE_SEED, "token_embd.weight"))
    print(f"weights generated in {time.time() - t0:.0f}s", flush=True)
    prompt = lw.prompt_ids(N_PROMPT, cfg["n_vocab"], PROMPT_SEED)
    t0 = time.time()
    ids, margin, logits = lw.run_cpu(cfg, N_PROMPT + N_GEN, weights, embd, prompt, N_GEN, threads=0, want_logits=True)
    out = {"config": cfg, "recipe": recipe, "logit_scale": float(np.abs(logits).max()), "base_seed": BASE_SEED, "prompt_seed": PROMPT_SEED, "n_prompt": N_PROMPT, "n_gen": N_GEN,
           "ids": ids.tolist(), "top2_margin": [float(m) for m in margin], "distinct_tokens": int(len(set(ids.tolist()))),
           "min_margin": float(margin.min()), "cpu_seconds": time.time() - t0}
    stem = "config3_golden" if recipe == "plain" else "config3_centered_golden"
    name = f"{stem}.json" if cfg["n_layer"] == 32 else f"{stem}_trial_{cfg['n_layer']}.json"
    with open(os.path.join(HERE, name), "w") as f:
        json.dump(out, f)
    print(name, "distinct", out["distinct_tokens"], "min margin", out["min_margin"], f"{out['cpu_seconds']:.0f}s")


if __name__ == "__main__":
    main()
