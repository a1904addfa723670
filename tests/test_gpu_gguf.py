"""From a model file to products on the device: tensors of a GGUF image go to the executor packed (whole, one expert part,
a run of rows: QuantMat / quant_mat_rows, langtax/src/decode.rs:476-485, :9680-9713), the crate-facing product keyed by
the tensor's blob range hits without reading the weights again, and a Llama-family file loads into a device-resident
session that generates what a session built from the same arrays generates."""
import numpy as np
import pytest

import gguf_files as gf
import llama_walk as lw
from helpers import F16, Q4_K, Q6_K, Q8_0, check_kernel, random_packed

pytestmark = pytest.mark.gpu
GGML_OF = {2: 0, 0: 1, 1: 30, 12: 2, 6: 6, 7: 7, 13: 8, 17: 12, 19: 14}  # executor tag -> ggml type id


def test_tensors_parts_and_row_ranges_upload_packed(orc):
    from llama_rust_b200 import Executor, NativeCudaError
    from llama_rust_b200.gguf import GgufFile
    rng = np.random.default_rng(3)
    cols, rows, parts = 512, 48, 3
    mats = {"w_q4k": (Q4_K, random_packed(rng, Q4_K, rows, cols)), "w_q6k": (Q6_K, random_packed(rng, Q6_K, rows, cols)),
            "w_q8": (Q8_0, random_packed(rng, Q8_0, rows, cols)), "w_f16": (F16, random_packed(rng, F16, rows, cols))}
    exps = random_packed(rng, Q4_K, parts * rows, cols)
    tensors = [(n, GGML_OF[dt], (cols, rows), w.tobytes()) for n, (dt, w) in mats.items()]
    tensors.append(("blk.0.ffn_up_exps.weight", 12, (cols, rows, parts), exps.tobytes()))
    tensors.append(("w_q2k", 10, (cols, rows), bytes(rows * cols // 256 * 84)))
    g = GgufFile(gf.write_gguf(gf.DEFAULT_KV, tensors))
    ex = Executor(0)
    x = rng.standard_normal(cols).astype(np.float32)
    for name, (dt, w) in mats.items():
        m = g.upload(ex, name)
        assert (m.dtype, m.rows, m.cols) == (dt, rows, cols)
        assert np.array_equal(ex.download(m), w)
        y = np.empty(rows, np.float32)
        ex.gemv_resident(m, x, y)
        check_kernel(y, orc.gemv(dt, cols, w, x, rows), name)
        m.free()
        part = g.upload(ex, name, first_row=16, n_rows=24)       # quant_mat_rows
        rb = len(w) // rows
        assert part.rows == 24 and np.array_equal(ex.download(part), w[16 * rb:40 * rb])
        part.free()
    rb = len(exps) // (parts * rows)
    for p in range(parts):                                          # one expert of a 3-D tensor
        m = g.upload(ex, "blk.0.ffn_up_exps.weight", part=p)
        assert m.rows == rows and np.array_equal(ex.download(m), exps[p * rows * rb:(p + 1) * rows * rb])
        m.free()
    m = g.upload(ex, "blk.0.ffn_up_exps.weight", part=2, first_row=8, n_rows=8)
    assert np.array_equal(ex.download(m), exps[(2 * rows + 8) * rb:(2 * rows + 16) * rb])
    m.free()
    for bad in (dict(name="absent"), dict(name="w_q8", part=1), dict(name="w_q8", first_row=40, n_rows=9),
                dict(name="w_q8", first_row=1), dict(name="blk.0.ffn_up_exps.weight", part=3)):
        with pytest.raises(NativeCudaError) as err:
            g.upload(ex, **bad)
        assert err.value.code == 1
    # the keyed crate-facing product: one upload, then hits that never look at the bytes
    y = np.empty(rows, np.float32)
    before = ex.counters()["uploads"]
    for _ in range(3):
        g.matmul(ex, "w_q6k", 1, x, y)
        check_kernel(y, orc.gemv(Q6_K, cols, mats["w_q6k"][1], x, rows), "keyed")
    g.matmul(ex, "blk.0.ffn_up_exps.weight", 1, x, y, part=1)
    check_kernel(y, orc.gemv(Q4_K, cols, exps[rows * rb:2 * rows * rb], x, rows), "keyed expert")
    g.matmul(ex, "blk.0.ffn_up_exps.weight", 1, x, y, part=1)
    c = ex.counters()
    assert (c["cache_misses"], c["cache_hits"], c["uploads"] - before) == (2, 3, 2)
    ex.pin_key(g.key("w_q6k"))
    assert g.key("w_q6k")[1] == g.tensor("w_q6k").start
    ex.close()
    g.close()


def test_a_llama_file_loads_into_a_session(orc):
    from llama_rust_b200 import Executor
    from llama_rust_b200.gguf import GgufFile, llama_config, load_llama
    from test_gpu_session import _session
    cfg = dict(n_layer=2, n_embd=512, n_head=8, n_head_kv=2, head_dim=64, n_ff=1024, n_vocab=1000)
    n_ctx, n_gen = 64, 12
    tl = lw.tensor_list(cfg)
    weights, embd = lw.centered_weights(cfg, 17)
    rng = np.random.default_rng(8)
    norms = [(1 + 0.1 * rng.standard_normal(512).astype(np.float32), 1 + 0.1 * rng.standard_normal(512).astype(np.float32))
             for _ in range(cfg["n_layer"])]
    out_norm = 1 + 0.1 * rng.standard_normal(512).astype(np.float32)
    kv = gf.DEFAULT_KV + [("general.architecture", gf.STRING, "llama"), ("llama.block_count", gf.U32, 2),
                          ("llama.embedding_length", gf.U32, 512), ("llama.feed_forward_length", gf.U32, 1024),
                          ("llama.attention.head_count", gf.U32, 8), ("llama.attention.head_count_kv", gf.U32, 2),
                          ("llama.rope.freq_base", gf.F32, 10000.0), ("llama.attention.layer_norm_rms_epsilon", gf.F32, 1e-5),
                          ("llama.context_length", gf.U32, n_ctx)]
    tensors = [("token_embd.weight", 12, (512, 1000), embd.tobytes()), ("output_norm.weight", 0, (512,), out_norm.tobytes())]
    tensors += [(name, GGML_OF[dt], (c, r), w.tobytes()) for (name, dt, r, c), w in zip(tl, weights)]
    for i, (a, f) in enumerate(norms):
        tensors += [(f"blk.{i}.attn_norm.weight", 0, (512,), a.tobytes()), (f"blk.{i}.ffn_norm.weight", 0, (512,), f.tobytes())]
    g = GgufFile(gf.write_gguf(kv, tensors))
    got = llama_config(g)
    assert {k: got[k] for k in cfg} == cfg and got["n_ctx"] == n_ctx
    ex = Executor(0)
    ex.set_path(3)
    s = load_llama(ex, g)
    prompt = lw.prompt_ids(9, cfg["n_vocab"], 4)
    first = s.prefill(prompt, want_logits=True)
    ids, _ = s.decode(n_gen)
    # the same model from the arrays
    mats = [ex.upload(dt, r, c, w) for (name, dt, r, c), w in zip(tl, weights)]
    embd_mat = ex.upload(Q4_K, 1000, 512, embd)
    from llama_rust_b200 import Session
    layers = []
    for li in range(2):
        L = dict(zip(("attn_q", "attn_k", "attn_v", "attn_output", "ffn_gate", "ffn_up", "ffn_down"), mats[7 * li:7 * li + 7]))
        L["attn_norm"], L["ffn_norm"] = norms[li]
        layers.append(L)
    ref = Session(ex, dict(cfg, n_ctx=n_ctx), embd_mat, layers, output=mats[14], output_norm=out_norm)
    want_first = ref.prefill(prompt, want_logits=True)
    want_ids, _ = ref.decode(n_gen)
    assert np.array_equal(first.view(np.uint32), want_first.view(np.uint32)) and np.array_equal(ids, want_ids)
    assert len(set(ids.tolist())) > 1
    s.free(); ref.free(); ex.close(); g.close()


def test_a_llama_file_with_routed_experts_loads_into_a_session(orc):
    """architecture=llama with llama.expert_count > 0: the router and the 3-D ffn_*_exps tensors (one expert per slice of the
    slowest dimension, as the reference's quant_mat takes them, decode.rs:9612) become a session whose logits are those of
    the session built from the same arrays."""
    from llama_rust_b200 import Executor, Session
    from llama_rust_b200.gguf import GgufFile, llama_config, load_llama
    from helpers import F32, random_packed
    cfg = dict(n_layer=2, n_embd=256, n_head=4, n_head_kv=2, head_dim=64, n_ff=256, n_vocab=64)
    NE, NU, E, FF, n_ctx = 4, 2, 256, 256, 32
    rng = np.random.default_rng(21)
    tl = [t for t in lw.tensor_list(cfg) if ".ffn_" not in t[0]]
    dense = [lw.center_q4k(random_packed(rng, Q4_K, r, c)) if dt == Q4_K else random_packed(rng, dt, r, c) for _, dt, r, c in tl]
    embd = lw.center_q4k(random_packed(rng, Q4_K, 64, E))
    router = [(rng.standard_normal((NE, E)) * 0.5).astype(np.float32) for _ in range(2)]
    exps = {k: [[lw.center_q4k(random_packed(rng, Q4_K, r, c)) for _ in range(NE)] for _ in range(2)]
            for k, (r, c) in (("ffn_gate_exps", (FF, E)), ("ffn_up_exps", (FF, E)), ("ffn_down_exps", (E, FF)))}
    kv = gf.DEFAULT_KV + [("general.architecture", gf.STRING, "llama"), ("llama.block_count", gf.U32, 2),
                          ("llama.embedding_length", gf.U32, E), ("llama.feed_forward_length", gf.U32, FF),
                          ("llama.attention.head_count", gf.U32, 4), ("llama.attention.head_count_kv", gf.U32, 2),
                          ("llama.expert_count", gf.U32, NE), ("llama.expert_used_count", gf.U32, NU),
                          ("llama.context_length", gf.U32, n_ctx)]
    ones = np.ones(E, np.float32)
    tensors = [("token_embd.weight", 12, (E, 64), embd.tobytes()), ("output_norm.weight", 0, (E,), ones.tobytes())]
    tensors += [(name, GGML_OF[dt], (c, r), w.tobytes()) for (name, dt, r, c), w in zip(tl, dense)]
    for i in range(2):
        tensors += [(f"blk.{i}.attn_norm.weight", 0, (E,), ones.tobytes()), (f"blk.{i}.ffn_norm.weight", 0, (E,), ones.tobytes()),
                    (f"blk.{i}.ffn_gate_inp.weight", 0, (E, NE), router[i].tobytes())]
        for k, (r, c) in (("ffn_gate_exps", (FF, E)), ("ffn_up_exps", (FF, E)), ("ffn_down_exps", (E, FF))):
            tensors.append((f"blk.{i}.{k}.weight", 12, (c, r, NE), b"".join(w.tobytes() for w in exps[k][i])))
    g = GgufFile(gf.write_gguf(kv, tensors))
    got = llama_config(g)
    assert got["n_expert"] == NE and got["n_expert_used"] == NU
    ex = Executor(0)
    ex.set_path(3)
    s = load_llama(ex, g)
    prompt = [3, 9, 27, 17, 5]
    first = s.prefill(prompt, want_logits=True)
    ids, _ = s.decode(6)
    by_name = {name: ex.upload(dt, r, c, w) for (name, dt, r, c), w in zip(tl, dense)}
    layers = []
    for i in range(2):
        L = {k: by_name[f"blk.{i}.{k}.weight"] for k in ("attn_q", "attn_k", "attn_v", "attn_output")}
        L["ffn_gate_inp"] = ex.upload(F32, NE, E, router[i].view(np.uint8).reshape(-1))
        L["n_expert_used"] = NU
        for k, (r, c) in (("ffn_gate_exps", (FF, E)), ("ffn_up_exps", (FF, E)), ("ffn_down_exps", (E, FF))):
            L[k] = [ex.upload(Q4_K, r, c, w) for w in exps[k][i]]
        layers.append(L)
    embd_mat = ex.upload(Q4_K, 64, E, embd)  # the session reads the model's matrices for as long as it lives
    ref = Session(ex, dict(cfg, n_ctx=n_ctx), embd_mat, layers, output=by_name["output.weight"], output_norm=ones)
    want_first = ref.prefill(prompt, want_logits=True)
    want_ids, _ = ref.decode(6)
    assert np.all(np.isfinite(first))
    assert np.array_equal(first.view(np.uint32), want_first.view(np.uint32)) and np.array_equal(ids, want_ids)
    # token by token a step chooses its experts' products on the device (no row counts on the host); the prompt as one
    # chunk goes through the packed rows: the same bits either way
    ref.reset()
    for tok in prompt[:-1]:
        ref.prefill([tok])
    single = ref.prefill(prompt[-1:], want_logits=True)
    assert np.array_equal(single.view(np.uint32), want_first.view(np.uint32))
    ids_again, _ = ref.decode(6)
    assert np.array_equal(ids_again, want_ids)
    s.free(); ref.free(); ex.close(); g.close()
