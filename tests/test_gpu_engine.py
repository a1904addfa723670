"""Model-level boundary suite: the flow of the reference's `end_to_end_models_match_scalar_snapshot`
(langtax/tests/native_cuda_parity.rs:196-290) on the device-resident session.  For tiny Llama models in three weight
formats: a contiguous and a paged cache (blocks of 2 positions) give the same logits for a prefill, three decode steps and
a divergent prompt that re-uses the cached prefix; every one of those logit vectors is checked against the CPU walk of the
oracle at the reference's tolerance (1e-4 + 1e-4 |e|); and an Engine that mixes differently sized prompt chunks and decode
tokens of several sequences in one batch generates what independent sessions generate.  The reference's snapshot comes
from a scalar build of the crate; here the scalar CPU walk of the oracle plays that part.  Its fourth model (a routed-
expert model) has no session here: the routed layer is checked at the layer level in test_gpu_moe.py."""
import numpy as np
import pytest

import llama_walk as lw
from helpers import F32, Q4_0, Q4_K, Q6_K, random_packed

pytestmark = pytest.mark.gpu

MODELS = {
    "llama-f32": (dict(n_layer=2, n_embd=64, n_head=4, n_head_kv=2, head_dim=16, n_ff=128, n_vocab=48), F32, F32, F32),
    "llama-q4_0": (dict(n_layer=2, n_embd=64, n_head=4, n_head_kv=2, head_dim=16, n_ff=128, n_vocab=48), Q4_0, Q4_0, F32),
    "llama-q4_k": (dict(n_layer=2, n_embd=256, n_head=4, n_head_kv=2, head_dim=64, n_ff=512, n_vocab=48), Q4_K, Q6_K, Q4_K),
    # architecture=llama with routed experts (llama_moe_into decode.rs:10366): four experts, two per token, F32 router
    "llama-moe-q4_k": (dict(n_layer=2, n_embd=256, n_head=4, n_head_kv=2, head_dim=64, n_ff=256, n_vocab=48, n_expert=4, n_used=2),
                       Q4_K, Q6_K, Q4_K),
}


def _model(name):
    cfg, kind, kind_v, embd_kind = MODELS[name]
    rng = np.random.default_rng(sum(name.encode()))
    tl = lw.tensor_list(cfg)
    kinds = [kind_v if (n.endswith("attn_v.weight") or n.endswith("ffn_down.weight") or n == "output.weight") else kind
             for n, _, _, _ in tl]
    # weights of order 1/sqrt(fan-in) so that logits are of order one and tokens compete
    weights = []
    for (n, _, rows, cols), k in zip(tl, kinds):
        w = random_packed(rng, k, rows, cols)
        if k == F32:
            w = (rng.standard_normal(rows * cols) / np.sqrt(cols)).astype(np.float32).view(np.uint8)
        elif k == Q4_K:
            w = lw.center_q4k(w)
        weights.append(w)
    if embd_kind == F32:
        embd = rng.standard_normal(cfg["n_vocab"] * cfg["n_embd"]).astype(np.float32).view(np.uint8)
    else:
        embd = lw.center_q4k(random_packed(rng, Q4_K, cfg["n_vocab"], cfg["n_embd"]))
    moe = None
    if cfg.get("n_expert"):
        E, FF, NE = cfg["n_embd"], cfg["n_ff"], cfg["n_expert"]
        moe = dict(n_used=cfg["n_used"], router_kind=F32, expert_kind=Q4_K,
                   router=[(rng.standard_normal(NE * E) * 0.5).astype(np.float32).view(np.uint8) for _ in range(cfg["n_layer"])],
                   gate=[[lw.center_q4k(random_packed(rng, Q4_K, FF, E)) for _ in range(NE)] for _ in range(cfg["n_layer"])],
                   up=[[lw.center_q4k(random_packed(rng, Q4_K, FF, E)) for _ in range(NE)] for _ in range(cfg["n_layer"])],
                   down=[[lw.center_q4k(random_packed(rng, Q4_K, E, FF)) for _ in range(NE)] for _ in range(cfg["n_layer"])])
        for i, (n, _, _, _) in enumerate(tl):  # the dense ffn tensors do not exist in such a model
            if ".ffn_" in n:
                weights[i] = None
    return cfg, tl, kinds, weights, embd_kind, embd, moe


def _check(actual, expected, what):  # native_cuda_parity.rs:150-158
    a, e = np.asarray(actual, np.float64), np.asarray(expected, np.float64)
    assert np.all(np.isfinite(a)) and np.all(np.abs(a - e) <= 1e-4 + 1e-4 * np.abs(e)), (what, np.abs(a - e).max())


def _sessions(ex, name, n_ctx=32, **kw):
    from llama_rust_b200 import Session
    cfg, tl, kinds, weights, embd_kind, embd, moe = _model(name)
    mats = [None if w is None else ex.upload(k, r, c, w) for (n, _, r, c), k, w in zip(tl, kinds, weights)]
    embd_mat = ex.upload(embd_kind, cfg["n_vocab"], cfg["n_embd"], embd)
    layers = [dict(zip(("attn_q", "attn_k", "attn_v", "attn_output", "ffn_gate", "ffn_up", "ffn_down"), mats[7 * li:7 * li + 7]))
              for li in range(cfg["n_layer"])]
    if moe is not None:
        E, FF, NE = cfg["n_embd"], cfg["n_ff"], cfg["n_expert"]
        for li, L in enumerate(layers):
            L["n_expert_used"] = moe["n_used"]
            L["ffn_gate_inp"] = ex.upload(F32, NE, E, moe["router"][li])
            L["ffn_gate_exps"] = [ex.upload(Q4_K, FF, E, w) for w in moe["gate"][li]]
            L["ffn_up_exps"] = [ex.upload(Q4_K, FF, E, w) for w in moe["up"][li]]
            L["ffn_down_exps"] = [ex.upload(Q4_K, E, FF, w) for w in moe["down"][li]]

    def make(**kw):
        return Session(ex, dict(cfg, n_ctx=n_ctx), embd_mat, layers, output=mats[-1], **kw)

    def cpu_logits(tokens):
        return lw.run_cpu(cfg, n_ctx, weights, embd, np.asarray(tokens, np.int32), 0, want_logits=True, kinds=kinds,
                          embd_kind=embd_kind, moe=moe)[2]

    def cpu_greedy(tokens, n):
        ids, margin, _ = lw.run_cpu(cfg, n_ctx, weights, embd, np.asarray(tokens, np.int32), n, kinds=kinds, embd_kind=embd_kind,
                                    moe=moe)
        return ids, margin
    return make, cpu_logits, cpu_greedy, (mats, embd_mat, layers)


@pytest.mark.parametrize("name", list(MODELS))
def test_dense_paged_and_reused_prompt_logits_match_the_scalar_walk(orc, name):
    from llama_rust_b200 import Executor
    ex = Executor(0)
    make, cpu_logits, _, keep = _sessions(ex, name)
    dense = make()
    paged = make(n_seq=1, kv_blocks=16, block_tokens=2)
    seq = [1, 2, 3]
    d, p = dense.prefill(seq, want_logits=True), paged.prefill(seq, want_logits=True)
    _check(p, d, f"{name}/prefill paged vs dense")
    _check(d, cpu_logits(seq), f"{name}/prefill")
    for step, token in enumerate([4, 5, 1]):
        seq.append(token)
        d, p = dense.prefill([token], want_logits=True), paged.prefill([token], want_logits=True)
        _check(p, d, f"{name}/decode-{step} paged vs dense")
        _check(d, cpu_logits(seq), f"{name}/decode-{step}")
    # a divergent full prompt re-uses the cached prefix [1, 2] and replaces the rest
    d, p = dense.prompt([1, 2, 4]), paged.prompt([1, 2, 4])
    assert dense.position == 3 and dense.cached_ids() == [1, 2, 4]
    _check(p, d, f"{name}/reused-prompt paged vs dense")
    _check(d, cpu_logits([1, 2, 4]), f"{name}/reused-prompt")
    # the whole prompt already cached: the last token is forwarded again (decode.rs:1178-1184)
    again = dense.prompt([1, 2, 4])
    assert np.array_equal(again.view(np.uint32), d.view(np.uint32)) and dense.position == 3
    # reuse_prefix rewinds and a token appended after it lands behind the kept prefix (decode.rs:16466-16476)
    dense.reset()
    dense.prefill([1, 2, 3, 4])
    assert dense.prompt_suffix([1, 2, 0]) == [0] and dense.position == 2 and dense.cached_ids() == [1, 2]
    dense.prefill([5])
    assert dense.position == 3 and dense.cached_ids() == [1, 2, 5]
    _check(dense.prompt([1, 2, 5]), cpu_logits([1, 2, 5]), f"{name}/append after rewind")
    dense.free(); paged.free(); ex.close()


@pytest.mark.parametrize("name", list(MODELS))
def test_engine_batches_generate_what_independent_sessions_generate(orc, name):  # native_cuda_parity.rs:258-289
    from llama_rust_b200 import Engine, EngineCfg, Executor
    ex = Executor(0)
    ex.set_path(3)  # a row's result must not depend on the rows that share its batch
    make, _, cpu_greedy, keep = _sessions(ex, name)
    prompts = [[1, 2, 3], [1, 2, 4, 5], [1, 2]]
    pool = make(n_seq=2, kv_blocks=64, block_tokens=2)
    engine = Engine(pool, EngineCfg(max_seqs=2, prefill_chunk=2))
    first, second = engine.add(prompts[0], 4), engine.add(prompts[1], 4)
    assert engine.step() > 0
    third = engine.add(prompts[2], 4)
    assert engine.waiting() == 1 and engine.active() == 2
    engine.run()
    assert engine.stats.gemm_peak > 1, "batched path unused"
    alone = make()
    for sid, prompt in zip((first, second, third), prompts):
        alone.reset()
        logits = alone.prefill(prompt, want_logits=True)
        expected = []
        for _ in range(4):
            tok = int(np.argmax(logits))
            expected.append(tok)
            logits = alone.prefill([tok], want_logits=True)
        out = engine.take(sid)
        assert out.prompt == prompt and out.generated == expected and out.completion_tokens == 4, (name, prompt)
        ids, margin = cpu_greedy(prompt, 4)
        n = 0
        while n < 4 and margin[n] > 1e-3:  # up to the first step the scalar walk itself decides narrowly
            n += 1
        assert expected[:n] == ids[:n].tolist(), (name, prompt, margin)
    assert engine.take(first) is None and engine.all_done()
    alone.free(); pool.free(); ex.close()


def test_engine_preempts_recomputes_and_stops_at_eos(orc):
    """A pool too small for all sequences at once: one loses its blocks, is recomputed from its prompt and the tokens it
    had generated, and still ends with the tokens it generates alone (engine.rs on_cap / replay)."""
    from llama_rust_b200 import Engine, EngineCfg, Executor
    ex = Executor(0)
    ex.set_path(3)
    make, _, _, keep = _sessions(ex, "llama-q4_k")
    prompts = [[1, 2, 3, 4, 5, 6], [7, 8, 9], [3, 1, 4, 1, 5, 9, 2, 6]]
    n_predict = 10
    alone = make()
    want = []
    for p in prompts:
        alone.reset()
        alone.prefill(p)
        want.append(alone.decode(n_predict)[0].tolist())
    # 3 sequences need up to (8 + 10) / 2 = 9 blocks each; 14 blocks do not hold them all
    pool = make(n_seq=3, kv_blocks=14, block_tokens=2)
    engine = Engine(pool, EngineCfg(max_seqs=3, prefill_chunk=4))
    ids = [engine.add(p, n_predict) for p in prompts]
    engine.run()
    assert engine.stats.preempts > 0
    for sid, p, w in zip(ids, prompts, want):
        out = engine.take(sid)
        assert out.generated == w, (p, out.generated, w)
    # eos ends a sequence early and is not part of its output; decode_first holds prompt chunks while others decode
    eos = want[0][3]
    pool.reset()
    engine = Engine(pool, EngineCfg(max_seqs=2, prefill_chunk=2, eos=eos, decode_first=True))
    a, b = engine.add(prompts[0], n_predict), engine.add(prompts[1], n_predict)
    engine.run()
    out = engine.take(a)
    cut = want[0].index(eos)
    assert out.generated == want[0][:cut] and out.completion_tokens == cut + 1
    wb = want[1][:want[1].index(eos)] if eos in want[1] else want[1]
    assert engine.take(b).generated == wb
    alone.free(); pool.free(); ex.close()
