"""Routed-expert FFN layer (llr_moe_ffn) against the oracle's restatement of the reference's
MoE walk (langtax/src/decode.rs:9938-10290): identical routing decisions, router weights to
f32 rounding, layer output within the matmul tolerances (integer path: relative 1e-5 of the
output scale per product, three chained products; tensor-core path: the bf16 bound)."""
import numpy as np
import pytest

from helpers import F32, Q4_K, random_packed

pytestmark = pytest.mark.gpu


def _layer(ex, rng, n_expert, n_embd, n_ff):
    router_w = (rng.standard_normal((n_expert, n_embd)) * 0.05).astype(np.float32)
    packs = {k: [random_packed(rng, Q4_K, r, c) for _ in range(n_expert)]
             for k, (r, c) in {"gate": (n_ff, n_embd), "up": (n_ff, n_embd), "down": (n_embd, n_ff)}.items()}
    mats = {k: [ex.upload(Q4_K, (n_ff if k != "down" else n_embd), (n_embd if k != "down" else n_ff), w) for w in v]
            for k, v in packs.items()}
    router = ex.upload(F32, n_expert, n_embd, router_w.view(np.uint8))
    return router_w, packs, mats, router


# 560 and 700 tokens over 8 experts put the busiest expert into the 160- and 192-row tiles of the grouped launch
@pytest.mark.parametrize("tokens,path,tol", [(1, 0, 3e-5), (24, 0, 3e-5), (300, 3, 3e-5), (300, 0, 2e-2),
                                             (560, 0, 2e-2), (700, 0, 2e-2), (1100, 0, 2e-2)])
def test_moe_layer_matches_reference_walk(orc, tokens, path, tol):
    from llama_rust_b200 import Executor
    ex = Executor(0)
    rng = np.random.default_rng(500 + tokens)
    n_expert, n_used, n_embd, n_ff = 8, 2, 512, 1024
    router_w, packs, mats, router = _layer(ex, rng, n_expert, n_embd, n_ff)
    x = rng.standard_normal((tokens, n_embd)).astype(np.float32)
    ref_out, ref_ids, ref_w = orc.moe_ffn(n_used, True, F32, router_w.view(np.uint8), Q4_K, packs["gate"], packs["up"],
                                          packs["down"], n_embd, n_ff, x)
    ex.set_path(path)
    out, ids, w = ex.moe_ffn(router, mats["gate"], mats["up"], mats["down"], n_used, True, x)
    assert np.array_equal(ids, ref_ids), "routing decisions differ"
    assert np.allclose(w, ref_w, rtol=2e-6, atol=1e-7)
    assert np.all(np.isfinite(out))
    scale = max(1.0, float(np.abs(ref_out).max()))
    assert np.abs(out - ref_out).max() <= tol * scale, f"max err {np.abs(out - ref_out).max():.3e} vs scale {scale:.3g}"
    # every token's output is the weighted sum of exactly its two experts: zeroing x of one
    # token must zero only that token's row
    x2 = x.copy()
    x2[0] = 0.0
    out2, _, _ = ex.moe_ffn(router, mats["gate"], mats["up"], mats["down"], n_used, True, x2)
    assert np.all(out2[0] == 0.0)
    ex.close()


def test_moe_layer_validates_shapes():
    from llama_rust_b200 import Executor, NativeCudaError
    ex = Executor(0)
    rng = np.random.default_rng(9)
    router_w, packs, mats, router = _layer(ex, rng, 4, 256, 512)
    x = np.zeros((3, 256), np.float32)
    with pytest.raises(NativeCudaError):
        ex.moe_ffn(router, mats["gate"], mats["up"], mats["down"], 5, True, x)  # n_used > n_expert
    with pytest.raises(NativeCudaError):
        ex.moe_ffn(router, mats["down"], mats["up"], mats["down"], 2, True, x)  # wrong shapes
    out, ids, w = ex.moe_ffn(router, mats["gate"], mats["up"], mats["down"], 2, False, x)
    assert np.all(out == 0.0) and ids.shape == (3, 2)
    ex.close()


def test_striped_experts_partials_sum_to_the_single_device_layer(orc):
    """Experts striped e % G: each "rank" runs the layer with only its experts resident (the others
    NULL) and the partial outputs are added.  With two experts per token that sum is bit-identical
    to the layer with every expert resident.  One GPU plays both ranks here; the two-process
    variant is in test_gpu_sharded_program.py."""
    from llama_rust_b200 import Executor, NativeCudaError
    n_expert, n_used, n_embd, n_ff = 8, 2, 1024, 2048
    ex = Executor(0)
    gate = [ex.synth(Q4_K, n_ff, n_embd, 10 + e) for e in range(n_expert)]
    up = [ex.synth(Q4_K, n_ff, n_embd, 30 + e) for e in range(n_expert)]
    down = [ex.synth(Q4_K, n_embd, n_ff, 50 + e) for e in range(n_expert)]
    rng = np.random.default_rng(3)
    router = ex.upload(F32, n_expert, n_embd, (rng.standard_normal((n_expert, n_embd)) * 0.05).astype(np.float32).view(np.uint8).reshape(-1))
    for tokens in (5, 96):  # per-expert decode kernels, grouped tensor-core launches
        x = rng.standard_normal((tokens, n_embd)).astype(np.float32)
        full, ids, w = ex.moe_ffn(router, gate, up, down, n_used, True, x)
        total = np.zeros_like(full)
        for world, rank in ((2, 0), (2, 1)):
            keep = [e % world == rank for e in range(n_expert)]
            part, ids_r, w_r = ex.moe_ffn(router, [m if k else None for m, k in zip(gate, keep)],
                                          [m if k else None for m, k in zip(up, keep)],
                                          [m if k else None for m, k in zip(down, keep)], n_used, True, x)
            assert np.array_equal(ids_r, ids) and np.array_equal(w_r, w)
            total = total + part
        assert np.array_equal(total, full), f"tokens={tokens}: {np.abs(total - full).max()}"
    with pytest.raises(NativeCudaError):  # no resident expert at all
        ex.moe_ffn(router, [None] * n_expert, [None] * n_expert, [None] * n_expert, n_used, True, x)
    ex.close()


@pytest.mark.parametrize("world", [1, 2, 3])
def test_expert_parallel_layer_with_peer_stores_on_one_gpu(world):
    """llr_moe_ep_*: experts striped e % world, tokens sharded, routed rows and results moved by peer stores.  One GPU
    plays every rank here (one executor per rank, the stages called rank after rank with a synchronize in between, so
    no wait ever spins); the output of every rank's tokens is bit-identical to the single-device layer on the f32-
    faithful path.  Three runs with changing token counts go through both halves of the arena; world = 3 leaves
    rank 2 with two experts and ranks 0 and 1 with three."""
    import torch
    from llama_rust_b200 import Executor, NativeCudaError
    from llama_rust_b200.executor import moe_ep_arena_bytes
    n_expert, n_used, n_embd, n_ff, t_max = 8, 2, 512, 1024, 48
    rng = np.random.default_rng(77 + world)
    router_w = (rng.standard_normal((n_expert, n_embd)) * 0.05).astype(np.float32)
    ref = Executor(0)
    ref.set_path(3)
    full = {k: [ref.synth(Q4_K, r, c, seed + e) for e in range(n_expert)]
            for k, (r, c, seed) in {"gate": (n_ff, n_embd, 100), "up": (n_ff, n_embd, 200), "down": (n_embd, n_ff, 300)}.items()}
    ref_router = ref.upload(F32, n_expert, n_embd, router_w.view(np.uint8).reshape(-1))
    exs = [Executor(0) for _ in range(world)]
    nbytes = moe_ep_arena_bytes(n_expert, n_used, n_embd, world, t_max)
    arenas = [ex.shared_alloc(nbytes)[0] for ex in exs]
    eps, mines, routers = [], [], []
    for r, ex in enumerate(exs):
        ex.set_path(3)
        mine = {k: [ex.synth(Q4_K, m.rows, m.cols, seed + e) if e % world == r else None for e, m in enumerate(full[k])]
                for k, seed in (("gate", 100), ("up", 200), ("down", 300))}
        router = ex.upload(F32, n_expert, n_embd, router_w.view(np.uint8).reshape(-1))
        eps.append(ex.moe_ep(router, mine["gate"], mine["up"], mine["down"], n_used, True, world, r, t_max, arenas[r], nbytes, arenas))
        mines.append(mine)
        routers.append(router)
    for run, counts in enumerate(([5, 48, 17], [48, 1, 30], [9, 9, 9])):
        counts = counts[:world]
        xs = [rng.standard_normal((n, n_embd)).astype(np.float32) for n in counts]
        want, want_ids, want_w = ref.moe_ffn(ref_router, full["gate"], full["up"], full["down"], n_used, True, np.concatenate(xs))
        x_t = [torch.from_numpy(x).cuda() for x in xs]
        out_t = [torch.full((n, n_embd), float("nan"), device="cuda") for n in counts]
        ids_t = [torch.zeros((n, n_used), dtype=torch.int32, device="cuda") for n in counts]
        w_t = [torch.zeros((n, n_used), dtype=torch.float32, device="cuda") for n in counts]
        torch.cuda.synchronize()
        for r in range(world):
            eps[r].dispatch(counts[r], x_t[r].data_ptr())
        for ex in exs:
            ex.synchronize()
        for r in range(world):
            eps[r].serve()
        for ex in exs:
            ex.synchronize()
        for r in range(world):
            eps[r].combine(out_t[r].data_ptr(), ids_t[r].data_ptr(), w_t[r].data_ptr())
        for ex in exs:
            ex.synchronize()
        got = np.concatenate([o.cpu().numpy() for o in out_t])
        assert np.array_equal(np.concatenate([i.cpu().numpy() for i in ids_t]), want_ids), run
        assert np.array_equal(np.concatenate([v.cpu().numpy() for v in w_t]).view(np.uint32), want_w.view(np.uint32)), run
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), (run, float(np.abs(got - want).max()))
    # the stages of a run come in order, and a rank holds exactly the experts e % world == rank
    with pytest.raises(NativeCudaError):
        eps[0].serve()
    with pytest.raises(NativeCudaError):
        eps[0].dispatch(t_max + 1, x_t[0].data_ptr())
    if world > 1:
        with pytest.raises(NativeCudaError, match="e % world"):  # rank 0's experts offered as rank 1
            exs[0].moe_ep(routers[0], mines[0]["gate"], mines[0]["up"], mines[0]["down"], n_used, True, world, 1, t_max, arenas[0], nbytes, arenas)
    for ep in eps:
        ep.free()
    # a second layer on arenas that still carry the first one's run counts would take stale flags for new ones: refused
    with pytest.raises(NativeCudaError, match="has served"):
        exs[0].moe_ep(routers[0], mines[0]["gate"], mines[0]["up"], mines[0]["down"], n_used, True, world, 0, t_max, arenas[0], nbytes, arenas)
    for ex, a in zip(exs, arenas):
        ex.shared_free(a)
        ex.close()
    ref.close()


def test_expert_parallel_wait_for_an_absent_rank_runs_out_and_the_executor_stays_usable():
    """A rank whose peer never delivers: the bounded device-side wait of serve() runs out (the flag is simply never
    set, nothing faults), the call reports LLR_ERR_CUDA with the reason, and the executor serves the next product."""
    import torch
    from llama_rust_b200 import Executor, NativeCudaError
    from llama_rust_b200.executor import moe_ep_arena_bytes
    n_expert, n_used, n_embd, n_ff, t_max = 4, 2, 256, 512, 8
    ex = Executor(0)
    ex.set_wait_limit(2000)  # about a millisecond
    rng = np.random.default_rng(5)
    router = ex.upload(F32, n_expert, n_embd, (rng.standard_normal((n_expert, n_embd)) * 0.05).astype(np.float32).view(np.uint8).reshape(-1))
    mine = {k: [ex.synth(Q4_K, r, c, 7 + e) if e % 2 == 0 else None for e in range(n_expert)]
            for k, (r, c) in {"gate": (n_ff, n_embd), "up": (n_ff, n_embd), "down": (n_embd, n_ff)}.items()}
    nbytes = moe_ep_arena_bytes(n_expert, n_used, n_embd, 2, t_max)
    arena0, arena1 = ex.shared_alloc(nbytes)[0], ex.shared_alloc(nbytes)[0]  # "rank 1" is memory nobody works on
    ep = ex.moe_ep(router, mine["gate"], mine["up"], mine["down"], n_used, True, 2, 0, t_max, arena0, nbytes, [arena0, arena1])
    x = torch.from_numpy(rng.standard_normal((t_max, n_embd)).astype(np.float32)).cuda()
    torch.cuda.synchronize()
    ep.dispatch(t_max, x.data_ptr())
    with pytest.raises(NativeCudaError, match="did not deliver"):
        ep.serve()
    w = random_packed(rng, Q4_K, 32, 256)
    m = ex.upload(Q4_K, 32, 256, w)
    y = np.empty(32, np.float32)
    ex.gemv_resident(m, np.ones(256, np.float32), y)
    assert np.all(np.isfinite(y))
    ep.free()
    ex.shared_free(arena0)
    ex.shared_free(arena1)
    ex.close()


def test_config5_full_size_layer(orc):
    """benchmark config 5 at its full size: 8 experts, top-2, 4096 / 14336, Q4_K experts generated on
    the device from seeds (792 MB), F32 router, 64 tokens.  One CPU walk of the layer (the
    oracle, 4.5e10 FLOP) is compared with the f32-faithful decode path and with the automatic
    choice (grouped tensor-core launches)."""
    from llama_rust_b200 import Executor, synth
    n_expert, n_used, n_embd, n_ff, tokens = 8, 2, 4096, 14336, 64
    with Executor(0) as ex:
        mats = {k: [ex.synth(Q4_K, r, c, synth.tensor_seed(5, f"config5.{k}.{e}")) for e in range(n_expert)]
                for k, (r, c) in {"gate": (n_ff, n_embd), "up": (n_ff, n_embd), "down": (n_embd, n_ff)}.items()}
        packs = {k: [ex.download(m) for m in v] for k, v in mats.items()}
        router_w = (synth.activations(n_expert * n_embd, synth.tensor_seed(5, "config5.router")) * np.float32(0.05)).reshape(n_expert, n_embd)
        router = ex.upload(F32, n_expert, n_embd, router_w.view(np.uint8).reshape(-1))
        x = synth.activations(tokens * n_embd, synth.tensor_seed(5, "config5.x")).reshape(tokens, n_embd)
        ref_out, ref_ids, ref_w = orc.moe_ffn(n_used, True, F32, router_w.view(np.uint8).reshape(-1), Q4_K, packs["gate"],
                                              packs["up"], packs["down"], n_embd, n_ff, x)
        scale = max(1.0, float(np.abs(ref_out).max()))
        for path, tol in ((3, 3e-5), (0, 2e-2)):
            ex.set_path(path)
            out, ids, w = ex.moe_ffn(router, mats["gate"], mats["up"], mats["down"], n_used, True, x)
            assert np.array_equal(ids, ref_ids), "routing decisions differ"
            # router logits are 4096-term f32 sums in another order than the CPU's: 1e-5 relative, the
            # reference's tolerance for its own row kernels
            assert np.allclose(w, ref_w, rtol=1e-5, atol=1e-6)
            assert np.all(np.isfinite(out))
            err = float(np.abs(out - ref_out).max())
            assert err <= tol * scale, f"path {path}: max err {err:.3e} vs scale {scale:.3g}"


def test_config5_full_size_layer_512_tokens_on_sampled_tokens(orc):
    """benchmark config 5 with 512 tokens (1024 routed rows, about 128 per expert: the wide grouped tiles).  The
    device runs the whole layer; a token's output depends on that token alone, so the CPU walk of the layer is run
    on every eighth token (64 tokens) and compared with the device's rows for those tokens: routing identical, the
    f32-faithful path within 3e-5 of the output scale, the grouped tensor-core path within 2e-2."""
    from llama_rust_b200 import Executor, synth
    n_expert, n_used, n_embd, n_ff, tokens = 8, 2, 4096, 14336, 512
    with Executor(0) as ex:
        mats = {k: [ex.synth(Q4_K, r, c, synth.tensor_seed(5, f"config5.{k}.{e}")) for e in range(n_expert)]
                for k, (r, c) in {"gate": (n_ff, n_embd), "up": (n_ff, n_embd), "down": (n_embd, n_ff)}.items()}
        packs = {k: [ex.download(m) for m in v] for k, v in mats.items()}
        router_w = (synth.activations(n_expert * n_embd, synth.tensor_seed(5, "config5.router")) * np.float32(0.05)).reshape(n_expert, n_embd)
        router = ex.upload(F32, n_expert, n_embd, router_w.view(np.uint8).reshape(-1))
        x = synth.activations(tokens * n_embd, synth.tensor_seed(5, "config5.x512")).reshape(tokens, n_embd)
        sel = np.arange(0, tokens, 8)
        ref_out, ref_ids, ref_w = orc.moe_ffn(n_used, True, F32, router_w.view(np.uint8).reshape(-1), Q4_K, packs["gate"],
                                              packs["up"], packs["down"], n_embd, n_ff, np.ascontiguousarray(x[sel]))
        scale = max(1.0, float(np.abs(ref_out).max()))
        for path, tol in ((3, 3e-5), (0, 2e-2)):
            ex.set_path(path)
            out, ids, w = ex.moe_ffn(router, mats["gate"], mats["up"], mats["down"], n_used, True, x)
            assert np.all(np.isfinite(out))
            assert np.array_equal(ids[sel], ref_ids), "routing decisions differ"
            assert np.allclose(w[sel], ref_w, rtol=1e-5, atol=1e-6)
            err = float(np.abs(out[sel] - ref_out).max())
            assert err <= tol * scale, f"path {path}: max err {err:.3e} vs scale {scale:.3g}"
            print(f"config5 T=512 path {path}: max err {err:.3e} of scale {scale:.3g}; rows per expert {np.bincount(ids.reshape(-1), minlength=n_expert).tolist()}")
