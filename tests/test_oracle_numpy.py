"""A second statement of the block formats, vectorized in numpy from the layouts alone (quant.rs:86-163 sizes, the
ggml bit packing), against the C++ oracle's block-by-block dequantizer: two independently written decoders must
produce the same bits on random blocks.  The oracle is the checker of every GPU parity test, so a layout slip in it
would go unnoticed wherever the CUDA kernels shared the slip; this file closes that loop on the CPU."""
import numpy as np
import pytest

from helpers import ALL, random_packed

F32 = np.float32


def _f16(b):  # two bytes per value, little endian -> f32 (exact)
    return np.ascontiguousarray(b).view("<f2").astype(F32)


def _blocks(w, nbytes):
    return np.ascontiguousarray(w, dtype=np.uint8).reshape(-1, nbytes)


def _fifth_bits(qh_bytes):  # u32 little endian -> [blocks, 32] bits
    qh = np.ascontiguousarray(qh_bytes).view("<u4").reshape(-1, 1)
    return ((qh >> np.arange(32, dtype=np.uint32)) & 1).astype(np.int32)


def _nibbles(q):  # [blocks, 16] bytes -> [blocks, 32]: low nibbles first, then high nibbles
    return np.concatenate([q & 15, q >> 4], axis=1).astype(np.int32)


def _k_scales(s):  # [blocks, 12] -> 6-bit scales and mins, [blocks, 8] each
    s = s.astype(np.int32)
    sc = np.concatenate([s[:, 0:4] & 63, (s[:, 8:12] & 15) | ((s[:, 0:4] >> 6) << 4)], axis=1)
    mn = np.concatenate([s[:, 4:8] & 63, (s[:, 8:12] >> 4) | ((s[:, 4:8] >> 6) << 4)], axis=1)
    return sc, mn


def _k_codes(qs):  # [blocks, 128] -> [blocks, 8 sub-blocks, 32]: sub-block 2g low nibbles, 2g+1 high nibbles of bytes 32g..
    q = qs.reshape(-1, 4, 32).astype(np.int32)
    return np.stack([q & 15, q >> 4], axis=2).reshape(-1, 8, 32)


def dequant(kind_name, w):
    if kind_name == "Q8_0":
        b = _blocks(w, 34)
        return b[:, 2:].view(np.int8).astype(F32) * _f16(b[:, :2])
    if kind_name == "Q4_0":
        b = _blocks(w, 18)
        return (_nibbles(b[:, 2:]) - 8).astype(F32) * _f16(b[:, :2])
    if kind_name == "Q4_1":
        b = _blocks(w, 20)
        return _nibbles(b[:, 4:]).astype(F32) * _f16(b[:, :2]) + _f16(b[:, 2:4])
    if kind_name == "Q5_0":
        b = _blocks(w, 22)
        return (_nibbles(b[:, 6:]) + 16 * _fifth_bits(b[:, 2:6]) - 16).astype(F32) * _f16(b[:, :2])
    if kind_name == "Q5_1":
        b = _blocks(w, 24)
        return (_nibbles(b[:, 8:]) + 16 * _fifth_bits(b[:, 4:8])).astype(F32) * _f16(b[:, :2]) + _f16(b[:, 2:4])
    if kind_name in ("Q4_K", "Q5_K"):
        five = kind_name == "Q5_K"
        b = _blocks(w, 176 if five else 144)
        d, dmin = _f16(b[:, 0:2]), _f16(b[:, 2:4])
        sc, mn = _k_scales(b[:, 4:16])
        q = _k_codes(b[:, 48:176] if five else b[:, 16:144])
        if five:  # bit k of mask byte l is the fifth bit of element l of sub-block k
            mask = b[:, 16:48].astype(np.int32)
            q = q + 16 * ((mask[:, None, :] >> np.arange(8)[None, :, None]) & 1)
        a = (d * sc.astype(F32))[:, :, None]        # rounded once
        m = (dmin * mn.astype(F32))[:, :, None]     # rounded once
        return (a * q.astype(F32) - m).reshape(len(b), 256)
    if kind_name == "Q6_K":
        b = _blocks(w, 210)
        ql = b[:, 0:128].reshape(-1, 2, 2, 32).astype(np.int32)  # [block, half, which 32 bytes, l]
        qh = b[:, 128:192].reshape(-1, 2, 32).astype(np.int32)
        sc = b[:, 192:208].view(np.int8).astype(F32).reshape(-1, 2, 8)
        d = _f16(b[:, 208:210])
        lo = np.stack([ql[:, :, 0] & 15, ql[:, :, 1] & 15, ql[:, :, 0] >> 4, ql[:, :, 1] >> 4], axis=2)  # [block, half, 4, 32]
        hi = np.stack([(qh >> s) & 3 for s in (0, 2, 4, 6)], axis=2)
        q = (lo | (hi << 4)) - 32
        ds = d[:, :, None] * sc                                   # [block, half, 8]: one scale per 16 elements
        scale = np.repeat(ds, 16, axis=2).reshape(-1, 2, 4, 32)
        return (scale * q.astype(F32)).reshape(len(b), 256)
    raise KeyError(kind_name)


@pytest.mark.parametrize("name", ["Q8_0", "Q4_0", "Q4_1", "Q5_0", "Q5_1", "Q4_K", "Q5_K", "Q6_K"])
def test_vectorized_decoder_and_the_oracle_give_the_same_bits(orc, name):
    kind = ALL[name]
    rng = np.random.default_rng(0x600D + kind)
    rows, cols = 6, 1024
    for _ in range(3):
        w = random_packed(rng, kind, rows, cols)
        want = orc.dequant_matrix(kind, rows, cols, w)
        got = dequant(name, w).reshape(rows, cols)
        assert got.dtype == np.float32
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), name


def test_vectorized_decoder_on_the_reference_fixture_blocks(orc):
    """The rows of the reference's boundary suite (native_cuda_parity.rs:27-122 as restated in helpers.formats)."""
    from helpers import formats
    for f in formats():
        if f.name not in ("Q8_0", "Q4_0", "Q5_0", "Q5_1", "Q4_K", "Q6_K"):
            continue
        rows = 5
        w = np.concatenate([np.asarray(f.pack_row(r), np.uint8).ravel() for r in range(rows)])
        want = orc.dequant_matrix(f.kind, rows, f.cols, w)
        assert np.array_equal(dequant(f.name, w).reshape(rows, f.cols).view(np.uint32), want.view(np.uint32)), f.name


@pytest.mark.parametrize("norm_w", [True, False])
def test_routed_layer_in_float64_numpy_agrees_with_the_oracle(orc, norm_w):
    """softmax_routed_layer (decode.rs:9938) written once more in float64 numpy from the reference's text: softmax over
    all experts, the n_used largest (ties to the lower index, topk_into :11363), weights divided by their clamped sum when
    norm_w (fill_router_weights :11392), and out = sum_j w_j * down_e(silu(gate_e x) * up_e x).  Same selections as the
    oracle, weights and outputs within float32 rounding."""
    from helpers import F32 as KIND_F32, Q4_K
    rng = np.random.default_rng(31 + int(norm_w))
    n_expert, n_used, n_embd, n_ff, tokens = 6, 2, 256, 512, 9
    router = (rng.standard_normal((n_expert, n_embd)) * 0.1).astype(np.float32)
    packs = {k: [random_packed(rng, Q4_K, r, c) for _ in range(n_expert)]
             for k, (r, c) in {"gate": (n_ff, n_embd), "up": (n_ff, n_embd), "down": (n_embd, n_ff)}.items()}
    x = rng.standard_normal((tokens, n_embd)).astype(np.float32)
    out, ids, w = orc.moe_ffn(n_used, norm_w, KIND_F32, router.view(np.uint8).reshape(-1), Q4_K, packs["gate"], packs["up"],
                              packs["down"], n_embd, n_ff, x)
    dense = {k: [orc.dequant_matrix(Q4_K, r, c, p).astype(np.float64) for p in packs[k]]
             for k, (r, c) in {"gate": (n_ff, n_embd), "up": (n_ff, n_embd), "down": (n_embd, n_ff)}.items()}
    for t in range(tokens):
        logits = router.astype(np.float64) @ x[t].astype(np.float64)
        p = np.exp(logits - logits.max())
        p /= p.sum()
        order = sorted(range(n_expert), key=lambda e: (-p[e], e))[:n_used]
        assert list(ids[t]) == order, t
        wt = p[order]
        if norm_w:
            wt = wt / max(wt.sum(), 1e-30)  # the clamp only matters for a vanishing sum
        assert np.allclose(w[t], wt, rtol=2e-5, atol=0), t
        acc = np.zeros(n_embd)
        for e, we in zip(order, wt):
            g, u = dense["gate"][e] @ x[t], dense["up"][e] @ x[t]
            acc += we * (dense["down"][e] @ (g / (1.0 + np.exp(-g)) * u))
        scale = max(1.0, float(np.abs(acc).max()))
        assert np.abs(out[t] - acc).max() <= 2e-4 * scale, (t, float(np.abs(out[t] - acc).max()), scale)


def test_dense_walk_in_float64_numpy_agrees_with_the_oracle(orc):
    """Llama::forward_layers (decode.rs:2737-3097) once more in float64 numpy from the reference's text: RMSNorm with unit
    weights, rotary embedding over adjacent pairs at angle pos * base^(-2i / head_dim) (rope, :11578), grouped-query
    attention with scores scaled by 1/sqrt(head_dim) over the positions up to the token's own, SwiGLU, residual adds,
    the last row's logits.  The oracle's walk is what every session test compares with; its pairing, scaling and head
    mapping must not be a private reading."""
    import llama_walk as lw
    from helpers import Q4_K
    cfg = dict(n_layer=2, n_embd=256, n_head=4, n_head_kv=2, head_dim=64, n_ff=256, n_vocab=40)
    rng = np.random.default_rng(23)
    tl = lw.tensor_list(cfg)
    kinds = [Q4_K] * len(tl)
    weights = [lw.center_q4k(random_packed(rng, Q4_K, r, c)) for _, _, r, c in tl]
    embd = lw.center_q4k(random_packed(rng, Q4_K, cfg["n_vocab"], cfg["n_embd"]))
    prompt = np.array([3, 17, 5, 39, 0, 8, 21], np.int32)
    want = lw.run_cpu(cfg, 16, weights, embd, prompt, 0, want_logits=True, kinds=kinds)[2].astype(np.float64)

    E, H, HKV, HD = cfg["n_embd"], cfg["n_head"], cfg["n_head_kv"], cfg["head_dim"]
    W = [orc.dequant_matrix(Q4_K, r, c, w).astype(np.float64) for (_, _, r, c), w in zip(tl, weights)]
    x = orc.dequant_matrix(Q4_K, cfg["n_vocab"], E, embd).astype(np.float64)[prompt]
    n = len(prompt)

    def rms(v):
        return v / np.sqrt((v * v).mean(axis=-1, keepdims=True) + 1e-5)

    def rope(v, heads):  # v [n, heads * HD]
        v = v.reshape(n, heads, HD // 2, 2)
        ang = np.arange(n)[:, None] * (10000.0 ** (-2.0 * np.arange(HD // 2) / HD))[None, :]
        c, s = np.cos(ang)[:, None, :], np.sin(ang)[:, None, :]
        return np.stack([v[..., 0] * c - v[..., 1] * s, v[..., 0] * s + v[..., 1] * c], axis=-1).reshape(n, heads * HD)

    for li in range(cfg["n_layer"]):
        wq, wk, wv, wo, wg, wu, wd = W[7 * li:7 * li + 7]
        xn = rms(x)
        q, k, v = rope(xn @ wq.T, H).reshape(n, H, HD), rope(xn @ wk.T, HKV).reshape(n, HKV, HD), (xn @ wv.T).reshape(n, HKV, HD)
        att = np.zeros((n, H, HD))
        for h in range(H):
            kv = h // (H // HKV)
            sc = q[:, h] @ k[:, kv].T / np.sqrt(HD)
            sc = np.where(np.tril(np.ones((n, n), bool)), sc, -np.inf)
            p = np.exp(sc - sc.max(axis=1, keepdims=True))
            att[:, h] = (p / p.sum(axis=1, keepdims=True)) @ v[:, kv]
        x = x + att.reshape(n, H * HD) @ wo.T
        xn = rms(x)
        g = xn @ wg.T
        x = x + (g / (1.0 + np.exp(-g)) * (xn @ wu.T)) @ wd.T
    got = rms(x[-1]) @ W[-1].T
    scale = np.abs(want).max()
    assert np.abs(got - want).max() <= 1e-4 * scale, (float(np.abs(got - want).max()), float(scale))
    assert int(np.argmax(got)) == int(np.argmax(want))


@pytest.mark.parametrize("name", ["Q8_0", "Q4_0", "Q4_1", "Q5_0", "Q5_1", "Q4_K", "Q5_K", "Q6_K"])
def test_row_products_against_the_vectorized_decoder_in_float64(orc, name):
    """y = W x with W from the numpy decoder above, accumulated in float64: the oracle's float64 product agrees to
    float64 rounding, and its f32 row kernels (scalar order and AVX2 order) stay within the forward error bound
    gamma(n) * sum |w_i x_i| of an n-term f32 sum."""
    kind = ALL[name]
    rng = np.random.default_rng(0xD07 + kind)
    rows, cols, tokens = 7, 2048, 3
    w = random_packed(rng, kind, rows, cols)
    x = rng.standard_normal((tokens, cols)).astype(np.float32)
    dense = dequant(name, w).reshape(rows, cols).astype(np.float64)
    want = x.astype(np.float64) @ dense.T                      # [tokens, rows]
    mass = np.abs(x).astype(np.float64) @ np.abs(dense).T
    f64 = orc.gemm_f64(kind, cols, tokens, w, x.ravel(), rows).reshape(tokens, rows)
    assert np.abs(f64 - want).max() <= 1e-12 * mass.max()
    u = 2.0 ** -24
    bound = (cols + 3) * u / (1 - (cols + 3) * u) * mass
    for simd in (False, True):
        y = orc.gemm(kind, cols, tokens, w, x.ravel(), rows, simd=simd).reshape(tokens, rows).astype(np.float64)
        assert np.all(np.abs(y - want) <= bound), (name, simd, float((np.abs(y - want) / bound).max()))
