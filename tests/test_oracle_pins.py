"""Pins the CPU oracle to the reference before anything trusts it.

Sources of truth, all from the reference itself:
* the published golden output of langtax/q8_gemv.c (README.md:276, 280),
  reproduced both by the restatement and by that file compiled unmodified
  (oracle/_ref/q8_gemv_ref, built by oracle/Makefile);
* the in-tree known-answer tests of langtax/src/quant.rs (layout bytes, "one
  nonzero" dots, scalar dot == dequant-then-dot bit equality);
* the binary16 facts of langtax/src/fp16.rs:169-279;
* the SIMD-vs-scalar error bound of langtax/src/simd/tests.rs:59-153.
"""
import re
import subprocess

import numpy as np
import pytest

GOLDEN_CHECKSUM = 0x80E188057FA1EEF0  # README.md:276
GOLDEN_Y0 = "78.165176"


def test_q8_gemv_golden_checksum_restatement(orc):
    w, xq = orc.demo_q8_0(4096, 4096)
    for simd in (False, True):
        y = orc.gemv_q8_0_q8_0(4096, w, xq, 4096, simd=simd)
        assert orc.y_checksum(y) == GOLDEN_CHECKSUM, f"simd={simd}"
        assert f"{y[0]:.6f}" == GOLDEN_Y0


def test_q8_gemv_reference_binary_agrees(orc):
    exe = orc.ref_q8_gemv_binary()
    if exe is None:
        pytest.skip("oracle/_ref/q8_gemv_ref not built (reference tree absent)")
    out = subprocess.run([exe], capture_output=True, text=True, check=True).stdout
    m = re.search(r"y_checksum=([0-9a-f]{16}) y0=([0-9.]+)", out)
    assert m, out
    assert int(m.group(1), 16) == GOLDEN_CHECKSUM
    assert m.group(2) == GOLDEN_Y0


def test_q8_0_f32_path_cross_checks_golden(orc):
    """The model path gemv_q8_0_f32 fed the dequantized x_q8 agrees with the golden y."""
    w, xq = orc.demo_q8_0(4096, 4096)
    y_gold = orc.gemv_q8_0_q8_0(4096, w, xq, 4096)
    x = orc.dequant_row(orc.Q8_0, 4096, xq)
    wf = orc.dequant_matrix(orc.Q8_0, 4096, 4096, w).astype(np.float64)
    abs_sum = np.abs(wf * x.astype(np.float64)).sum(axis=1)
    k = 4096 + 3.0
    bound = k * 2.0 ** -24 / (1 - k * 2.0 ** -24) * abs_sum  # simd/tests.rs:83-91
    for simd in (False, True):
        y = orc.gemv(orc.Q8_0, 4096, w, x, 4096, simd=simd)
        assert np.all(np.abs(y.astype(np.float64) - y_gold) <= bound)
        assert np.median(np.abs(y - y_gold) / (1 + np.abs(y_gold))) < 1e-5


# ---- fp16.rs -------------------------------------------------------------
def test_f16_known_values(orc):
    assert orc.f16_to_f32(0x0000) == 0.0
    assert orc.f16_to_f32(0x3C00) == 1.0
    assert orc.f16_to_f32(0xBC00) == -1.0
    assert orc.f16_to_f32(0x7BFF) == 65504.0
    assert orc.f16_to_f32(0x0001) == 2.0 ** -24
    assert orc.f16_to_f32(0x7C00) == float("inf")


def test_f16_exhaustive_matches_numpy(orc):
    checked = subnormals = 0
    for h in range(0x10000):
        if (h >> 10) & 0x1F == 0x1F:
            continue
        want = np.array([h], np.uint16).view(np.float16).astype(np.float32)[0]
        got = np.float32(orc.f16_to_f32(h))
        assert got.view(np.uint32) == want.view(np.uint32), hex(h)
        checked += 1
        if (h >> 10) & 0x1F == 0 and h & 0x3FF:
            subnormals += 1
    assert checked == 63488 and subnormals == 2046  # fp16.rs:216-217


def test_f16_subnormal_scale_from_real_gguf(orc):
    got = np.float32(orc.f16_to_f32(0x8000 | 299))  # fp16.rs:224-231
    assert got == np.float32(-299.0 * 2.0 ** -24)


def test_f32_to_f16_truncates_and_keeps_subnormals(orc):
    assert orc.f32_to_f16(1.0) == 0x3C00
    assert orc.f32_to_f16(65504.0) == 0x7BFF
    assert orc.f32_to_f16(1e9) == 0x7C00
    assert orc.f32_to_f16(2.0 ** -24) == 0x0001
    assert orc.f32_to_f16(2.0 ** -26) == 0x0000
    # truncation, not rounding: 1 + 0.995 ulp stays at 1.0 (round-to-nearest gives 0x3C01)
    assert orc.f32_to_f16(float(np.float32(1.0) + np.float32(2.0 ** -11) * np.float32(1.99))) == 0x3C00
    assert orc.f32_to_f16(-0.015625) == 0xA400


# ---- quant.rs known answers ----------------------------------------------
def test_pack_q5_0_layout_known_answer(orc):  # quant.rs:10907-10926
    qs = np.zeros(32, np.uint8)
    qs[0], qs[16], qs[7], qs[23] = 19, 28, 7, 15
    w = orc.pack_q5_0_block(0.25, qs)
    assert w.size == 22
    assert w[6] == 0xC3
    qh = int.from_bytes(bytes(w[2:6]), "little")
    assert qh & 0x00010001 == 0x00010001
    assert w[13] == 0xF7
    assert qh & ((1 << 7) | (1 << 23)) == 0
    x = np.zeros(32, np.float32)
    x[0], x[16], x[7], x[23] = 2, 4, 1, 3
    y = orc.gemv(orc.Q5_0, 32, w, x, 1)
    # (19-16)*.25*2 + (28-16)*.25*4 + (7-16)*.25*1 + (15-16)*.25*3
    assert y[0] == 1.5 + 12.0 - 2.25 - 0.75
    row = orc.dequant_row(orc.Q5_0, 32, w)
    assert row[0] == 0.75 and row[16] == 3.0 and row[7] == -2.25 and row[23] == -0.25


def test_pack_q4_1_known_answer(orc):  # quant.rs:10796-10828, gguf.rs:1506-1523
    qs = np.zeros(32, np.uint8)
    qs[0], qs[16], qs[7], qs[23] = 3, 12, 7, 15
    w = orc.pack_q4_1_block(0.25, 0.05, qs)
    assert w.size == 20 and w[4] == 0xC3 and w[11] == 0xF7
    m = np.float32(orc.f16_to_f32(int(w[2]) | int(w[3]) << 8))      # 0.05 truncated to binary16
    assert abs(float(m) - 0.05) < 2e-5 and float(m) <= 0.05
    x = np.zeros(32, np.float32)
    x[0], x[16], x[7], x[23] = 2, 4, 1, 3
    row = orc.dequant_row(orc.Q4_1, 32, w)
    want = np.full(32, m, np.float32)
    for i, q in ((0, 3), (16, 12), (7, 7), (23, 15)):
        want[i] = np.float32(np.float32(q * 0.25) + m)
    assert np.array_equal(row.view(np.uint32), want.view(np.uint32))
    y = orc.gemv(orc.Q4_1, 32, w, x, 1)[0]
    assert abs(y - 27.0) / 28.0 < 1e-5                               # (3/4+m)2 + (3+m)4 + (7/4+m) + (15/4+m)3 with m = 0.05
    acc = np.float32(0.0)
    for j in range(16):                                              # element j then j+16, one running sum
        acc = np.float32(acc + np.float32(row[j] * x[j]))
        acc = np.float32(acc + np.float32(row[j + 16] * x[j + 16]))
    assert acc.view(np.uint32) == np.float32(y).view(np.uint32)
    # gemm == repeated gemv, token-major (quant.rs:10831-10880)
    w2 = np.concatenate([orc.pack_q4_1_block(0.25, 0.05, np.where(np.arange(32) == 0, 3 + r, np.where(np.arange(32) == 16, 12 + r,
                                                                   np.where(np.arange(32) == 7, 7, 0))).astype(np.uint8)) for r in range(2)])
    xk = np.zeros((3, 32), np.float32)
    xk[:, 0] = [1, 2, 3]
    xk[:, 16] = 2
    yk = orc.gemm(orc.Q4_1, 32, 3, w2, xk, 2)
    for t in range(3):
        assert np.array_equal(yk[t], orc.gemv(orc.Q4_1, 32, w2, xk[t], 2))


def test_pack_q5_k_known_answer(orc):  # quant.rs:12078-12111, gguf.rs:1714-1731
    qs = np.zeros(256, np.uint8)
    qs[0], qs[32], qs[64], qs[128] = 3, 17, 20, 21
    w = orc.pack_q5_k_block(0.25, 0.05, [2, 1, 3, 1, 4, 1, 1, 1], [1, 0, 0, 0, 2, 0, 0, 0], qs)
    assert w.size == 176
    assert w[16] & 0b00010111 == 0b00010110      # qh[0]: bit 1 (q=17), bit 2 (q=20), bit 4 (q=21); bit 0 clear (q=3)
    assert np.array_equal(w[:16], orc.pack_q4_k_block(0.25, 0.05, [2, 1, 3, 1, 4, 1, 1, 1], [1, 0, 0, 0, 2, 0, 0, 0],
                                                      np.zeros(256, np.uint8))[:16])
    dmin = np.float32(orc.f16_to_f32(int(w[2]) | int(w[3]) << 8))
    x = np.zeros(256, np.float32)
    x[0], x[32], x[64], x[128] = 2, 4, 1, 3
    row = orc.dequant_row(orc.Q5_K, 256, w)
    assert row[0] == np.float32(np.float32(0.5 * 3) - dmin) and row[32] == 4.25 and row[64] == 15.0
    assert row[128] == np.float32(np.float32(21.0) - np.float32(dmin * 2))
    y = orc.gemv(orc.Q5_K, 256, w, x, 1)[0]
    assert abs(y - 97.6) / 98.6 < 1e-5            # 1.45*2 + 4.25*4 + 15 + 20.9*3
    acc = np.float32(0.0)
    for g in range(4):                            # per l: low half element, then high half element
        for l in range(32):
            for e in (64 * g + l, 64 * g + 32 + l):
                acc = np.float32(acc + np.float32(row[e] * x[e]))
    assert acc.view(np.uint32) == np.float32(y).view(np.uint32)
    # a one-block GGUF payload of the reference's own test: scales all 1, mins 0, d = 1 (gguf.rs:1714-1718)
    qs = np.zeros(256, np.uint8)
    qs[0], qs[32] = 3, 17
    w = orc.pack_q5_k_block(1.0, 0.0, [1] * 8, [0] * 8, qs)
    assert orc.dequant_row(orc.Q5_K, 256, w)[[0, 32, 1]].tolist() == [3.0, 17.0, 0.0]


def test_pack_q6_k_one_nonzero(orc):  # quant.rs:10321-10340
    qs = np.zeros(256, np.int8)
    qs[0], qs[32] = 1, 2
    sc = np.zeros(16, np.int8)
    sc[0] = sc[2] = 1
    w = orc.pack_q6_k_block(1.0, sc, qs)
    x = np.zeros(256, np.float32)
    x[0], x[32] = 3, 4
    for simd in (False, True):
        assert orc.gemv(orc.Q6_K, 256, w, x, 1, simd=simd)[0] == 11.0
    row = orc.dequant_row(orc.Q6_K, 256, w)
    assert float(np.dot(row, x)) == 11.0


def test_q4_k_sparse_dot_matches_dequant(orc):  # quant.rs:10342-10364
    qs = np.zeros(256, np.uint8)
    qs[0], qs[32] = 3, 5
    w = orc.pack_q4_k_block(0.25, 0.0, [2, 1, 1, 1, 1, 1, 1, 1], [0] * 8, qs)
    x = np.zeros(256, np.float32)
    x[0], x[32] = 2, 4
    y = orc.gemv(orc.Q4_K, 256, w, x, 1)[0]
    assert y == 0.25 * 2 * 3 * 2 + 0.25 * 1 * 5 * 4


def test_q4_k_dense_scalar_dot_bit_equals_dequant_then_dot(orc):  # quant.rs:10373-10393
    qs = (np.arange(256) % 16).astype(np.uint8)
    w = orc.pack_q4_k_block(0.25, 0.01, [2, 3, 4, 5, 1, 2, 3, 4], [1, 0, 1, 0, 1, 0, 1, 0], qs)
    x = (np.arange(256, dtype=np.float32) * np.float32(0.01) - np.float32(0.5)).astype(np.float32)
    via_gemv = np.float32(orc.dot_row(orc.Q4_K, w, x, simd=False))
    row = orc.dequant_row(orc.Q4_K, 256, w)
    acc = np.float32(0.0)
    for a, b in zip(row, x):
        acc = np.float32(acc + np.float32(a * b))
    assert acc.view(np.uint32) == via_gemv.view(np.uint32)


def test_q4_k_scale_bytes_roundtrip(orc):
    """pack_q4_k_scale_bytes (quant.rs:4852) against ggml get_scale_min_k4 (quant.rs:10396)."""
    rng = np.random.default_rng(7)
    for _ in range(50):
        sc = rng.integers(0, 64, 8)
        mn = rng.integers(0, 64, 8)
        w = orc.pack_q4_k_block(1.0, 1.0, sc, mn, np.ones(256, np.uint8))
        q = w[4:16]
        for j in range(8):
            if j < 4:
                got = (q[j] & 63, q[j + 4] & 63)
            else:
                got = ((q[j + 4] & 0x0F) | ((q[j - 4] >> 6) << 4), (q[j + 4] >> 4) | ((q[j] >> 6) << 4))
            assert got == (sc[j], mn[j])
        row = orc.dequant_row(orc.Q4_K, 256, w)
        for j in range(8):
            assert np.all(row[32 * j:32 * j + 32] == np.float32(sc[j]) - np.float32(mn[j]))


def test_all_zero_bytes_give_negative_zero_weights(orc):  # simd/tests.rs:1481-1508
    for kind, bias in ((orc.Q4_0, True), (orc.Q5_0, True), (orc.Q8_0, False)):
        rb = orc.row_bytes(kind, 32)
        row = orc.dequant_row(kind, 32, np.zeros(rb, np.uint8))
        assert np.all(row == 0.0)
        assert np.all(np.signbit(row) == bias)


def test_q5_1_offset_is_added_not_fused(orc):  # simd/tests.rs:1146-1172
    # d*q is inexact in f32 for a 5-bit q and an 11-bit d, so a fused q*d+m
    # would round once; the reference rounds twice.
    d, m = 0.333251953125, 1.0009765625  # exactly representable in binary16
    q5 = np.arange(32, dtype=np.uint8)
    w = orc.pack_q5_1_block(d, m, q5)
    row = orc.dequant_row(orc.Q5_1, 32, w)
    dd, mm = np.float32(orc.f16_to_f32(int(w[0]) | int(w[1]) << 8)), np.float32(
        orc.f16_to_f32(int(w[2]) | int(w[3]) << 8))
    for j in range(32):
        want = np.float32(np.float32(np.float32(j) * dd) + mm)
        assert row[j].view(np.uint32) == want.view(np.uint32)


# ---- every code value in every position: bit equality of simd and scalar -----
@pytest.mark.parametrize("name", ["Q4_0", "Q5_0", "Q5_1", "Q8_0"])
def test_single_term_rows_are_bit_equal(orc, name):  # simd/tests.rs:755, 933, 1110, 1272
    kind = orc.KINDS[name]
    codes = {"Q4_0": range(-8, 8), "Q5_0": range(32), "Q5_1": range(32), "Q8_0": range(-128, 128)}[name]
    for pos in range(32):
        for code in codes:
            if name == "Q4_0":
                v = np.zeros(32, np.int8) ; v[pos] = code
                w = orc.pack_q4_0_from_i4(0.375, v)
            elif name == "Q5_0":
                v = np.full(32, 16, np.uint8) ; v[pos] = code
                w = orc.pack_q5_0_block(0.375, v)
            elif name == "Q5_1":
                v = np.zeros(32, np.uint8) ; v[pos] = code
                w = orc.pack_q5_1_block(0.375, 0.0, v)
            else:
                v = np.zeros(32, np.int8) ; v[pos] = code
                w = orc.pack_q8_0_block(0.375, v)
            x = np.zeros(32, np.float32) ; x[pos] = 1.7
            s = np.float32(orc.dot_row(kind, w, x, simd=False))
            v_ = np.float32(orc.dot_row(kind, w, x, simd=True))
            assert s.view(np.uint32) == v_.view(np.uint32), (name, pos, code)


# ---- SIMD vs scalar within the reference's proven bound ---------------------
U = 2.0 ** -24


def _single_bound(n, abs_sum):
    k = n + 3.0
    g = k * U / (1 - k * U) if k * U < 0.5 else k * U
    return g * abs_sum


def _rand_row(orc, rng, kind, n_cols):
    """Uniform random bytes with sane binary16 scales (|N|*0.01, truncated)."""
    be, bb = orc.block_elems(kind), orc.block_bytes(kind)
    nb = n_cols // be
    raw = rng.integers(0, 256, (nb, bb), dtype=np.uint8)

    def put_scale(col):
        vals = np.abs(rng.standard_normal(nb)).astype(np.float32) * np.float32(0.01)
        for i, v in enumerate(vals):
            h = orc.f32_to_f16(float(v))
            raw[i, col], raw[i, col + 1] = h & 0xFF, h >> 8

    if kind in (orc.Q8_0, orc.Q4_0, orc.Q5_0):
        put_scale(0)
    elif kind in (orc.Q5_1, orc.Q4_K):
        put_scale(0)
        put_scale(2)
    elif kind == orc.Q6_K:
        put_scale(208)
    elif kind == orc.F16:
        return orc.pack_f16(rng.standard_normal(n_cols).astype(np.float32))
    elif kind == orc.BF16:
        return orc.pack_bf16(rng.standard_normal(n_cols).astype(np.float32))
    elif kind == orc.F32:
        return orc.pack_f32(rng.standard_normal(n_cols).astype(np.float32))
    return raw.reshape(-1)


@pytest.mark.parametrize("name", ["F32", "F16", "BF16", "Q4_0", "Q5_0", "Q5_1", "Q8_0", "Q4_K", "Q6_K"])
def test_simd_and_scalar_within_proven_bound(orc, name):  # simd/tests.rs:59-153
    kind = orc.KINDS[name]
    rng = np.random.default_rng(0x5EED)
    be = orc.block_elems(kind)
    for blocks in (1, 2, 3, 4, 5, 8, 16):  # simd/tests.rs:196-199
        n = blocks * max(be, 32)
        row = _rand_row(orc, rng, kind, n)
        x = rng.standard_normal(n).astype(np.float32)
        wf = orc.dequant_row(kind, n, row).astype(np.float64)
        exact = float(np.dot(wf, x.astype(np.float64)))
        abs_sum = float(np.sum(np.abs(wf * x.astype(np.float64))))
        s = orc.dot_row(kind, row, x, simd=False)
        v = orc.dot_row(kind, row, x, simd=True)
        single = _single_bound(n, abs_sum)
        assert abs(s - exact) <= single
        assert abs(v - exact) <= single
        assert abs(s - v) <= 2 * single
        assert abs(s - v) / abs_sum / U <= max(8 * np.sqrt(n), 64.0)


def test_gemm_equals_repeated_gemv_and_is_token_major(orc):  # quant.rs tests "gemm == repeated gemv"
    rng = np.random.default_rng(3)
    for name in ("Q4_K", "Q8_0", "Q6_K", "Q5_1"):
        kind = orc.KINDS[name]
        n_cols, n_rows, n_tok = 512, 11, 5
        w = np.concatenate([_rand_row(orc, rng, kind, n_cols) for _ in range(n_rows)])
        x = rng.standard_normal((n_tok, n_cols)).astype(np.float32)
        y = orc.gemm(kind, n_cols, n_tok, w, x, n_rows, simd=True)
        for t in range(n_tok):
            yt = orc.gemv(kind, n_cols, w, x[t], n_rows, simd=True, threads=1)
            assert np.array_equal(y[t].view(np.uint32), yt.view(np.uint32))


def test_threaded_gemv_is_bit_identical_to_sequential(orc):  # decode.rs:16251
    rng = np.random.default_rng(4)
    kind = orc.Q4_K
    w = np.concatenate([_rand_row(orc, rng, kind, 1024) for _ in range(37)])
    x = rng.standard_normal(1024).astype(np.float32)
    y1 = orc.gemv(kind, 1024, w, x, 37, threads=1)
    for t in (2, 3, 8):
        assert np.array_equal(orc.gemv(kind, 1024, w, x, 37, threads=t).view(np.uint32), y1.view(np.uint32))


def test_entry_point_validation(orc):  # quant.rs:6698-6742, 7199-7212
    x = np.zeros(32, np.float32)
    with pytest.raises(orc.OracleError) as e:
        orc.gemv(orc.Q8_0, 33, np.zeros(34, np.uint8), np.zeros(33, np.float32), 1)
    assert e.value.code == orc.ERR_UNALIGNED_COLS
    with pytest.raises(orc.OracleError):
        orc.gemv(orc.Q8_0, 32, np.zeros(33, np.uint8), x, 1)
    with pytest.raises(orc.OracleError):
        orc.gemv(orc.Q8_0, 32, np.zeros(34, np.uint8), np.zeros(31, np.float32), 1)
    with pytest.raises(orc.OracleError):
        orc.gemm(orc.Q8_0, 32, 0, np.zeros(34, np.uint8), np.zeros(0, np.float32), 1)
    assert orc.gemv(orc.Q8_0, 32, np.zeros(0, np.uint8), x, 0).size == 0
    with pytest.raises(orc.OracleError) as e:
        orc.row_bytes(3, 32)
    assert e.value.code == orc.ERR_DTYPE
