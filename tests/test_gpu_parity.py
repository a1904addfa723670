"""GPU parity at the executor boundary, through the C ABI.

Restates the reference's own hardware parity suite
(langtax/tests/native_cuda_parity.rs) and executor self-check
(native-cuda/src/main.rs) against this library, then holds the CUDA kernels to
the CPU row kernels (oracle: scalar + AVX2 restatement) on seeded inputs:
dequantized blocks bit-exact, GEMV within |gpu-cpu| <= 1e-5*(1+|cpu|).
"""
import numpy as np
import pytest

from helpers import (ALL, BF16, F16, F32, Q4_0, Q4_K, Q5_0, Q5_1, Q6_K, Q8_0, check_boundary,
                     check_gemv, check_kernel, formats, gemv_references, random_packed, values)

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def q():
    from llama_rust_b200 import quant
    quant.thread_executor()
    yield quant
    quant.reset_thread_executor()


@pytest.fixture(scope="module")
def ex():
    from llama_rust_b200 import Executor
    e = Executor(0)
    yield e
    e.close()


# ---- native_cuda_parity.rs -------------------------------------------------
@pytest.mark.parametrize("fmt", formats(), ids=lambda f: f.name)
def test_quantized_model_dispatch_matches_cpu_row_oracle(q, orc, fmt):  # parity.rs:161-190
    rows = 257
    packed = np.concatenate([fmt.pack_row(r) for r in range(rows)])
    rb = packed.size // rows
    for pas in range(2):
        for rnd, tokens in enumerate([1, 1, 3, 3, 7, 1]):
            x = np.concatenate([values(t + rnd * 3 + pas, fmt.cols) for t in range(tokens)])
            expected = orc.gemm_f64(fmt.kind, fmt.cols, tokens, packed, x, rows)
            actual = np.full(rows * tokens, np.nan, np.float32)
            if tokens == 1:
                q.GEMV[fmt.kind](fmt.cols, packed, x, actual)
            else:
                q.GEMM[fmt.kind](fmt.cols, tokens, packed, x, actual)
            check_boundary(actual, expected, fmt.name)
        # same buffer, same shape and dtype, different bytes: residency keys on content
        packed[:rb] = fmt.pack_row(rows + 5)


def test_warp_boundary_shapes_match_independent_f64_dots(q):  # parity.rs:336-376
    for rows in (1, 7, 9, 257):
        for cols in (63, 64, 65, 129, 1025):
            w = np.concatenate([values(r, cols) / np.float32(1.3) for r in range(rows)]).astype(np.float32)
            for rnd in range(2):
                for tokens in (1, 3):
                    x = np.concatenate([values(t + rnd * 17, cols) / np.float32(1.7) for t in range(tokens)]).astype(np.float32)
                    expected = x.reshape(tokens, cols).astype(np.float64) @ w.reshape(rows, cols).astype(np.float64).T
                    actual = np.full(rows * tokens, np.nan, np.float32)
                    if tokens == 1:
                        q.gemv_f32(cols, w.view(np.uint8), x, actual)
                    else:
                        q.gemm_f32(cols, tokens, w.view(np.uint8), x, actual)
                    check_boundary(actual, expected, f"warp-boundary {rows}x{cols}")


@pytest.mark.parametrize("fmt", formats(), ids=lambda f: f.name)
def test_multi_block_quantized_batches_match_cpu_oracle(q, orc, fmt):  # parity.rs:378-408
    for blocks in (2, 3):
        cols = fmt.cols * blocks
        for rows in (1, 9):
            packed = np.concatenate([fmt.pack_row(r + b * 5) for r in range(rows) for b in range(blocks)])
            for tokens in (1, 2, 7, 8, 9, 31, 32, 33):
                x = np.concatenate([values(t * 3 + 1, cols) for t in range(tokens)])
                expected = orc.gemm_f64(fmt.kind, cols, tokens, packed, x, rows)
                actual = np.full(rows * tokens, np.nan, np.float32)
                q.GEMM[fmt.kind](cols, tokens, packed, x, actual)
                check_boundary(actual, expected, fmt.name)


@pytest.mark.parametrize("fmt", formats(), ids=lambda f: f.name)
def test_invalid_matrix_operations_preserve_output_and_empty_rows_are_noop(q, fmt):  # parity.rs:410-431
    packed = fmt.pack_row(0)
    x = values(1, fmt.cols)
    out = np.array([123.5], np.float32)
    empty_b, empty_f = np.zeros(0, np.uint8), np.zeros(0, np.float32)
    with pytest.raises(q.QuantError):
        q.GEMV[fmt.kind](fmt.cols, empty_b, x, out)
    assert out[0] == 123.5, "invalid weights changed output"
    with pytest.raises(q.QuantError):
        q.GEMV[fmt.kind](fmt.cols, packed, empty_f, out)
    assert out[0] == 123.5, "invalid input changed output"
    with pytest.raises(q.QuantError):
        q.GEMM[fmt.kind](fmt.cols, 0, packed, x, out)
    assert out[0] == 123.5, "zero tokens changed output"
    doubled = np.concatenate([x, x])
    with pytest.raises(q.QuantError):
        q.GEMM[fmt.kind](fmt.cols, 2, packed, doubled, out)
    assert out[0] == 123.5, "unaligned output changed contents"
    q.GEMV[fmt.kind](fmt.cols, empty_b, x, empty_f.copy())
    q.GEMM[fmt.kind](fmt.cols, 2, empty_b, doubled, empty_f.copy())


def test_overflowing_shape_is_rejected_without_touching_output(q):  # parity.rs:427-429
    out = np.array([123.5], np.float32)
    with pytest.raises(q.QuantError):
        q.gemm_f32(2 ** 64 - 1, 2, np.zeros(0, np.uint8), np.zeros(0, np.float32), out)
    assert out[0] == 123.5


def test_unsupported_dtype_tag_is_an_error_not_a_fallback(q):
    out = np.array([123.5], np.float32)
    with pytest.raises(q.QuantError) as e:
        q.native_matmul(3, 256, 1, np.zeros(84, np.uint8), np.zeros(256, np.float32), out)  # Q2_K tag
    assert e.value.code == 3 and out[0] == 123.5


# ---- native-cuda/src/main.rs -----------------------------------------------
def test_executor_self_check_shapes_and_recovery(ex):  # main.rs:4-70
    from llama_rust_b200 import Executor, NativeCudaError
    shapes = [(r, c) for r in (1, 7, 9, 257) for c in (63, 64, 65, 129, 1025)] + [(17, 33), (1, 1), (257, 129), (17, 33)]
    for rows, cols in shapes:
        w = ((np.arange(rows * cols) % 23).astype(np.float32) - 11.0) / np.float32(16.0)
        m = ex.upload(F32, rows, cols, w.view(np.uint8))
        for rnd, tokens in enumerate([1, 1, 3, 3, 1, 7, 1]):
            x = (((np.arange(tokens * cols) * 5 + rnd * 7) % 29).astype(np.float32) - 14.0) / np.float32(16.0)
            expected = x.reshape(tokens, cols).astype(np.float64) @ w.reshape(rows, cols).astype(np.float64).T
            actual = np.full(rows * tokens, np.nan, np.float32)
            if tokens == 1:
                ex.gemv_resident(m, x, actual)
            else:
                ex.gemm_resident(m, tokens, x, actual)
            check_boundary(actual, expected, f"self-check {rows}x{cols} t={tokens}")
        m.free()
    m = ex.upload(F32, 2, 3, np.float32([1, -2, 3, 4, 5, -6]).view(np.uint8))
    out = np.float32([123.5, -456.0])
    with pytest.raises(NativeCudaError):
        ex.gemv_resident(m, np.float32([1, 2]), out)
    with pytest.raises(NativeCudaError):
        ex.gemm_resident(m, 0, np.zeros(0, np.float32), out)
    other = Executor(0)
    with pytest.raises(NativeCudaError) as e:
        other.gemv_resident(m, np.float32([1, 2, 3]), out)
    assert e.value.code == 5 and "different executor" in str(e.value)
    other.close()
    assert list(out) == [123.5, -456.0]
    ex.gemv_resident(m, np.float32([1, 2, 3]), out)  # the executor is still usable
    assert list(out) == [6.0, -4.0]
    free, total = ex.memory_info()
    assert 0 < free <= total


# ---- dequantized blocks are bit-exact ----------------------------------------
@pytest.mark.parametrize("name", list(ALL))
@pytest.mark.parametrize("scale_mode", ["normal", "any_f16"])
def test_dequantized_blocks_match_bit_for_bit(ex, orc, name, scale_mode):
    kind = ALL[name]
    if scale_mode == "any_f16" and kind in (F32, F16, BF16):
        pytest.skip("no block scale")
    rng = np.random.default_rng(0xD0 + kind)
    rows, cols = 37, 1536
    w = random_packed(rng, kind, rows, cols, scale_mode)
    m = ex.upload(kind, rows, cols, w)
    got = ex.dequant_rows(m)
    want = orc.dequant_matrix(kind, rows, cols, w)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), name
    part = ex.dequant_rows(m, 5, 3)
    assert np.array_equal(part.view(np.uint32), want[5:8].view(np.uint32))
    m.free()


def test_f16_weights_every_bit_pattern_bit_exact(ex, orc):  # fp16.rs:195-218
    pats = np.arange(0x10000, dtype=np.uint16)
    m = ex.upload(F16, 16, 4096, pats.view(np.uint8))
    got = ex.dequant_rows(m).reshape(-1)
    want = orc.dequant_matrix(F16, 16, 4096, pats.view(np.uint8)).reshape(-1)
    finite = ((pats >> 10) & 0x1F) != 0x1F
    assert np.array_equal(got.view(np.uint32)[finite], want.view(np.uint32)[finite])
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))  # Inf and NaN payloads too
    m.free()


def test_all_zero_bytes_dequantize_to_negative_zero(ex):  # simd/tests.rs:1481-1508
    for kind, neg in ((Q4_0, True), (Q5_0, True), (Q8_0, False), (Q4_K, False), (Q6_K, True)):
        from llama_rust_b200 import row_bytes
        w = np.zeros(row_bytes(kind, 256) * 2, np.uint8)
        m = ex.upload(kind, 2, 256, w)
        got = ex.dequant_rows(m)
        assert np.all(got == 0.0) and np.all(np.signbit(got) == neg), kind
        m.free()


# ---- decode GEMV against the CPU row kernels --------------------------------------
PATHS = {"generic": 1, "staged": 2, "auto": 0}


@pytest.mark.parametrize("path", list(PATHS))
@pytest.mark.parametrize("name", list(ALL))
def test_gemv_matches_cpu_row_kernels(ex, orc, name, path):
    """Every kernel family (shape-agnostic, staged FMA, integer tensor core) against the CPU
    row kernels on seeded random blocks, M = 1, 2, 3, 4, 8 and 11 (two passes)."""
    kind = ALL[name]
    ex.set_path(PATHS[path])
    rng = np.random.default_rng(0xA0 + kind)
    for rows, cols in ((64, 4096), (33, 2048 + 256), (5, 14336), (17, 6144)):
        w = random_packed(rng, kind, rows, cols)
        m = ex.upload(kind, rows, cols, w)
        for tokens in (1, 2, 3, 4, 8, 11):
            x = rng.standard_normal(tokens * cols).astype(np.float32)
            cpu, exact, abs_sum = gemv_references(kind, rows, cols, w, x, tokens)
            y = np.full(rows * tokens, np.nan, np.float32)
            ex.gemm_resident(m, tokens, x, y)
            check_gemv(y, cpu, exact, abs_sum, cols, f"{name} {rows}x{cols} M={tokens} {path}")
        m.free()
    ex.set_path(0)


@pytest.mark.parametrize("name", ["Q4_K", "Q6_K", "Q8_0", "Q4_0", "Q5_0", "Q5_1", "Q4_1", "Q5_K"])
def test_tensor_core_gemv_handles_awkward_activations(ex, orc, name):
    """Outliers, tiny values, zero blocks and a non-finite activation through the digit split."""
    kind = ALL[name]
    rng = np.random.default_rng(0xB0 + kind)
    rows, cols = 48, 4096
    w = random_packed(rng, kind, rows, cols)
    m = ex.upload(kind, rows, cols, w)
    x = rng.standard_normal(cols).astype(np.float32)
    x[7] = 3000.0          # a massive activation next to ordinary ones
    x[300:556] = 0.0       # an all-zero 256-block
    x[600:700] *= 1e-12    # values far below their block's maximum
    x[1024:1280] *= 1e20   # a block with a huge common scale
    x[2048:2304] *= 1e-30  # and a tiny one
    cpu, exact, abs_sum = gemv_references(kind, rows, cols, w, x, 1)
    y = np.empty(rows, np.float32)
    ex.gemv_resident(m, x, y)
    check_gemv(y, cpu, exact, abs_sum, cols, name + " awkward x")
    x[5] = np.inf
    ex.gemv_resident(m, x, y)
    assert np.all(np.isnan(y)), "a non-finite activation must poison its output row"
    m.free()


@pytest.mark.parametrize("name", ["Q4_K", "Q5_K", "Q6_K", "Q8_0", "Q4_0", "Q4_1", "Q5_0", "Q5_1"])
def test_tensor_core_gemv_one_nonzero_activation_at_every_column(ex, orc, name):
    """The reference's single-term idea (simd/tests.rs:755: one non-zero term per position) on the integer tensor-core
    kernel: with x = 1.7 e_c the result is column c of the dequantized matrix times 1.7, for every column of two
    256-column groups and for one and three activation rows.  A weight, digit plane or fifth-bit that sits at the wrong
    place changes a result by the size of a weight; rounding differences stay below 4e-6 of the largest one."""
    kind = ALL[name]
    rng = np.random.default_rng(0xD0 + kind)
    rows, cols = 40, (2048 if name == "Q6_K" else 512)  # the kernel takes Q6_K rows in pieces of 2048 columns
    w = random_packed(rng, kind, rows, cols)
    m = ex.upload(kind, rows, cols, w)
    wf = orc.dequant_matrix(kind, rows, cols, w).astype(np.float64)
    tol = 4e-6 * np.abs(wf).max() * 1.7
    ex.set_path(3)
    for c in range(cols):
        x = np.zeros((3, cols), np.float32)
        x[0, c] = 1.7
        x[2, c] = -0.85
        x[1, (c * 7 + 3) % cols] = 1.7
        y1 = np.empty(rows, np.float32)
        ex.gemv_resident(m, x[0], y1)
        assert np.abs(y1 - wf[:, c] * 1.7).max() <= tol, (name, c, 1)
        y3 = np.empty(3 * rows, np.float32)
        ex.gemm_resident(m, 3, x, y3)
        y3 = y3.reshape(3, rows)
        assert np.abs(y3[0] - wf[:, c] * 1.7).max() <= tol, (name, c, 3)
        assert np.abs(y3[1] - wf[:, (c * 7 + 3) % cols] * 1.7).max() <= tol, (name, c, "row 1")
        assert np.abs(y3[2] + wf[:, c] * 0.85).max() <= tol, (name, c, "row 2")
    ex.set_path(0)
    m.free()


def test_config1_q8_0_4096_gemv_seed0(ex, orc):
    """benchmark config 1: Q8_0 4096x4096, x ~ N(0,1), seed 0, M = 1, every kernel family."""
    from llama_rust_b200 import synth
    w = synth.packed_matrix(Q8_0, 4096, 4096, synth.tensor_seed(0, "config1.w"))
    x = synth.activations(4096, synth.tensor_seed(0, "config1.x"))
    cpu, exact, abs_sum = gemv_references(Q8_0, 4096, 4096, w, x, 1)
    m = ex.upload(Q8_0, 4096, 4096, w)
    for path in (1, 2, 0):
        ex.set_path(path)
        y = np.empty(4096, np.float32)
        ex.gemv_resident(m, x, y)
        vs_cpu, vs_exact = check_gemv(y, cpu, exact, abs_sum, 4096, f"config1 path {path}")
        err_u = np.abs(y - exact.ravel()) / abs_sum.ravel() / 2.0 ** -24
        assert err_u.max() < 64.0  # the reference's envelope for n = 4096 is 8*sqrt(n) = 512 u
    m.free()
    ex.set_path(0)


@pytest.mark.parametrize("name,rows,cols", [("Q4_K", 4096, 4096), ("Q4_K", 1024, 4096), ("Q4_K", 2048, 14336),
                                            ("Q6_K", 1024, 4096), ("Q6_K", 1024, 14336), ("Q6_K", 4008, 4096)])
def test_config2_decode_shapes(ex, orc, name, rows, cols):
    """benchmark config 2 shapes (row counts trimmed where the CPU oracle would take long), M = 1, 2, 4, 8."""
    from llama_rust_b200 import synth
    kind = ALL[name]
    seed = synth.tensor_seed(2, f"config2.{name}.{rows}x{cols}")
    m = ex.synth(kind, rows, cols, seed)
    w = ex.download(m)
    for tokens in (1, 2, 4, 8):
        x = synth.activations(tokens * cols, synth.tensor_seed(2, f"x.{tokens}"))
        cpu, exact, abs_sum = gemv_references(kind, rows, cols, w, x, tokens)
        y = np.empty(rows * tokens, np.float32)
        ex.gemm_resident(m, tokens, x, y)
        check_gemv(y, cpu, exact, abs_sum, cols, f"{name} {rows}x{cols} M={tokens}")
    m.free()


@pytest.mark.parametrize("name,rows,cols", [("Q4_K", 14336, 4096), ("Q4_K", 4096, 14336), ("Q6_K", 128256, 4096)])
def test_config2_full_row_counts_on_sampled_rows(ex, orc, name, rows, cols):
    """benchmark config 2 at its true row counts (gate/up, down, lm_head), M = 1, 2, 4, 8.  The device computes the
    whole product; the CPU row kernels run on a sample of the weight rows (the first and last 128 and 256 spread
    over the matrix).  Every output must be finite; the sampled ones are held to the full parity bar.  The
    per-element figures are printed for the record (pytest -rP shows them)."""
    from llama_rust_b200 import row_bytes, synth
    kind = ALL[name]
    m = ex.synth(kind, rows, cols, synth.tensor_seed(2, f"config2.full.{name}.{rows}x{cols}"))
    w = ex.download(m)
    rng = np.random.default_rng(rows + cols)
    sel = np.unique(np.concatenate([np.arange(128), np.arange(rows - 128, rows), rng.integers(0, rows, 256)]))
    rb = row_bytes(kind, cols)
    wsel = np.ascontiguousarray(w.reshape(rows, rb)[sel]).reshape(-1)
    for tokens in (1, 2, 4, 8):
        x = synth.activations(tokens * cols, synth.tensor_seed(2, f"x.full.{tokens}"))
        y = np.full(rows * tokens, np.nan, np.float32)
        ex.gemm_resident(m, tokens, x, y)
        assert np.all(np.isfinite(y))
        cpu, exact, abs_sum = gemv_references(kind, len(sel), cols, wsel, x, tokens)
        got = np.ascontiguousarray(y.reshape(tokens, rows)[:, sel])
        per_elem, vs_exact = check_gemv(got, cpu, exact, abs_sum, cols, f"{name} {rows}x{cols} M={tokens}")
        print(f"config2 {name} {rows}x{cols} M={tokens}: max |gpu-cpu|/(1+|cpu|) = {per_elem:.2e}, max |gpu-exact|/(1+|exact|) = {vs_exact:.2e}")
    m.free()


def test_gemv_is_linear_and_deterministic(ex):
    """Size-independent properties on a benchmark-size matrix (gate/up 14336x4096 Q4_K)."""
    from llama_rust_b200 import synth
    m = ex.synth(Q4_K, 14336, 4096, 7)
    x1, x2 = synth.activations(4096, 1), synth.activations(4096, 2)
    y1, y2, y12, y1b = (np.empty(14336, np.float32) for _ in range(4))
    ex.gemv_resident(m, x1, y1)
    ex.gemv_resident(m, x2, y2)
    ex.gemv_resident(m, x1 + x2, y12)
    ex.gemv_resident(m, x1, y1b)
    assert np.array_equal(y1.view(np.uint32), y1b.view(np.uint32))
    scale = 1.0 + np.abs(y1) + np.abs(y2)
    assert (np.abs(y12 - (y1 + y2)) / scale).max() < 2e-5
    yb = np.empty(2 * 14336, np.float32)
    ex.gemm_resident(m, 2, np.concatenate([x1, x2]), yb)
    assert (np.abs(yb[:14336] - y1) / (1 + np.abs(y1))).max() < 1e-5
    assert (np.abs(yb[14336:] - y2) / (1 + np.abs(y2))).max() < 1e-5
    m.free()


# ---- device synth == host synth -----------------------------------------------------
@pytest.mark.parametrize("name", list(ALL))
def test_device_generator_matches_host_generator(ex, name):
    from llama_rust_b200 import synth
    kind = ALL[name]
    m = ex.synth(kind, 19, 1024, 0xC0FFEE)
    assert np.array_equal(ex.download(m), synth.packed_matrix(kind, 19, 1024, 0xC0FFEE))
    m.free()


@pytest.mark.parametrize("name", ["Q4_K", "Q6_K", "Q8_0", "Q4_0", "Q5_1", "Q4_1", "Q5_K"])
def test_a_row_of_activations_gives_the_same_bits_alone_and_inside_a_batch(ex, name):
    """The f32-faithful kernels hand their partial sums over every 4096 columns whatever the number of activation
    rows, so one activation row alone (its digit planes span 8192 columns) and the same row inside a batch of 2..8 give
    identical bits, also for rows longer than 4096 columns (ffn_down: 14336).  Engine batches and expert buckets rely
    on it."""
    from llama_rust_b200 import synth
    kind = ALL[name]
    ex.set_path(3)
    for rows, cols in ((64, 14336), (48, 8192), (32, 6144)):
        m = ex.synth(kind, rows, cols, synth.tensor_seed(9, f"{name}.{rows}.{cols}"))
        x = synth.activations(8 * cols, 77).reshape(8, cols)
        alone = np.empty((8, rows), np.float32)
        for t in range(8):
            ex.gemv_resident(m, x[t], alone[t])
        for batch in (2, 3, 8):
            y = np.empty(batch * rows, np.float32)
            ex.gemm_resident(m, batch, x[:batch], y)
            assert np.array_equal(y.reshape(batch, rows).view(np.uint32), alone[:batch].view(np.uint32)), (name, cols, batch)
        m.free()
    ex.set_path(0)


# ---- residency -----------------------------------------------------------------------
def test_residency_is_content_addressed_and_bounded(monkeypatch, orc):
    from llama_rust_b200 import Executor
    rng = np.random.default_rng(5)
    w = [random_packed(rng, Q8_0, 64, 256) for _ in range(3)]  # 64*8*34 = 17408 bytes each
    x = rng.standard_normal(256).astype(np.float32)
    monkeypatch.setenv("LLAMA_CUDA_CACHE_BYTES", str(2 * 17408))
    e = Executor(0)
    y = np.empty(64, np.float32)
    e.matmul(Q8_0, 64, 256, 1, w[0], x, y)
    e.matmul(Q8_0, 64, 256, 1, w[0].copy(), x, y)  # same bytes, another address: hit
    c = e.counters()
    assert (c["cache_misses"], c["cache_hits"], c["uploads"]) == (1, 1, 1)
    e.matmul(Q8_0, 64, 256, 1, w[1], x, y)
    e.matmul(Q8_0, 64, 256, 1, w[2], x, y)  # evicts w[0]
    c = e.counters()
    assert c["evictions"] == 1 and c["resident_bytes"] == 2 * 17408 and c["cache_limit"] == 2 * 17408
    e.matmul(Q8_0, 64, 256, 1, w[0], x, y)
    assert e.counters()["cache_misses"] == 4
    check_kernel(y, orc.gemv(Q8_0, 256, w[0], x, 64), "after eviction")
    e.close()
    monkeypatch.setenv("LLAMA_CUDA_CACHE_BYTES", "0")  # no residency, still executes
    e = Executor(0)
    e.matmul(Q8_0, 64, 256, 1, w[1], x, y)
    e.matmul(Q8_0, 64, 256, 1, w[1], x, y)
    c = e.counters()
    assert c["cache_hits"] == 0 and c["resident_bytes"] == 0 and c["uploads"] == 2
    check_kernel(y, orc.gemv(Q8_0, 256, w[1], x, 64), "uncached")
    e.close()
    monkeypatch.setenv("LLAMA_CUDA_CACHE_BYTES", "lots")
    e = Executor(0)
    with pytest.raises(Exception) as err:
        e.matmul(Q8_0, 64, 256, 1, w[1], x, y)
    assert err.value.code == 8
    e.close()


def test_keyed_residency_pins_and_verified_hits(monkeypatch, orc):
    """A caller key replaces the fingerprint (a hit reads only the key), pinned entries outlive eviction, and
    LLAMA_CUDA_CACHE_VERIFY=1 compares all bytes on a fingerprint hit (native_gpu.rs:96-98)."""
    from llama_rust_b200 import Executor
    rng = np.random.default_rng(6)
    w = [random_packed(rng, Q8_0, 64, 256) for _ in range(4)]
    x = rng.standard_normal(256).astype(np.float32)
    want = [orc.gemv(Q8_0, 256, wi, x, 64) for wi in w]
    monkeypatch.setenv("LLAMA_CUDA_CACHE_BYTES", str(2 * 17408))
    e = Executor(0)
    y = np.empty(64, np.float32)
    e.matmul_keyed((1, 100), Q8_0, 64, 256, 1, w[0], x, y)
    check_kernel(y, want[0], "keyed miss")
    e.matmul_keyed((1, 100), Q8_0, 64, 256, 1, w[1], x, y)  # the key decides, not the bytes: still matrix 0
    check_kernel(y, want[0], "keyed hit")
    c = e.counters()
    assert (c["cache_misses"], c["cache_hits"], c["uploads"]) == (1, 1, 1)
    e.matmul(Q8_0, 64, 256, 1, w[0], x, y)                   # a fingerprinted entry never matches a keyed one
    assert e.counters()["cache_misses"] == 2
    e.pin_key((1, 100))
    e.matmul(Q8_0, 64, 256, 1, w[2], x, y)                   # evicts the fingerprinted w[0], not the pinned key
    e.matmul(Q8_0, 64, 256, 1, w[3], x, y)                   # evicts w[2]
    c = e.counters()
    assert c["evictions"] == 2 and c["resident_bytes"] == 2 * 17408
    e.matmul_keyed((1, 100), Q8_0, 64, 256, 1, w[0], x, y)
    assert e.counters()["cache_hits"] == 2
    check_kernel(y, want[0], "pinned survives")
    e.pin_key((1, 100), False)
    e.matmul(Q8_0, 64, 256, 1, w[2], x, y)
    e.matmul(Q8_0, 64, 256, 1, w[1], x, y)                   # now the key goes too
    e.matmul_keyed((1, 100), Q8_0, 64, 256, 1, w[0], x, y)
    assert e.counters()["cache_hits"] == 2
    with pytest.raises(Exception):
        e.pin_key((9, 9))
    e.close()
    # with both slots pinned a third matrix runs once without residency
    e = Executor(0)
    e.matmul_keyed((1, 1), Q8_0, 64, 256, 1, w[0], x, y); e.pin_key((1, 1))
    e.matmul_keyed((1, 2), Q8_0, 64, 256, 1, w[1], x, y); e.pin_key((1, 2))
    e.matmul(Q8_0, 64, 256, 1, w[2], x, y)
    check_kernel(y, want[2], "beside pinned")
    c = e.counters()
    assert c["evictions"] == 0 and c["resident_bytes"] == 2 * 17408
    e.close()
    monkeypatch.setenv("LLAMA_CUDA_CACHE_VERIFY", "1")
    e = Executor(0)
    for i in (0, 0, 1, 0):
        e.matmul(Q8_0, 64, 256, 1, w[i].copy(), x, y)
        check_kernel(y, want[i], "verified")
    c = e.counters()
    assert (c["cache_misses"], c["cache_hits"]) == (2, 2)
    e.close()


def test_pinned_and_pageable_buffers_give_the_same_bits():
    """Decode-sized host-pointer calls deliver the result from the kernel into the caller's pinned
    buffer (or a pinned staging buffer for pageable memory) and signal completion through a mapped
    word; both routes and the copy-and-synchronize route must agree bit for bit."""
    import torch
    from llama_rust_b200 import Executor, synth
    from helpers import Q4_K, Q6_K
    ex = Executor(0)
    for dt, rows, cols in ((Q4_K, 4096, 4096), (Q6_K, 1024, 14336)):
        m = ex.synth(dt, rows, cols, 4242)
        for tokens in (1, 3, 8, 11):
            x = synth.activations(tokens * cols, 9).astype(np.float32)
            y_pageable = np.full(tokens * rows, np.nan, np.float32)
            ex.gemm_resident(m, tokens, x, y_pageable)
            xp = torch.from_numpy(x).pin_memory()
            yp = torch.full((tokens * rows,), float("nan")).pin_memory()
            for _ in range(2):  # the completion ticket changes from call to call
                yp.fill_(float("nan"))
                ex.gemm_resident(m, tokens, xp.numpy(), yp.numpy())
                assert np.array_equal(yp.numpy(), y_pageable)
        m.free()
    ex.close()
