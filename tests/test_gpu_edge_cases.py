"""The reference's SIMD edge-case tests (langtax/src/simd/tests.rs), run against the CUDA kernels through the
GEMV entry (one activation row) and the GEMM entry (several), instead of against the AVX2 kernels:

* every code value in every position with one non-zero term (:755, :933, :1110, :1272, Q8_0 including -128);
* the Q5_1 probe for an offset that is fused into the product instead of added after it (:1146-1172);
* cancelling rows and one huge term among tiny ones, held to gamma(n+3) * sum|w x| (:1533-1595);
* block counts 1, 2, 3, 4, 5, 8, 16 (:196-199).

What can be asked of a kernel depends on its arithmetic.  The shape-agnostic kernel (path 1) multiplies the
bit-exact dequantized weight by the activation with one FMA per term, as the scalar CPU kernel does, so a row
with a single non-zero term must come out bit-equal.  The staged kernel (path 2) factors the block scale out
of the sum and the integer tensor-core kernel (path 3) splits the activation into digits: both round in another
order, and are held to the reference's proven bound for any correctly rounded summation order."""
import numpy as np
import pytest

from helpers import ALL, F32, Q4_0, Q5_0, Q5_1, Q8_0, random_packed

pytestmark = pytest.mark.gpu

U = 2.0 ** -24
PATHS = {"generic": 1, "staged": 2, "auto": 0}


def gamma_bound(n, abs_sum):
    k = n + 3.0
    return k * U / (1 - k * U) * abs_sum


@pytest.fixture(scope="module")
def ex():
    from llama_rust_b200 import Executor
    e = Executor(0)
    yield e
    e.close()


def _single_term_blocks(orc, name):
    """One 32-column row per (position, code): every other code is the format's zero."""
    codes = {"Q4_0": range(-8, 8), "Q5_0": range(32), "Q5_1": range(32), "Q8_0": range(-128, 128)}[name]
    rows = {}
    for pos in range(32):
        blocks = []
        for code in codes:
            if name == "Q4_0":
                v = np.zeros(32, np.int8); v[pos] = code
                blocks.append(orc.pack_q4_0_from_i4(0.375, v))
            elif name == "Q5_0":
                v = np.full(32, 16, np.uint8); v[pos] = code
                blocks.append(orc.pack_q5_0_block(0.375, v))
            elif name == "Q5_1":
                v = np.zeros(32, np.uint8); v[pos] = code
                blocks.append(orc.pack_q5_1_block(0.375, 0.0, v))
            else:
                v = np.zeros(32, np.int8); v[pos] = code
                blocks.append(orc.pack_q8_0_block(0.375, v))
        rows[pos] = np.concatenate(blocks)
    return rows, len(codes)


@pytest.mark.parametrize("name", ["Q4_0", "Q5_0", "Q5_1", "Q8_0"])
def test_single_term_rows_every_code_every_position(ex, orc, name):  # simd/tests.rs:755, 933, 1110, 1272
    kind = ALL[name]
    rows, n_codes = _single_term_blocks(orc, name)
    for pos in range(32):
        w = rows[pos]
        x = np.zeros(32, np.float32); x[pos] = 1.7
        cpu = orc.gemv(kind, 32, w, x, n_codes, simd=False, threads=1)
        m = ex.upload(kind, n_codes, 32, w)
        for pname, path in PATHS.items():
            ex.set_path(path)
            y = np.empty(n_codes, np.float32)
            ex.gemv_resident(m, x, y)                      # the GEMV table
            y3 = np.empty(3 * n_codes, np.float32)
            x3 = np.zeros((3, 32), np.float32); x3[0, pos] = 1.7; x3[2, pos] = -0.3
            ex.gemm_resident(m, 3, x3, y3)                 # the GEMM table
            cpu3 = orc.gemm(kind, 32, 3, w, x3, n_codes, simd=False)
            if pname == "generic":
                assert np.array_equal(y.view(np.uint32), cpu.view(np.uint32)), (name, pos, pname)
                assert np.array_equal(y3.view(np.uint32), cpu3.reshape(-1).view(np.uint32)), (name, pos, pname, "gemm")
            else:  # one product of two roundings instead of one: within two units in the last place
                assert np.all(np.abs(y - cpu) <= 2 * U * np.abs(cpu) * 2 + 1e-45), (name, pos, pname)
                assert np.all(np.abs(y3 - cpu3.reshape(-1)) <= 2 * U * np.abs(cpu3.reshape(-1)) * 2 + 1e-45), (name, pos, pname)
        m.free()
    ex.set_path(0)


def test_q5_1_offset_is_added_after_the_rounded_product(ex, orc):  # simd/tests.rs:1146-1172
    """The reference's probe for a fused q*d + m: random codes, a scale with a full mantissa (as far as binary16 keeps
    it), a tiny offset, all-ones activations, 64 trials.  The device dequantizer must give the scalar kernel's weights
    bit for bit (product rounded, then the offset added), and every GEMV kernel must agree with the scalar CPU row dot
    within the reference's agreement bound max(64, 8 sqrt(n)) * u * sum|w x|; the shape-agnostic kernel, which
    multiplies the bit-exact weights one by one, is also held to the single-kernel bound gamma(n+3)."""
    rng = np.random.default_rng(0x5EED5102)
    for trial in range(64):
        qs = rng.integers(0, 32, 32).astype(np.uint8)
        d = float(np.float32(np.uint32(0x3F7FFFFF).view(np.float32)) * np.float32(1.0 + rng.random()))
        mm = float(np.uint32(0x34000001).view(np.float32))
        w = orc.pack_q5_1_block(d, mm, qs)
        want_w = orc.dequant_row(Q5_1, 32, w)
        dd = np.float32(orc.f16_to_f32(int(w[0]) | int(w[1]) << 8))
        m32 = np.float32(orc.f16_to_f32(int(w[2]) | int(w[3]) << 8))
        twice = np.array([np.float32(np.float32(np.float32(q) * dd) + m32) for q in qs], np.float32)
        assert np.array_equal(want_w.view(np.uint32), twice.view(np.uint32))
        m = ex.upload(Q5_1, 1, 32, w)
        assert np.array_equal(ex.dequant_rows(m).reshape(-1).view(np.uint32), twice.view(np.uint32)), trial
        x = np.ones(32, np.float32)
        cpu = float(orc.dot_row(Q5_1, w, x, simd=False))
        abs_sum = float(np.abs(twice.astype(np.float64)).sum())
        exact = float(twice.astype(np.float64).sum())
        for pname, path in PATHS.items():
            ex.set_path(path)
            y = np.empty(1, np.float32)
            ex.gemv_resident(m, x, y)
            assert abs(float(y[0]) - cpu) <= max(64.0, 8 * np.sqrt(32)) * U * abs_sum, (pname, trial)
            if pname == "generic":
                assert abs(float(y[0]) - exact) <= gamma_bound(32, abs_sum), (pname, trial)
        m.free()
    ex.set_path(0)


def _signed(rng, scale):
    return np.float32((rng.random() * 2.0 - 1.0) * scale)


@pytest.mark.parametrize("path", list(PATHS))
def test_cancelling_rows_stay_within_the_bound(ex, path):  # simd/tests.rs:1533-1567
    ex.set_path(PATHS[path])
    rng = np.random.default_rng(0x5EEDCA11)
    for n in (8, 64, 256, 4096):
        w = np.array([_signed(rng, 1000.0) for _ in range(n)], np.float32)
        x = np.where(np.arange(n) % 2 == 0, 1.0, -1.0).astype(np.float32)
        for i in range(n // 2):  # near-total cancellation: mirror the first half
            w[n - 1 - i] = -w[i] if (n - 1 - i) % 2 == i % 2 else w[i]
        exact = float(np.dot(w.astype(np.float64), x.astype(np.float64)))
        abs_sum = float(np.sum(np.abs(w.astype(np.float64) * x)))
        m = ex.upload(F32, 1, n, w.view(np.uint8))
        for tokens in (1, 2):
            y = np.empty(tokens, np.float32)
            ex.gemm_resident(m, tokens, np.tile(x, tokens), y)
            assert np.all(np.abs(y.astype(np.float64) - exact) <= gamma_bound(n, abs_sum)), (path, n, tokens, y, exact)
        m.free()
    ex.set_path(0)


@pytest.mark.parametrize("path", list(PATHS))
def test_wide_dynamic_range_stays_within_the_bound(ex, path):  # simd/tests.rs:1570-1595
    ex.set_path(PATHS[path])
    rng = np.random.default_rng(0x5EEDD17A)
    for n in (9, 33, 257, 1024):
        for spike in (0, 1, 7, 8):
            w = np.array([_signed(rng, 1e-6) for _ in range(n)], np.float32)
            x = np.array([_signed(rng, 1e-6) for _ in range(n)], np.float32)
            w[spike] = 1e12
            exact = float(np.dot(w.astype(np.float64), x.astype(np.float64)))
            abs_sum = float(np.sum(np.abs(w.astype(np.float64) * x.astype(np.float64))))
            m = ex.upload(F32, 1, n, w.view(np.uint8))
            y = np.empty(1, np.float32)
            ex.gemv_resident(m, x, y)
            assert abs(float(y[0]) - exact) <= gamma_bound(n, abs_sum), (path, n, spike)
            m.free()
    ex.set_path(0)


@pytest.mark.parametrize("name", list(ALL))
def test_block_count_sweep_within_the_proven_bound(ex, orc, name):  # simd/tests.rs:196-199, 59-91
    """Rows of 1, 2, 3, 4, 5, 8 and 16 blocks (of at least 32 columns), random bits, on every kernel that takes the
    shape: |gpu - exact| <= gamma(n+3) sum|w x| and |gpu - cpu| within twice that, for one and for three activation rows."""
    kind = ALL[name]
    rng = np.random.default_rng(0x5EED + kind)
    be = max(orc.block_elems(kind), 32)
    for blocks in (1, 2, 3, 4, 5, 8, 16):
        n = blocks * be
        rows = 5
        w = random_packed(rng, kind, rows, n)
        wf = orc.dequant_matrix(kind, rows, n, w).astype(np.float64)
        m = ex.upload(kind, rows, n, w)
        for tokens in (1, 3):
            x = rng.standard_normal((tokens, n)).astype(np.float32)
            exact = x.astype(np.float64) @ wf.T
            abs_sum = np.abs(x.astype(np.float64)) @ np.abs(wf).T
            cpu = orc.gemm(kind, n, tokens, w, x, rows, simd=True)
            for pname, path in list(PATHS.items()) + [("mma", 3)]:
                ex.set_path(path)
                y = np.empty(tokens * rows, np.float32)
                ex.gemm_resident(m, tokens, x, y)
                y = y.reshape(tokens, rows).astype(np.float64)
                bound = gamma_bound(n, abs_sum)
                assert np.all(np.abs(y - exact) <= bound + 1e-30), (name, blocks, tokens, pname)
                assert np.all(np.abs(y - cpu) <= 2 * bound + 1e-30), (name, blocks, tokens, pname)
        m.free()
    ex.set_path(0)
