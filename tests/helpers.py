"""Fixtures shared by the parity tests: the deterministic inputs of the reference's
own GPU parity suite (langtax/tests/native_cuda_parity.rs:27-122) and seeded
random packed rows."""
import numpy as np

from oracle import pyoracle as orc

F16, BF16, F32, Q5_0, Q5_1, Q4_0, Q8_0, Q4_K, Q6_K = 0, 1, 2, 6, 7, 12, 13, 17, 19
Q4_1, Q5_K = 5, 18
ALL = {"F32": F32, "F16": F16, "BF16": BF16, "Q4_0": Q4_0, "Q5_0": Q5_0, "Q5_1": Q5_1,
       "Q8_0": Q8_0, "Q4_K": Q4_K, "Q6_K": Q6_K, "Q4_1": Q4_1, "Q5_K": Q5_K}


def values(row: int, cols: int) -> np.ndarray:
    """native_cuda_parity.rs:27-34"""
    c = np.arange(cols)
    return (((row * 7 + c * 11) % 31) - 15).astype(np.float32) / np.float32(16.0)


class Format:
    def __init__(self, name, kind, cols, pack_row):
        self.name, self.kind, self.cols, self.pack_row = name, kind, cols, pack_row


def formats():
    """native_cuda_parity.rs:36-122, plus Q5_0 and Q5_1 built the same way."""
    i = np.arange(32)
    k = np.arange(256)
    return [
        Format("F32", F32, 33, lambda r: orc.pack_f32(values(r, 33))),
        Format("F16", F16, 33, lambda r: orc.pack_f16(values(r, 33))),
        Format("BF16", BF16, 33, lambda r: orc.pack_bf16(values(r, 33))),
        Format("Q4_0", Q4_0, 32, lambda r: orc.pack_q4_0_from_i4(0.125, ((r * 3 + i * 7) % 16) - 8)),
        Format("Q8_0", Q8_0, 32, lambda r: orc.pack_q8_0_block(0.015625, ((r * 3 + i * 7) % 127) - 63)),
        Format("Q4_K", Q4_K, 256, lambda r: orc.pack_q4_k_block(
            0.03125, 0.015625, [1, 2, 3, 4, 5, 6, 7, 8], [2, 1, 0, 3, 1, 4, 2, 5], (r * 3 + k * 7) % 16)),
        Format("Q6_K", Q6_K, 256, lambda r: orc.pack_q6_k_block(
            0.0078125, [1, 2, -3, 4, 5, -6, 7, 8, -1, 2, 3, -4, 5, 6, -7, 8], ((r * 3 + k * 7) % 64) - 32)),
        Format("Q5_0", Q5_0, 32, lambda r: orc.pack_q5_0_block(0.0625, (r * 3 + i * 7) % 32)),
        Format("Q5_1", Q5_1, 32, lambda r: orc.pack_q5_1_block(0.0625, -0.5, (r * 3 + i * 7) % 32)),
    ]


def check_boundary(actual, expected, name):
    """native_cuda_parity.rs:150-158: |a - e| <= 1e-4 + 1e-4|e|, everything finite."""
    a = np.asarray(actual, np.float64).ravel()
    e = np.asarray(expected, np.float64).ravel()
    assert a.shape == e.shape
    assert np.all(np.isfinite(a)) and np.all(np.isfinite(e)), name
    bad = np.abs(a - e) > 1e-4 + 1e-4 * np.abs(e)
    assert not bad.any(), f"{name}: {int(bad.sum())} outputs off, first at {int(np.argmax(bad))}"


def check_kernel(actual, cpu, name, tol=1e-5):
    """The reference's CPU-kernel metric, quant.rs:10315: |y - e| / (1 + |e|) < 1e-5.
    Meaningful for short rows only: at the benchmark sizes the reference's own scalar
    and SIMD kernels differ by 1e-4 .. 7e-4 in this metric (see check_gemv)."""
    a = np.asarray(actual, np.float64).ravel()
    e = np.asarray(cpu, np.float64).ravel()
    rel = np.abs(a - e) / (1.0 + np.abs(e))
    assert rel.max() < tol, f"{name}: max rel {rel.max():.3e} at {int(np.argmax(rel))}"
    return float(rel.max())


U = 2.0 ** -24


def gemv_references(kind, rows, cols, w, x, tokens):
    """cpu: the AVX2 row kernels (what `--features simd` computes); exact: f64 dot of the
    f32-dequantized weights (native_cuda_parity.rs:124-148); abs_sum: sum |w_i x_i| per output."""
    cpu = orc.gemm(kind, cols, tokens, w, x, rows, simd=True)
    wf = orc.dequant_matrix(kind, rows, cols, w).astype(np.float64)
    xt = np.asarray(x, np.float64).reshape(tokens, cols)
    exact = xt @ wf.T
    abs_sum = np.abs(xt) @ np.abs(wf).T
    return cpu, exact, abs_sum


def check_gemv(actual, cpu, exact, abs_sum, n, name):
    """GEMV parity bar.
    (A) relative tolerance 1e-5 against the CPU row kernels, relative to the output
        vector's scale:  max|gpu - cpu| <= 1e-5 * max(1, max|cpu|);
    (B) the bounds the reference holds its own SIMD kernels to (simd/tests.rs:59-91):
        |gpu - exact| <= gamma(n+3) * sum|w x|  and
        |gpu - cpu|   <= max(64, 8 sqrt(n)) * u * sum|w x|;
    The per-element metric |gpu - cpu| / (1 + |cpu|) of the reference's unit tests
    (quant.rs:10315) is returned for the record but not asserted at these sizes: for a
    near-zero output of a long row it measures the f32 summation noise of the CPU kernel
    itself -- the reference's own scalar and AVX2 kernels differ by 1e-4 .. 7e-4 in it on
    the benchmark shapes, and its fixtures that use it are a few blocks long."""
    a = np.asarray(actual, np.float64).reshape(np.shape(exact))
    c = np.asarray(cpu, np.float64).reshape(np.shape(exact))
    assert np.all(np.isfinite(a)), name
    scale = max(1.0, float(np.abs(c).max()))
    da = np.abs(a - c)
    assert da.max() <= 1e-5 * scale, f"{name}: (A) max|gpu-cpu| {da.max():.3e} vs 1e-5*{scale:.3g}"
    k = n + 3.0
    gamma = k * U / (1 - k * U)
    assert np.all(np.abs(a - exact) <= gamma * abs_sum + 1e-30), f"{name}: (B) off the f64 value beyond gamma(n+3)"
    assert np.all(da <= max(64.0, 8.0 * np.sqrt(n)) * U * abs_sum + 1e-30), f"{name}: (B) outside the observed envelope"
    return float((da / (1.0 + np.abs(c))).max()), float((np.abs(a - exact) / (1.0 + np.abs(exact))).max())


def random_packed(rng, kind, rows, cols, scale_mode="normal"):
    """Uniform random quant bits with |N|*0.01 binary16 scales (benchmark configs)."""
    be, bb = orc.block_elems(kind), orc.block_bytes(kind)
    if be == 1:
        v = (rng.standard_normal(rows * cols) * 0.02).astype(np.float32)
        return {F32: orc.pack_f32, F16: orc.pack_f16, BF16: orc.pack_bf16}[kind](v)
    nb = rows * (cols // be)
    raw = rng.integers(0, 256, (nb, bb), dtype=np.uint8)
    from llama_rust_b200.synth import f32_to_f16_trunc

    def put(col):
        if scale_mode == "any_f16":  # every finite binary16 pattern, simd/tests.rs:795
            h = rng.integers(0, 0x10000, nb).astype(np.uint16)
            h = np.where((h >> 10) & 0x1F == 0x1F, h & 0x83FF, h)
        else:
            h = f32_to_f16_trunc((np.abs(rng.standard_normal(nb)) * 0.01).astype(np.float32))
        raw[:, col] = h & 0xFF
        raw[:, col + 1] = h >> 8
    for col in {Q8_0: [0], Q4_0: [0], Q5_0: [0], Q5_1: [0, 2], Q4_K: [0, 2], Q6_K: [208], Q4_1: [0, 2], Q5_K: [0, 2]}[kind]:
        put(col)
    if kind == Q8_0:  # codes uniform in [-127, 127]
        q = raw[:, 2:].view(np.int8)
        q[q == -128] = -127
    return raw.reshape(-1)
