"""The reference's quantized matrix-product entry points, served by the B200 executor.

Same names, argument order and error behaviour as the public functions of
langtax/src/quant.rs: ``gemv_<t>_f32(n_cols, w, x, y)`` (quant.rs:6144, 6191, 6214,
6891, 7010, 7033, 7176, 7199) and ``gemm_<t>_f32(n_cols, n_tokens, w, x, y)``
(quant.rs:6237-6478).  ``w`` is packed GGUF bytes, ``x`` token-major f32, ``y`` a
preallocated f32 array that is overwritten only when the whole call succeeds.
Each call goes where the reference's goes: through ``native_matmul``
(quant.rs:6683) into the thread's executor (``native_gpu::matmul``,
langtax/src/native_gpu.rs:124), here the C ABI's ``llr_matmul``.
"""
from __future__ import annotations

import threading

import numpy as np

from .executor import (BF16, F16, F32, Q4_0, Q4_K, Q5_0, Q5_1, Q6_K, Q8_0, Executor,
                       NativeCudaError)

QuantError = NativeCudaError

QK8_0 = QK4_0 = QK5_0 = QK5_1 = 32
QK_K = 256

_tls = threading.local()


def thread_executor() -> Executor:
    """One executor per inference thread (native_gpu.rs:114-116), created on first use."""
    ex = getattr(_tls, "executor", None)
    if ex is None:
        ex = _tls.executor = Executor(0)
    return ex


def reset_thread_executor() -> None:
    ex = getattr(_tls, "executor", None)
    if ex is not None:
        ex.close()
        _tls.executor = None


def native_matmul(kind: int, n_cols: int, n_tokens: int, w, x, y: np.ndarray) -> None:
    """quant.rs:6683-6758: shape validation, then the executor.  rows = len(y) / n_tokens."""
    if not isinstance(y, np.ndarray) or y.dtype != np.float32 or not y.flags.c_contiguous:
        raise TypeError("y must be a C-contiguous float32 numpy array")
    rows = (y.size // n_tokens) if n_tokens else 0
    thread_executor().matmul(kind, rows, n_cols, n_tokens, w, x, y)


def _gemv(kind):
    def f(n_cols: int, w, x, y: np.ndarray) -> None:
        native_matmul(kind, n_cols, 1, w, x, y)
    return f


def _gemm(kind):
    def f(n_cols: int, n_tokens: int, w, x, y: np.ndarray) -> None:
        native_matmul(kind, n_cols, n_tokens, w, x, y)
    return f


gemv_f16, gemm_f16 = _gemv(F16), _gemm(F16)
gemv_bf16, gemm_bf16 = _gemv(BF16), _gemm(BF16)
gemv_f32, gemm_f32 = _gemv(F32), _gemm(F32)
gemv_q4_0_f32, gemm_q4_0_f32 = _gemv(Q4_0), _gemm(Q4_0)
gemv_q5_0_f32, gemm_q5_0_f32 = _gemv(Q5_0), _gemm(Q5_0)
gemv_q5_1_f32, gemm_q5_1_f32 = _gemv(Q5_1), _gemm(Q5_1)
gemv_q8_0_f32, gemm_q8_0_f32 = _gemv(Q8_0), _gemm(Q8_0)
gemv_q4_k_f32, gemm_q4_k_f32 = _gemv(Q4_K), _gemm(Q4_K)
gemv_q6_k_f32, gemm_q6_k_f32 = _gemv(Q6_K), _gemm(Q6_K)

GEMV = {F16: gemv_f16, BF16: gemv_bf16, F32: gemv_f32, Q4_0: gemv_q4_0_f32, Q5_0: gemv_q5_0_f32,
        Q5_1: gemv_q5_1_f32, Q8_0: gemv_q8_0_f32, Q4_K: gemv_q4_k_f32, Q6_K: gemv_q6_k_f32}
GEMM = {F16: gemm_f16, BF16: gemm_bf16, F32: gemm_f32, Q4_0: gemm_q4_0_f32, Q5_0: gemm_q5_0_f32,
        Q5_1: gemm_q5_1_f32, Q8_0: gemm_q8_0_f32, Q4_K: gemm_q4_k_f32, Q6_K: gemm_q6_k_f32}


def dequant_rows(kind: int, n_rows: int, n_cols: int, w) -> np.ndarray:
    """dequant_<t>_row (quant.rs:7511-8853) for every row, computed on the device."""
    ex = thread_executor()
    m = ex.upload(kind, n_rows, n_cols, w)
    try:
        return ex.dequant_rows(m)
    finally:
        m.free()
