"""ctypes view of the CPU oracle (``oracle/liboracle.so``).

TEST INFRASTRUCTURE ONLY: imported by ``tests/``, by ``__graft_entry__.smoke()``
and by ``bench.py``'s CPU-baseline legs, never by the shipped package.  Every
function here is a thin call into the C++ restatement of the reference's CPU
kernels (``oracle_scalar.cpp``, ``oracle_simd.cpp``); see ``oracle.h`` for the
reference file:line each one follows.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "liboracle.so")

F16, BF16, F32, Q5_0, Q5_1, Q4_0, Q8_0, Q4_K, Q6_K = 0, 1, 2, 6, 7, 12, 13, 17, 19
Q4_1, Q5_K = 5, 18
KINDS = {"F16": F16, "BF16": BF16, "F32": F32, "Q5_0": Q5_0, "Q5_1": Q5_1,
         "Q4_0": Q4_0, "Q8_0": Q8_0, "Q4_K": Q4_K, "Q6_K": Q6_K, "Q4_1": Q4_1, "Q5_K": Q5_K}
OK, ERR_UNALIGNED_COLS, ERR_SIZE, ERR_DTYPE, ERR_OVERFLOW = 0, 1, 2, 3, 4


class OracleError(Exception):
    def __init__(self, code: int):
        super().__init__(f"oracle error {code}")
        self.code = code


def build() -> None:
    """Compile the oracle (and, where the reference tree is mounted, its q8_gemv.c)."""
    subprocess.run(["make", "-C", _HERE, "all"], check=True, stdout=subprocess.DEVNULL)


def _load() -> C.CDLL:
    if not os.path.exists(_LIB_PATH):
        build()
    lib = C.CDLL(_LIB_PATH)
    i64, u8p, f32p, f64p = C.c_int64, C.c_void_p, C.c_void_p, C.c_void_p
    lib.orc_f16_to_f32.restype = C.c_float
    lib.orc_f16_to_f32.argtypes = [C.c_uint16]
    lib.orc_f32_to_f16.restype = C.c_uint16
    lib.orc_f32_to_f16.argtypes = [C.c_float]
    lib.orc_bf16_to_f32.restype = C.c_float
    lib.orc_bf16_to_f32.argtypes = [C.c_uint16]
    lib.orc_f32_to_bf16.restype = C.c_uint16
    lib.orc_f32_to_bf16.argtypes = [C.c_float]
    lib.orc_row_bytes.restype = i64
    lib.orc_row_bytes.argtypes = [C.c_int, i64]
    lib.orc_block_elems.argtypes = [C.c_int]
    lib.orc_block_bytes.argtypes = [C.c_int]
    lib.orc_dequant_row.argtypes = [C.c_int, i64, u8p, i64, f32p, i64]
    lib.orc_dequant_matrix.argtypes = [C.c_int, i64, i64, u8p, i64, f32p]
    lib.orc_dot_row_scalar.restype = C.c_float
    lib.orc_dot_row_scalar.argtypes = [C.c_int, u8p, i64, f32p, i64]
    lib.orc_dot_row_simd.restype = C.c_float
    lib.orc_dot_row_simd.argtypes = [C.c_int, u8p, i64, f32p, i64]
    lib.orc_gemv.argtypes = [C.c_int, i64, u8p, i64, f32p, i64, f32p, i64, C.c_int, C.c_int]
    lib.orc_gemm.argtypes = [C.c_int, i64, i64, u8p, i64, f32p, i64, f32p, i64, C.c_int, C.c_int]
    lib.orc_gemm_f64.argtypes = [C.c_int, i64, i64, u8p, i64, f32p, i64, f64p, i64]
    lib.orc_gemv_q8_0_q8_0.argtypes = [i64, u8p, i64, u8p, i64, f32p, i64, C.c_int]
    lib.orc_demo_q8_0.restype = None
    lib.orc_demo_q8_0.argtypes = [i64, i64, u8p, u8p]
    lib.orc_y_checksum.restype = C.c_uint64
    lib.orc_y_checksum.argtypes = [f32p, i64]
    lib.orc_pack_q8_0_block.restype = None
    lib.orc_pack_q8_0_block.argtypes = [C.c_float, u8p, u8p]
    lib.orc_pack_q4_0_from_i4.restype = None
    lib.orc_pack_q4_0_from_i4.argtypes = [C.c_float, u8p, u8p]
    lib.orc_pack_q5_0_block.restype = None
    lib.orc_pack_q5_0_block.argtypes = [C.c_float, u8p, u8p]
    lib.orc_pack_q5_1_block.restype = None
    lib.orc_pack_q5_1_block.argtypes = [C.c_float, C.c_float, u8p, u8p]
    lib.orc_pack_q4_1_block.restype = None
    lib.orc_pack_q4_1_block.argtypes = [C.c_float, C.c_float, u8p, u8p]
    lib.orc_pack_q5_k_block.restype = None
    lib.orc_pack_q5_k_block.argtypes = [C.c_float, C.c_float, u8p, u8p, u8p, u8p]
    lib.orc_pack_q4_k_block.restype = None
    lib.orc_pack_q4_k_block.argtypes = [C.c_float, C.c_float, u8p, u8p, u8p, u8p]
    lib.orc_pack_q6_k_block.restype = None
    lib.orc_pack_q6_k_block.argtypes = [C.c_float, u8p, u8p, u8p]
    lib.orc_pack_f16.restype = None
    lib.orc_pack_f16.argtypes = [f32p, i64, u8p]
    lib.orc_pack_bf16.restype = None
    lib.orc_pack_bf16.argtypes = [f32p, i64, u8p]
    lib.orc_rmsnorm.restype = None
    lib.orc_rmsnorm.argtypes = [f32p, f32p, i64, C.c_float]
    lib.orc_rope_norm.restype = None
    lib.orc_rope_norm.argtypes = [f32p, i64, i64, i64, i64, C.c_float]
    lib.orc_softmax.restype = None
    lib.orc_softmax.argtypes = [f32p, i64]
    lib.orc_silu.restype = C.c_float
    lib.orc_silu.argtypes = [C.c_float]
    lib.orc_argmax.restype = i64
    lib.orc_argmax.argtypes = [f32p, i64]
    lib.orc_topk.restype = None
    lib.orc_topk.argtypes = [f32p, i64, i64, C.c_void_p]
    lib.orc_moe_ffn.argtypes = [C.c_int, C.c_int, C.c_int, C.c_int, u8p, i64, C.c_int, C.c_void_p, C.c_void_p,
                                C.c_void_p, i64, i64, i64, f32p, f32p, C.c_void_p, f32p, C.c_int]
    return lib


lib = _load()


def _p(a: np.ndarray) -> int:
    return a.ctypes.data


def _u8(a) -> np.ndarray:
    return np.ascontiguousarray(np.frombuffer(a, dtype=np.uint8) if isinstance(a, (bytes, bytearray))
                                else a, dtype=np.uint8)


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


def _check(rc: int) -> None:
    if rc != OK:
        raise OracleError(rc)


def have_simd() -> bool:
    return bool(lib.orc_have_simd())


def f16_to_f32(h: int) -> float:
    return lib.orc_f16_to_f32(h)


def f32_to_f16(f: float) -> int:
    return lib.orc_f32_to_f16(f)


def row_bytes(kind: int, n_cols: int) -> int:
    rb = lib.orc_row_bytes(kind, n_cols)
    if rb < 0:
        raise OracleError(-rb)
    return rb


def block_elems(kind: int) -> int:
    return lib.orc_block_elems(kind)


def block_bytes(kind: int) -> int:
    return lib.orc_block_bytes(kind)


# ---- packers ---------------------------------------------------------------
def pack_q8_0_block(d: float, qs) -> np.ndarray:
    q = np.ascontiguousarray(qs, dtype=np.int8)
    assert q.size == 32
    out = np.zeros(34, np.uint8)
    lib.orc_pack_q8_0_block(d, _p(q), _p(out))
    return out


def pack_q4_0_from_i4(d: float, v) -> np.ndarray:
    q = np.ascontiguousarray(v, dtype=np.int8)
    assert q.size == 32
    out = np.zeros(18, np.uint8)
    lib.orc_pack_q4_0_from_i4(d, _p(q), _p(out))
    return out


def pack_q5_0_block(d: float, q5) -> np.ndarray:
    q = np.ascontiguousarray(q5, dtype=np.uint8)
    assert q.size == 32
    out = np.zeros(22, np.uint8)
    lib.orc_pack_q5_0_block(d, _p(q), _p(out))
    return out


def pack_q5_1_block(d: float, m: float, q5) -> np.ndarray:
    q = np.ascontiguousarray(q5, dtype=np.uint8)
    assert q.size == 32
    out = np.zeros(24, np.uint8)
    lib.orc_pack_q5_1_block(d, m, _p(q), _p(out))
    return out


def pack_q4_k_block(d: float, dmin: float, scales, mins, q4) -> np.ndarray:
    sc = np.ascontiguousarray(scales, dtype=np.uint8)
    mn = np.ascontiguousarray(mins, dtype=np.uint8)
    q = np.ascontiguousarray(q4, dtype=np.uint8)
    assert sc.size == 8 and mn.size == 8 and q.size == 256
    out = np.zeros(144, np.uint8)
    lib.orc_pack_q4_k_block(d, dmin, _p(sc), _p(mn), _p(q), _p(out))
    return out


def pack_q4_1_block(d: float, m: float, q4) -> np.ndarray:
    q = np.ascontiguousarray(q4, dtype=np.uint8)
    assert q.size == 32
    out = np.zeros(20, np.uint8)
    lib.orc_pack_q4_1_block(d, m, _p(q), _p(out))
    return out


def pack_q5_k_block(d: float, dmin: float, scales, mins, q5) -> np.ndarray:
    sc = np.ascontiguousarray(scales, dtype=np.uint8)
    mn = np.ascontiguousarray(mins, dtype=np.uint8)
    q = np.ascontiguousarray(q5, dtype=np.uint8)
    assert sc.size == 8 and mn.size == 8 and q.size == 256
    out = np.zeros(176, np.uint8)
    lib.orc_pack_q5_k_block(d, dmin, _p(sc), _p(mn), _p(q), _p(out))
    return out


def pack_q6_k_block(d: float, scales, qs) -> np.ndarray:
    sc = np.ascontiguousarray(scales, dtype=np.int8)
    q = np.ascontiguousarray(qs, dtype=np.int8)
    assert sc.size == 16 and q.size == 256
    out = np.zeros(210, np.uint8)
    lib.orc_pack_q6_k_block(d, _p(sc), _p(q), _p(out))
    return out


def pack_f32(values) -> np.ndarray:
    return _f32(values).view(np.uint8).copy()


def pack_f16(values) -> np.ndarray:
    v = _f32(values).ravel()
    out = np.zeros(2 * v.size, np.uint8)
    lib.orc_pack_f16(_p(v), v.size, _p(out))
    return out


def pack_bf16(values) -> np.ndarray:
    v = _f32(values).ravel()
    out = np.zeros(2 * v.size, np.uint8)
    lib.orc_pack_bf16(_p(v), v.size, _p(out))
    return out


# ---- kernels ---------------------------------------------------------------
def dequant_row(kind: int, n_cols: int, row) -> np.ndarray:
    r = _u8(row)
    y = np.zeros(n_cols, np.float32)
    _check(lib.orc_dequant_row(kind, n_cols, _p(r), r.size, _p(y), y.size))
    return y


def dequant_matrix(kind: int, n_rows: int, n_cols: int, w) -> np.ndarray:
    wb = _u8(w)
    y = np.zeros((n_rows, n_cols), np.float32)
    _check(lib.orc_dequant_matrix(kind, n_rows, n_cols, _p(wb), wb.size, _p(y)))
    return y


def dot_row(kind: int, row, x, simd: bool = False) -> float:
    r, xv = _u8(row), _f32(x)
    fn = lib.orc_dot_row_simd if simd else lib.orc_dot_row_scalar
    return fn(kind, _p(r), r.size, _p(xv), xv.size)


def gemv(kind: int, n_cols: int, w, x, n_rows: int, simd: bool = True, threads: int = 0) -> np.ndarray:
    wb, xv = _u8(w), _f32(x)
    y = np.zeros(n_rows, np.float32)
    _check(lib.orc_gemv(kind, n_cols, _p(wb), wb.size, _p(xv), xv.size, _p(y), y.size,
                        int(simd), threads))
    return y


def gemm(kind: int, n_cols: int, n_tokens: int, w, x, n_rows: int, simd: bool = True,
         threads: int = 0) -> np.ndarray:
    """Token-major result of shape (n_tokens, n_rows)."""
    wb, xv = _u8(w), _f32(x).ravel()
    y = np.zeros(max(n_tokens, 0) * n_rows, np.float32)
    _check(lib.orc_gemm(kind, n_cols, n_tokens, _p(wb), wb.size, _p(xv), xv.size, _p(y), y.size,
                        int(simd), threads))
    return y.reshape(n_tokens, n_rows)


def gemm_f64(kind: int, n_cols: int, n_tokens: int, w, x, n_rows: int) -> np.ndarray:
    wb, xv = _u8(w), _f32(x).ravel()
    out = np.zeros(n_tokens * n_rows, np.float64)
    _check(lib.orc_gemm_f64(kind, n_cols, n_tokens, _p(wb), wb.size, _p(xv), xv.size, _p(out),
                            out.size))
    return out.reshape(n_tokens, n_rows)


def gemv_q8_0_q8_0(n_cols: int, w, xq, n_rows: int, simd: bool = False) -> np.ndarray:
    wb, xb = _u8(w), _u8(xq)
    y = np.zeros(n_rows, np.float32)
    _check(lib.orc_gemv_q8_0_q8_0(n_cols, _p(wb), wb.size, _p(xb), xb.size, _p(y), y.size,
                                  int(simd)))
    return y


def demo_q8_0(n_cols: int, n_rows: int):
    rb = row_bytes(Q8_0, n_cols)
    w = np.zeros(rb * n_rows, np.uint8)
    xq = np.zeros(rb, np.uint8)
    lib.orc_demo_q8_0(n_cols, n_rows, _p(w), _p(xq))
    return w, xq


def y_checksum(y) -> int:
    v = _f32(y)
    return lib.orc_y_checksum(_p(v), v.size)


def moe_ffn(n_used: int, norm_w: bool, router_kind: int, router, expert_kind: int, gate, up, down,
            n_embd: int, n_ff: int, x):
    """Routed-expert FFN layer; returns (out[tokens, n_embd], sel_ids[tokens, n_used], sel_w)."""
    n_expert = len(gate)
    rt = _u8(router)
    xs = _f32(x).reshape(-1, n_embd)
    tokens = xs.shape[0]
    keep = [[_u8(a) for a in lst] for lst in (gate, up, down)]
    ptrs = [(C.c_void_p * n_expert)(*[a.ctypes.data for a in lst]) for lst in keep]
    out = np.zeros((tokens, n_embd), np.float32)
    ids = np.zeros((tokens, n_used), np.int32)
    w = np.zeros((tokens, n_used), np.float32)
    _check(lib.orc_moe_ffn(n_expert, n_used, int(norm_w), router_kind, _p(rt), rt.size, expert_kind,
                           ptrs[0], ptrs[1], ptrs[2], n_embd, n_ff, tokens, _p(xs), _p(out), _p(ids), _p(w), 0))
    return out, ids, w


def rmsnorm(x, w, eps: float) -> np.ndarray:
    """rmsnorm_inplace (langtax/src/decode.rs:11498) on a copy of one activation row."""
    out = np.array(x, dtype=np.float32).reshape(-1).copy()
    wv = _f32(w)
    lib.orc_rmsnorm(_p(out), _p(wv), out.size, eps)
    return out


def silu(x) -> np.ndarray:
    """silu_inplace (decode.rs:11826), element by element."""
    v = _f32(x)
    return np.array([lib.orc_silu(float(a)) for a in v], dtype=np.float32)


def ref_q8_gemv_binary() -> str | None:
    """Path of the reference's own q8_gemv.c compiled unmodified, if it was built."""
    p = os.path.join(_HERE, "_ref", "q8_gemv_ref")
    return p if os.path.exists(p) else None
