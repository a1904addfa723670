"""Seeded synthetic inputs for the quantized matrix-product path (host generator).

Bit-identical twin of the device generator (``csrc/llr_synth.cu``): the same
seed gives the same packed bytes on both sides.  Everything is integer or
correctly rounded IEEE arithmetic, so there is no libm in the way:

* stream: SplitMix64 (the reference's test RNG, langtax/src/sample.rs:306-312)
  used as a counter generator, ``word(i) = mix(seed + (i+1)*0x9E3779B97F4A7C15)``;
* quant bits: raw bytes of the stream, little-endian within a word (Q8_0 codes
  are ``byte % 255 - 127``, i.e. uniform in [-127, 127]);
* "normal" n: Irwin-Hall over the twelve 16-bit fields of three consecutive
  words, ``n = (S - 393210) / 65536`` in binary64 (mean 0, variance 1, |n| <= 6);
* block scales: ``|n| * 0.01`` rounded to binary32, then truncated to binary16
  like the reference's ``f32_to_f16`` (langtax/src/fp16.rs:36-62);
* activations: ``float32(n)``; F16/BF16/F32 weights: ``float32(n * 0.02)``.

Words consumed per block (in this order): Q8_0 7 (4 quants, 3 scale); Q4_0 5
(2, 3); Q5_0 6 (1 qh [low 4 bytes], 2 quants, 3 d); Q5_1 9 (Q5_0 + 3 for m);
Q4_K 24 (16 quants, 2 scale bytes [12 bytes], 3 d, 3 dmin); Q6_K 29 (16 ql, 8 qh,
2 scales, 3 d); Q4_1 8 (2 quants, 3 d, 3 m); Q5_K 28 (16 quants, 4 qh, 2 scale bytes
[12 bytes], 3 d, 3 dmin); element formats 3 per element.
"""
from __future__ import annotations

import numpy as np

from .executor import BF16, F16, F32, Q4_0, Q4_1, Q4_K, Q5_0, Q5_1, Q5_K, Q6_K, Q8_0

_GAMMA = np.uint64(0x9E3779B97F4A7C15)
_M1 = np.uint64(0xBF58476D1CE4E5B9)
_M2 = np.uint64(0x94D049BB133111EB)

BLOCK_ELEMS = {F16: 1, BF16: 1, F32: 1, Q5_0: 32, Q5_1: 32, Q4_0: 32, Q4_1: 32, Q8_0: 32, Q4_K: 256, Q5_K: 256, Q6_K: 256}
BLOCK_BYTES = {F16: 2, BF16: 2, F32: 4, Q5_0: 22, Q5_1: 24, Q4_0: 18, Q4_1: 20, Q8_0: 34, Q4_K: 144, Q5_K: 176, Q6_K: 210}
WORDS_PER_BLOCK = {Q8_0: 7, Q4_0: 5, Q5_0: 6, Q5_1: 9, Q4_1: 8, Q4_K: 24, Q5_K: 28, Q6_K: 29, F16: 3, BF16: 3, F32: 3}


def tensor_seed(base: int, name: str) -> int:
    """One stream per tensor: base seed xor FNV-1a-64 of the tensor name."""
    h = 0xCBF29CE484222325
    for b in name.encode():
        h = ((h ^ b) * 0x100000001B3) & 0xFFFFFFFFFFFFFFFF
    return (base ^ h) & 0xFFFFFFFFFFFFFFFF


def words(seed: int, start: int, count: int) -> np.ndarray:
    """SplitMix64 outputs ``start .. start+count-1`` of the stream ``seed``."""
    with np.errstate(over="ignore"):
        i = np.arange(start + 1, start + count + 1, dtype=np.uint64)
        z = np.uint64(seed & 0xFFFFFFFFFFFFFFFF) + i * _GAMMA
        z = (z ^ (z >> np.uint64(30))) * _M1
        z = (z ^ (z >> np.uint64(27))) * _M2
        return z ^ (z >> np.uint64(31))


def _normal_from(w3: np.ndarray) -> np.ndarray:
    """w3: (..., 3) uint64 -> binary64 Irwin-Hall normal."""
    s = np.zeros(w3.shape[:-1], np.int64)
    for sh in (0, 16, 32, 48):
        s += ((w3 >> np.uint64(sh)) & np.uint64(0xFFFF)).astype(np.int64).sum(axis=-1)
    return (s.astype(np.float64) - 393210.0) / 65536.0


def f32_to_f16_trunc(f: np.ndarray) -> np.ndarray:
    """Vectorised langtax/src/fp16.rs:36-62 (round toward zero, subnormals kept)."""
    b = np.ascontiguousarray(f, np.float32).view(np.uint32).astype(np.int64)
    sign = (b >> 16) & 0x8000
    biased = (b >> 23) & 0xFF
    exp = biased - 127 + 15
    man = (b >> 13) & 0x3FF
    out = np.where(exp >= 31, sign | 0x7C00, 0)
    out = np.where((exp > 0) & (exp < 31), sign | (exp << 10) | man, out)
    shift = 1 - exp
    sub = (exp <= 0) & (biased != 0) & (shift <= 11)
    out = np.where(sub, sign | (((0x400 | man) >> np.clip(shift, 0, 62)) & 0x3FF), out)
    out = np.where((exp <= 0) & ~sub, sign, out)
    return out.astype(np.uint16)


def f32_to_bf16(f: np.ndarray) -> np.ndarray:
    u = np.ascontiguousarray(f, np.float32).view(np.uint32).astype(np.uint64)
    return ((u + np.uint64(0x7FFF) + ((u >> np.uint64(16)) & np.uint64(1))) >> np.uint64(16)).astype(np.uint16)


def _scale16(wblk: np.ndarray, k: int) -> np.ndarray:
    n = _normal_from(wblk[:, k:k + 3])
    return f32_to_f16_trunc((np.abs(n) * 0.01).astype(np.float32))


def _bytes_of(wblk: np.ndarray, k: int, nbytes: int) -> np.ndarray:
    nw = (nbytes + 7) // 8
    raw = np.ascontiguousarray(wblk[:, k:k + nw]).view(np.uint8).reshape(wblk.shape[0], nw * 8)
    return raw[:, :nbytes]


def _put16(out: np.ndarray, col: int, v: np.ndarray) -> None:
    out[:, col] = (v & 0xFF).astype(np.uint8)
    out[:, col + 1] = (v >> 8).astype(np.uint8)


def packed_blocks(dtype: int, first_block: int, n_blocks: int, seed: int) -> np.ndarray:
    """Packed bytes of blocks ``first_block .. first_block+n_blocks-1`` of a tensor stream."""
    wpb, bb = WORDS_PER_BLOCK[dtype], BLOCK_BYTES[dtype]
    w = words(seed, first_block * wpb, n_blocks * wpb).reshape(n_blocks, wpb)
    out = np.zeros((n_blocks, bb), np.uint8)
    if dtype == Q8_0:
        b = _bytes_of(w, 0, 32).astype(np.int32)
        out[:, 2:34] = ((b % 255) - 127).astype(np.int8).view(np.uint8)
        _put16(out, 0, _scale16(w, 4))
    elif dtype == Q4_0:
        out[:, 2:18] = _bytes_of(w, 0, 16)
        _put16(out, 0, _scale16(w, 2))
    elif dtype == Q5_0:
        out[:, 2:6] = _bytes_of(w, 0, 4)
        out[:, 6:22] = _bytes_of(w, 1, 16)
        _put16(out, 0, _scale16(w, 3))
    elif dtype == Q5_1:
        out[:, 4:8] = _bytes_of(w, 0, 4)
        out[:, 8:24] = _bytes_of(w, 1, 16)
        _put16(out, 0, _scale16(w, 3))
        _put16(out, 2, _scale16(w, 6))
    elif dtype == Q4_1:
        out[:, 4:20] = _bytes_of(w, 0, 16)
        _put16(out, 0, _scale16(w, 2))
        _put16(out, 2, _scale16(w, 5))
    elif dtype == Q5_K:
        out[:, 48:176] = _bytes_of(w, 0, 128)
        out[:, 16:48] = _bytes_of(w, 16, 32)
        out[:, 4:16] = _bytes_of(w, 20, 12)
        _put16(out, 0, _scale16(w, 22))
        _put16(out, 2, _scale16(w, 25))
    elif dtype == Q4_K:
        out[:, 16:144] = _bytes_of(w, 0, 128)
        out[:, 4:16] = _bytes_of(w, 16, 12)
        _put16(out, 0, _scale16(w, 18))
        _put16(out, 2, _scale16(w, 21))
    elif dtype == Q6_K:
        out[:, 0:128] = _bytes_of(w, 0, 128)
        out[:, 128:192] = _bytes_of(w, 16, 64)
        out[:, 192:208] = _bytes_of(w, 24, 16)
        _put16(out, 208, _scale16(w, 26))
    else:
        v = (_normal_from(w[:, 0:3]) * 0.02).astype(np.float32)
        if dtype == F32:
            out[:, :] = v.view(np.uint8).reshape(n_blocks, 4)
        elif dtype == F16:
            _put16(out, 0, f32_to_f16_trunc(v))
        else:
            _put16(out, 0, f32_to_bf16(v))
    return out.reshape(-1)


def packed_matrix(dtype: int, rows: int, cols: int, seed: int) -> np.ndarray:
    """rows x cols packed weights, rows contiguous (the layout llr_matrix_upload takes)."""
    be = BLOCK_ELEMS[dtype]
    assert cols % be == 0
    total = rows * (cols // be)
    chunks, step = [], 1 << 18
    for b0 in range(0, total, step):
        chunks.append(packed_blocks(dtype, b0, min(step, total - b0), seed))
    return np.concatenate(chunks) if chunks else np.zeros(0, np.uint8)


def activations(n: int, seed: int) -> np.ndarray:
    """n float32 values ~ N(0,1) (Irwin-Hall), element i from words 3i..3i+2."""
    w = words(seed, 0, 3 * n).reshape(n, 3)
    return _normal_from(w).astype(np.float32)
