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
