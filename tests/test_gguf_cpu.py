"""The library's GGUF reader (llr_gguf_*, host code: no GPU needed) against the CPU restatement of the reference's
parser (oracle/gguf_oracle.py, langtax/src/gguf.rs:714-806), on the cases the reference's own tests cover
(gguf.rs:1027-2030: every metadata type with nested arrays, payloads equal to the file bytes, blob ranges,
removed / unsupported type ids) plus every truncation of a file and seeded corruptions."""
import struct

import numpy as np
import pytest

import gguf_files as gf
from oracle import gguf_oracle as go


def _open(image):
    from llama_rust_b200.gguf import GgufError, GgufFile
    try:
        return GgufFile(bytes(image)), None
    except GgufError as e:
        return None, e


def _oracle(image):
    try:
        return go.parse(image), None
    except go.GgufOracleError as e:
        return None, e


def _agree(image):
    """Both readers accept the image with the same tensors, or both reject it with the same error variant."""
    g, err = _open(image)
    want, werr = _oracle(image)
    if werr is not None:
        assert err is not None and err.kind == werr.kind, (err, werr)
        if werr.detail is not None:
            assert str(werr.detail) in str(err)
        return None
    assert err is None, (err, "oracle accepts")
    alignment, kv, tensors = want
    assert g.alignment == alignment and g.blob_len == len(image)
    got = g.tensors()
    assert [(t.name, t.ggml_type, t.shape, t.start, t.end) for t in got] == tensors
    _same_metadata(g, kv)
    return g


def _same_metadata(g, kv):
    """Every value the restatement read (the last one of a repeated key), through the typed readers of the library."""
    for key, v in kv.items():
        if "\x00" in key:
            continue  # keys are looked up as C strings
        ty = v[0]
        if ty == 9:
            assert g.kv_type(key) == (9, v[1], len(v[2])), key
            if v[1] == 5:
                assert g.kv_i32s(key) == [x[1] for x in v[2]], key
        elif ty == 8:
            assert g.kv_string(key) == v[1], key
        elif ty == 7:
            assert g.kv_bool(key) == v[1], key
        elif ty in (6, 12):
            fmt, ifmt = ("<f", "<I") if ty == 6 else ("<d", "<Q")
            if v[1] == v[1]:  # a NaN's payload is not kept by the restatement's float
                assert g.kv_bits(key) == (struct.unpack(ifmt, struct.pack(fmt, v[1]))[0], ty), key
        else:
            assert g.kv_bits(key) == (v[1] & (2 ** 64 - 1), ty), key


def _sample_file():
    rng = np.random.default_rng(11)
    nested = (gf.ARRAY, [(gf.U8, [1, 2])])
    kv = gf.DEFAULT_KV + [
        ("llama.ok", gf.BOOL, True), ("llama.scale", gf.F32, 1.5), ("llama.ids", gf.ARRAY, (gf.U32, [7, 9])),
        ("llama.u8", gf.U8, 1), ("llama.i8", gf.I8, -2), ("llama.u16", gf.U16, 3), ("llama.i16", gf.I16, -4),
        ("llama.i32", gf.I32, -5), ("llama.u64", gf.U64, 6), ("llama.i64", gf.I64, -7), ("llama.f64", gf.F64, 2.0),
        ("llama.nested", gf.ARRAY, nested), ("llama.merges", gf.ARRAY, (gf.STRING, ["a b", "c d"])),
        ("llama.types", gf.ARRAY, (gf.I32, [1, -1, 3])),
    ]
    payload = {n: rng.integers(0, 256, size, dtype=np.uint8).tobytes() for n, size in
               (("w_q8", 34), ("x_q8", 34), ("w_q4", 18), ("w_q4k", 288), ("x_q8k", 292), ("norm", 16), ("exps", 3 * 4 * 210))}
    tensors = [("w_q8", 8, (32, 1), payload["w_q8"]), ("x_q8", 8, (32,), payload["x_q8"]), ("w_q4", 2, (32, 1), payload["w_q4"]),
               ("w_q4k", 12, (256, 2), payload["w_q4k"]), ("x_q8k", 15, (256,), payload["x_q8k"]),
               ("norm", 0, (4,), payload["norm"]), ("exps", 14, (256, 4, 3), payload["exps"])]
    return gf.write_gguf(kv, tensors), payload


def test_metadata_of_every_type_and_payloads_equal_to_the_file_bytes():  # gguf.rs:1242-1393, :1936-1957
    image, payload = _sample_file()
    g = _agree(image)
    assert g.kv_u32("general.alignment") == 32 and g.kv_string("general.name") == "llama-rust"
    assert g.kv_bool("llama.ok") is True and g.kv_f32("llama.scale") == 1.5
    assert g.kv_u32("llama.scale") is None and g.kv_f32("llama.ok") is None and g.kv_string("llama.u8") is None  # typed readers
    assert g.kv_u32("absent") is None
    want = {"llama.u8": (1, 0), "llama.i8": (-2, 1), "llama.u16": (3, 2), "llama.i16": (-4, 3), "llama.i32": (-5, 5),
            "llama.u64": (6, 10), "llama.i64": (-7, 11)}
    for key, (val, ty) in want.items():
        assert g.kv_bits(key) == (val & (2 ** 64 - 1), ty), key
    assert g.kv_bits("llama.f64") == (struct.unpack("<Q", struct.pack("<d", 2.0))[0], 12)
    assert g.kv_type("llama.ids") == (9, 4, 2) and g.kv_type("llama.nested") == (9, 9, 1)
    assert g.kv_type("llama.merges") == (9, 8, 2)
    assert g.kv_i32s("llama.types") == [1, -1, 3] and g.kv_i32s("llama.ids") is None
    for t in g.tensors():
        assert image[t.start:t.end] == payload[t.name] and g.read(t.start, t.end).tobytes() == payload[t.name]
        assert t.start % 32 == 0
    e = g.tensor("exps")
    assert (e.n_cols, e.n_rows, e.n_parts, e.dtype) == (256, 4, 3, 19)
    assert g.tensor("x_q8k").dtype == -1 and g.tensor("x_q8").n_rows == 1 and g.tensor("nope") is None
    g.close()


def test_hand_assembled_image_pins_the_byte_layout():
    """A file written out byte by byte here, independent of the test writer: one F32 vector named "n" of 2 elements."""
    head = b"GGUF" + bytes([3, 0, 0, 0]) + (1).to_bytes(8, "little") + (0).to_bytes(8, "little")
    table = (1).to_bytes(8, "little") + b"n" + (1).to_bytes(4, "little") + (2).to_bytes(8, "little") + \
        (0).to_bytes(4, "little") + (0).to_bytes(8, "little")
    assert len(head) == 24 and len(table) == 33          # the table ends at byte 57, data starts at 64
    image = head + table + bytes(7) + np.array([1.5, -2.0], np.float32).tobytes()
    g = _agree(image)
    t = g.tensor("n")
    assert (t.start, t.end, t.shape, t.ggml_type, t.dtype) == (64, 72, (2,), 0, 2)
    assert np.array_equal(g.f32s("n"), np.array([1.5, -2.0], np.float32))
    g.close()
    assert _open(image[:71])[1].kind == "Truncated"


def test_every_truncation_is_reported_as_the_reference_reports_it():
    image, _ = _sample_file()
    data_start = min(t[3] for t in go.parse(image)[2])
    for n in list(range(0, data_start + 40)) + list(range(len(image) - 40, len(image))):
        _agree(image[:n])


def test_type_ids_removed_unsupported_and_accepted():  # gguf.rs:117-119, :165-204, :1960-2030
    for tid in range(-1, 46):
        n_el = 256 * 128
        size = n_el // go.LAYOUT[tid][1] * go.LAYOUT[tid][0] if tid in go.LAYOUT else 64
        image = gf.write_gguf(gf.DEFAULT_KV, [("w", 0, (n_el,), bytes(size))], type_ids=[tid])
        g = _agree(image)
        if g is not None:
            g.close()
    _, err = _open(gf.write_gguf(gf.DEFAULT_KV, [("w", 0, (4, 2), bytes(32))], type_ids=[36]))
    assert err.kind == "RemovedType" and "36" in str(err) and "removed" in str(err)
    _, err = _open(gf.write_gguf(gf.DEFAULT_KV, [("w", 0, (4, 2), bytes(32))], type_ids=[24]))
    assert err.kind == "UnsupportedType" and "24" in str(err)


def test_shapes_versions_magic_and_strings():
    ok = [("w", 12, (256, 2), bytes(288))]
    assert _agree(gf.write_gguf(gf.DEFAULT_KV, ok)) is not None
    for bad in (gf.write_gguf(gf.DEFAULT_KV, ok, magic=b"GGML"), gf.write_gguf(gf.DEFAULT_KV, ok, version=2),
                gf.write_gguf(gf.DEFAULT_KV, [("w", 12, (255, 2), bytes(288))]),       # not a multiple of the block
                gf.write_gguf(gf.DEFAULT_KV, [("w", 0, (), bytes(4))]),                # no dimension
                gf.write_gguf(gf.DEFAULT_KV, [("w", 0, (1, 1, 1, 1, 1), bytes(4))]),   # five dimensions
                gf.write_gguf(gf.DEFAULT_KV, [("w", 0, (0,), bytes(4))]),
                gf.write_gguf(gf.DEFAULT_KV, [("w", 0, (-4,), bytes(16))]),
                gf.write_gguf(gf.DEFAULT_KV, [("w", 0, (2 ** 40, 2 ** 40), bytes(16))]),  # element count overflows
                gf.write_gguf(gf.DEFAULT_KV, [("w", 0, (2 ** 62,), bytes(16))]),         # payload beyond the file
                gf.write_gguf([(b"\xff\xfe", gf.U32, 1)], ok),                         # key is not UTF-8
                gf.write_gguf(gf.DEFAULT_KV, [(b"\xc0\x80", 12, (256, 2), bytes(288))]),  # overlong encoding
                gf.write_gguf([("k", 13, 0)] if False else gf.DEFAULT_KV, ok)[:24]):
        _agree(bad)
    # an unknown metadata value type
    image = bytearray(gf.write_gguf([("k", gf.U32, 5)], ok))
    image[24 + 8 + 1:24 + 8 + 1 + 4] = (13).to_bytes(4, "little")
    _, err = _open(image)
    assert err.kind == "UnsupportedKv" and "13" in str(err)
    _agree(image)
    # negative counts
    image = bytearray(gf.write_gguf(gf.DEFAULT_KV, ok))
    image[8:16] = (-1).to_bytes(8, "little", signed=True)
    _agree(image)


def test_alignment_key_repeated_keys_and_repeated_names():
    kv = [("general.alignment", gf.U32, 64), ("x", gf.U32, 1), ("x", gf.U32, 2)]
    tensors = [("w", 0, (3,), bytes(range(12))), ("w", 0, (5,), bytes(range(20))), ("v", 1, (6,), bytes(range(12)))]
    image = gf.write_gguf(kv, tensors, layout_alignment=64)
    g = _agree(image)
    assert g.alignment == 64 and g.kv_u32("x") == 2                 # the last value of a key wins
    assert g.tensor("w").shape == (3,) and len(g.tensors()) == 3    # the first tensor of a name wins
    assert all(t.start % 64 == 0 for t in g.tensors())
    g.close()
    # alignment 0 or of another type falls back to 32
    for kv in ([("general.alignment", gf.U32, 0)], [("general.alignment", gf.U64, 64)]):
        g = _agree(gf.write_gguf(kv, tensors))
        assert g.alignment == 32
        g.close()


def test_seeded_corruptions_never_disagree_with_the_reference_rules():
    image, _ = _sample_file()
    table_end = min(t[3] for t in go.parse(image)[2])
    rng = np.random.default_rng(5)
    for _ in range(450):
        bad = bytearray(image)
        kind = int(rng.integers(0, 3))
        if kind == 0:  # a few bytes of the tables replaced
            for _ in range(int(rng.integers(1, 4))):
                bad[int(rng.integers(0, table_end))] = int(rng.integers(0, 256))
        elif kind == 1:  # one bit flipped, then the file cut anywhere
            bad[int(rng.integers(0, table_end))] ^= 1 << int(rng.integers(0, 8))
            bad = bad[: int(rng.integers(0, len(bad)))]
        else:  # eight bytes replaced by an extreme count or offset
            at = int(rng.integers(0, table_end - 8))
            bad[at:at + 8] = [0, 1, 2 ** 31, 2 ** 32 - 1, 2 ** 63, 2 ** 64 - 1][int(rng.integers(0, 6))].to_bytes(8, "little")
        want, werr = _oracle(bytes(bad))
        if werr is None and sum(len(v[2]) for v in want[1].values() if v[0] == 9) > 10 ** 6:
            continue  # a corrupted count that still fits the file: nothing to learn, much to allocate
        g = _agree(bytes(bad))
        if g is not None:
            g.close()


def test_a_tensor_name_with_nul_bytes_crosses_the_boundary_whole():
    """A name is any UTF-8 string (read_string, gguf.rs:903), NUL bytes included: the record carries its length, and a
    lookup by C string neither finds such a tensor nor takes it for the prefix before the NUL."""
    from llama_rust_b200.gguf import GgufFile
    payload = bytes(range(16))
    image = gf.write_gguf(gf.DEFAULT_KV, [("a\x00b", 0, (4,), payload), ("a", 0, (4,), payload[::-1])])
    g = _agree(image)
    assert [t.name for t in g.tensors()] == ["a\x00b", "a"]
    t = g.tensor("a")
    assert t is not None and g.read(t.start, t.end).tobytes() == payload[::-1]
    g.close()
    assert isinstance(GgufFile(image), GgufFile)


def test_stable_keys_are_the_blob_ranges_of_rows_and_parts():
    """quant_mat / quant_mat_rows (decode.rs:9612-9713): rows [first, first + n) of part p of a tensor start at
    start + (p * rows + first) * row_bytes; the key of that slice is (open file, that byte offset).  Host arithmetic
    only: no executor is involved."""
    from llama_rust_b200 import NativeCudaError
    image, _ = _sample_file()
    g = _agree(image)
    w, e, nrm = g.tensor("w_q4k"), g.tensor("exps"), g.tensor("norm")
    file_id = g.key("w_q4k")[0]
    assert g.key("w_q4k") == (file_id, w.start) and g.key("w_q4k", 0, 1, 1) == (file_id, w.start + 144)
    assert g.key("exps", 2) == (file_id, e.start + 2 * 4 * 210) and g.key("exps", 1, 3, 1) == (file_id, e.start + (4 + 3) * 210)
    assert g.key("exps", 0, 0, 4) == g.key("exps") and g.key("norm") == (file_id, nrm.start)
    assert e.start + 3 * 4 * 210 == e.end
    for bad in (("exps", 3), ("exps", 0, 4, 1), ("exps", 0, 2, 3), ("exps", 0, 1, 0), ("w_q4k", 1), ("absent",), ("x_q8k",)):
        with pytest.raises(NativeCudaError):
            g.key(*bad)
    other = _agree(image)
    assert other.key("w_q4k")[0] != file_id  # another open file, another key space
    other.close()
    g.close()


def test_open_from_a_path_maps_the_file(tmp_path):
    from llama_rust_b200.gguf import GgufError, GgufFile
    image, payload = _sample_file()
    p = tmp_path / "m.gguf"
    p.write_bytes(image)
    with GgufFile(str(p)) as g:
        assert g.blob_len == len(image)
        t = g.tensor("w_q4k")
        assert g.read(t.start, t.end).tobytes() == payload["w_q4k"]
    with pytest.raises(GgufError):
        GgufFile(str(tmp_path / "absent.gguf"))


def test_llama_hyper_parameters_of_dense_and_routed_expert_files():
    """`llama_config` (decode.rs:1905-1930, 7461-7515): the walk's hyper-parameters from `<arch>.*` metadata, with the
    reference's defaults (kv heads = heads, head_dim = n_embd / heads, eps 1e-5, base 10000), the vocabulary from the
    embedding's rows, and the expert counts of architecture=llama files with routed experts (llama_moe_into :10366)."""
    from llama_rust_b200.gguf import GgufError, GgufFile, llama_config
    base = gf.DEFAULT_KV + [("general.architecture", gf.STRING, "llama"), ("llama.block_count", gf.U32, 3),
                            ("llama.embedding_length", gf.U32, 64), ("llama.feed_forward_length", gf.U32, 128),
                            ("llama.attention.head_count", gf.U32, 4)]
    embd = [("token_embd.weight", 0, (64, 10), np.zeros(640, np.float32).tobytes())]
    cfg = llama_config(GgufFile(gf.write_gguf(base, embd)))
    assert cfg == dict(n_layer=3, n_embd=64, n_head=4, n_head_kv=4, head_dim=16, n_ff=128, n_vocab=10, n_ctx=2048, rms_eps=1e-5,
                       rope_base=10000.0)
    moe = base + [("llama.attention.head_count_kv", gf.U32, 2), ("llama.expert_count", gf.U32, 8), ("llama.expert_used_count", gf.U32, 2),
                  ("llama.context_length", gf.U32, 512)]
    cfg = llama_config(GgufFile(gf.write_gguf(moe, embd)), n_ctx=100)
    assert (cfg["n_head_kv"], cfg["n_expert"], cfg["n_expert_used"], cfg["n_ctx"]) == (2, 8, 2, 100)
    assert llama_config(GgufFile(gf.write_gguf(moe, embd)))["n_ctx"] == 512
    with pytest.raises(GgufError):  # more experts used than there are
        llama_config(GgufFile(gf.write_gguf(base + [("llama.expert_count", gf.U32, 2), ("llama.expert_used_count", gf.U32, 3)], embd)))
    with pytest.raises(GgufError):  # a required key is missing
        llama_config(GgufFile(gf.write_gguf(base[:-1], embd)))
