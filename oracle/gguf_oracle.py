"""TEST INFRASTRUCTURE ONLY: CPU restatement of the reference's GGUF v3 reader, the checker for llr_gguf_*.

Follows langtax/src/gguf.rs: `parse_gguf` (:714-806), `read_kv_value` (:925-950), the ggml type table
(`GgmlType::from_i32` :165-204, `is_ggml_removed_type_id` :117-119, `layout` :248-283) and the block sizes of
langtax/src/quant.rs:86-183.  Errors carry the name of the reference's GgufError variant (:338-370).

Parity unpinned: the reference holds no byte-level golden GGUF file; its own tests build files with `write_gguf`
(:640-712) and read them back.  The files of tests/gguf_files.py follow that writer's layout rule for rule (header,
metadata, tensor table, payloads aligned to `general.alignment` relative to the aligned end of the table), and the
hand-assembled image in tests/test_gguf_cpu.py pins the byte layout independently of both."""
import struct

REMOVED = {4, 5, 31, 32, 33, 36, 37, 38}
# ggml type id -> (bytes per block, elements per block)
LAYOUT = {0: (4, 1), 1: (2, 1), 30: (2, 1), 2: (18, 32), 3: (20, 32), 6: (22, 32), 7: (24, 32), 8: (34, 32), 9: (36, 32),
          10: (84, 256), 11: (110, 256), 12: (144, 256), 13: (176, 256), 14: (210, 256), 15: (292, 256), 16: (66, 256),
          17: (74, 256), 18: (98, 256), 19: (50, 256), 20: (18, 32), 21: (110, 256), 22: (82, 256), 23: (136, 256),
          29: (56, 256), 34: (54, 256), 35: (66, 256), 39: (17, 32), 40: (36, 64), 41: (18, 128), 42: (18, 64)}
SCALARS = {0: "<B", 1: "<b", 2: "<H", 3: "<h", 4: "<I", 5: "<i", 6: "<f", 10: "<Q", 11: "<q", 12: "<d"}


class GgufOracleError(Exception):
    def __init__(self, kind, detail=None):
        super().__init__(kind if detail is None else f"{kind}({detail})")
        self.kind, self.detail = kind, detail


class _Reader:
    def __init__(self, data):
        self.d, self.pos = memoryview(data), 0

    def take(self, n):
        if n > len(self.d) - self.pos:
            raise GgufOracleError("Truncated")
        s = self.d[self.pos:self.pos + n]
        self.pos += n
        return bytes(s)

    def num(self, fmt):
        return struct.unpack(fmt, self.take(struct.calcsize(fmt)))[0]

    def string(self):
        raw = self.take(self.num("<Q"))
        try:
            return raw.decode("utf-8")
        except UnicodeDecodeError:
            raise GgufOracleError("Utf8")

    def value(self, ty):
        if ty in SCALARS:
            return (ty, self.num(SCALARS[ty]))
        if ty == 7:
            return (7, self.num("<B") != 0)
        if ty == 8:
            return (8, self.string())
        if ty == 9:
            elem, n = self.num("<i"), self.num("<Q")
            return (9, elem, [self.value(elem) for _ in range(n)])
        raise GgufOracleError("UnsupportedKv", ty)


def parse(data):
    """-> (alignment, kv dict, tensors [(name, ggml type, shape, start, end)]) or raises GgufOracleError."""
    r = _Reader(data)
    if r.take(4) != b"GGUF":
        raise GgufOracleError("Magic")
    version = r.num("<I")
    if version != 3:
        raise GgufOracleError("Version", version)
    n_tensors, n_kv = r.num("<q"), r.num("<q")
    if n_tensors < 0 or n_kv < 0:
        raise GgufOracleError("Truncated")
    kv = {}
    for _ in range(n_kv):
        key = r.string()
        kv[key] = r.value(r.num("<i"))
    al = kv.get("general.alignment")
    alignment = al[1] if al is not None and al[0] == 4 and al[1] > 0 else 32
    raw = []
    for _ in range(n_tensors):
        name = r.string()
        n_dims = r.num("<I")
        if n_dims == 0 or n_dims > 4:
            raise GgufOracleError("Shape")
        shape = []
        for _ in range(n_dims):
            d = r.num("<q")
            if d <= 0:
                raise GgufOracleError("Shape")
            shape.append(d)
        ty = r.num("<i")
        if ty in REMOVED:
            raise GgufOracleError("RemovedType", ty)
        if ty not in LAYOUT:
            raise GgufOracleError("UnsupportedType", ty)
        raw.append((name, ty, tuple(shape), r.num("<Q")))
    data_start = -(-r.pos // alignment) * alignment
    tensors = []
    for name, ty, shape, offset in raw:
        n_el = 1
        for d in shape:
            n_el *= d
        if n_el >= 1 << 64:
            raise GgufOracleError("Shape")
        block, k = LAYOUT[ty]
        if n_el % k:
            raise GgufOracleError("Shape")
        start = data_start + offset
        end = start + n_el // k * block
        if end > len(data):
            raise GgufOracleError("Truncated")
        tensors.append((name, ty, shape, start, end))
    return alignment, kv, tensors
