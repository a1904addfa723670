"""Builds GGUF v3 images for the tests, laid out as the reference's writer lays them out (langtax/src/gguf.rs:640-712):
header, metadata, tensor table, zero padding to the alignment, then each payload at the next multiple of the alignment
counted from the start of the data section.  The alignment used for the layout is 32 whatever `general.alignment` says,
as in the reference's writer."""
import struct

U8, I8, U16, I16, U32, I32, F32, BOOL, STRING, ARRAY, U64, I64, F64 = range(13)
_FMT = {U8: "<B", I8: "<b", U16: "<H", I16: "<h", U32: "<I", I32: "<i", F32: "<f", U64: "<Q", I64: "<q", F64: "<d"}
GGML = {"F32": 0, "F16": 1, "BF16": 30, "Q4_0": 2, "Q4_1": 3, "Q5_0": 6, "Q5_1": 7, "Q8_0": 8, "Q4_K": 12, "Q5_K": 13, "Q6_K": 14}


def _string(s):
    b = s if isinstance(s, bytes) else s.encode()
    return struct.pack("<Q", len(b)) + b


def _payload(ty, v):
    if ty in _FMT:
        return struct.pack(_FMT[ty], v)
    if ty == BOOL:
        return struct.pack("<B", 1 if v else 0)
    if ty == STRING:
        return _string(v)
    if ty == ARRAY:
        elem, items = v
        return struct.pack("<iQ", elem, len(items)) + b"".join(_payload(elem, i) for i in items)
    raise ValueError(ty)


def write_gguf(kv, tensors, type_ids=None, version=3, magic=b"GGUF", layout_alignment=32):
    """kv: [(key, value type, value)]; tensors: [(name, ggml type id, shape (columns first), payload bytes)]."""
    offsets, off = [], 0
    for _, _, _, data in tensors:
        off = -(-off // layout_alignment) * layout_alignment
        offsets.append(off)
        off += len(data)
    buf = bytearray(magic + struct.pack("<Iqq", version, len(tensors), len(kv)))
    for key, ty, val in kv:
        buf += _string(key) + struct.pack("<i", ty) + _payload(ty, val)
    for i, ((name, ty, shape, _), offset) in enumerate(zip(tensors, offsets)):
        buf += _string(name) + struct.pack("<I", len(shape))
        for d in shape:
            buf += struct.pack("<q", d)
        buf += struct.pack("<iQ", type_ids[i] if type_ids else ty, offset)
    data_start = -(-len(buf) // layout_alignment) * layout_alignment
    buf += bytes(data_start - len(buf))
    for (_, _, _, data), offset in zip(tensors, offsets):
        buf += bytes(data_start + offset - len(buf))
        buf += bytes(data)
    return bytes(buf)


DEFAULT_KV = [("general.alignment", U32, 32), ("general.name", STRING, "llama-rust")]
