"""Model files: the GGUF reader of the library (llr_gguf_*) and the loader that turns a Llama-family file into a
device-resident session.

Mirrors the reference's `Gguf` accessors (langtax/src/gguf.rs:534-628: tensor, tensors, kv_u32, kv_f32, kv_bool,
kv_string, kv_i32s, alignment, blob_len) and the step from a tensor's blob range to a matrix the executor owns
(`quant_mat`, `quant_mat_rows`, langtax/src/decode.rs:9612-9713).  Weight bytes go from the mapped file to the device
packed; nothing is dequantized on the host."""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import numpy as np

from . import _lib

from .executor import Executor, Matrix, NativeCudaError, Session, lib

GGUF_ERRORS = {20: "Magic", 21: "Version", 22: "Truncated", 23: "Utf8", 24: "UnsupportedType", 25: "RemovedType",
               26: "UnsupportedKv", 27: "Shape"}


class GgufError(ValueError):
    """GgufError of the reference (gguf.rs:338-370): `kind` is the variant's name, `code` the library's status."""

    def __init__(self, code: int, message: str):
        super().__init__(message)
        self.code, self.kind = code, GGUF_ERRORS.get(code, "Invalid")


@dataclass(frozen=True)
class TensorInfo:
    name: str
    ggml_type: int
    dtype: int          # executor tag, -1 without a kernel
    shape: tuple        # GGUF order: columns first
    start: int
    end: int

    @property
    def n_cols(self) -> int:
        return self.shape[0]

    @property
    def n_rows(self) -> int:
        return self.shape[1] if len(self.shape) > 1 else 1

    @property
    def n_parts(self) -> int:
        return self.shape[2] if len(self.shape) > 2 else 1


def _info(t: _lib.GgufTensor) -> TensorInfo:
    return TensorInfo(C.string_at(t.name, t.name_len).decode(), t.ggml_type, t.dtype, tuple(t.shape[:t.n_dims]), t.start, t.end)


class GgufFile:
    def __init__(self, source):
        """source: a path (mapped read-only) or a bytes-like image (kept alive by this object)."""
        h = C.c_void_p()
        import os
        if isinstance(source, (str, os.PathLike)):
            self._image = None
            rc = lib().llr_gguf_open(os.fsencode(source), C.byref(h))
        else:
            self._image = np.frombuffer(bytes(source), np.uint8)
            rc = lib().llr_gguf_open_bytes(self._image.ctypes.data, self._image.size, C.byref(h))
        self._h = h.value
        if rc != 0:
            msg = lib().llr_gguf_last_error(self._h).decode() if self._h else "invalid argument"
            self.close()
            raise GgufError(rc, msg)

    def close(self) -> None:
        if getattr(self, "_h", None):
            lib().llr_gguf_close(self._h)
            self._h = None

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.close()

    def _check(self, rc: int) -> None:
        if rc != 0:
            raise NativeCudaError(rc, lib().llr_gguf_last_error(self._h).decode() or "GGUF call failed")

    # --- file level -------------------------------------------------------------------------------------------
    def _sizes(self):
        n, a, b = C.c_size_t(), C.c_size_t(), C.c_size_t()
        lib().llr_gguf_info(self._h, C.byref(n), C.byref(a), C.byref(b))
        return n.value, a.value, b.value

    @property
    def alignment(self) -> int:
        return self._sizes()[1]

    @property
    def blob_len(self) -> int:
        return self._sizes()[2]

    def tensors(self) -> list[TensorInfo]:
        out, t = [], _lib.GgufTensor()
        for i in range(self._sizes()[0]):
            lib().llr_gguf_tensor_at(self._h, i, C.byref(t))
            out.append(_info(t))
        return out

    def tensor(self, name: str) -> TensorInfo | None:
        t = _lib.GgufTensor()
        return _info(t) if lib().llr_gguf_find(self._h, name.encode(), C.byref(t)) == 0 else None

    # --- metadata ---------------------------------------------------------------------------------------------
    def kv_u32(self, key: str):
        v = C.c_uint32()
        return v.value if lib().llr_gguf_kv_u32(self._h, key.encode(), C.byref(v)) == 0 else None

    def kv_f32(self, key: str):
        v = C.c_float()
        return v.value if lib().llr_gguf_kv_f32(self._h, key.encode(), C.byref(v)) == 0 else None

    def kv_bool(self, key: str):
        v = C.c_int()
        return bool(v.value) if lib().llr_gguf_kv_bool(self._h, key.encode(), C.byref(v)) == 0 else None

    def kv_string(self, key: str):
        p, n = C.c_char_p(), C.c_size_t()
        if lib().llr_gguf_kv_string(self._h, key.encode(), C.byref(p), C.byref(n)) != 0:
            return None
        return C.string_at(p, n.value).decode()

    def kv_i32s(self, key: str):
        n = C.c_size_t()
        if lib().llr_gguf_kv_i32s(self._h, key.encode(), None, 0, C.byref(n)) != 0:
            return None
        out = np.empty(n.value, np.int32)
        lib().llr_gguf_kv_i32s(self._h, key.encode(), out.ctypes.data, out.size, C.byref(n))
        return out.tolist()

    def kv_bits(self, key: str):
        """(raw 64-bit pattern, gguf value type) of any scalar value, or None."""
        b, t = C.c_uint64(), C.c_int()
        if lib().llr_gguf_kv_bits(self._h, key.encode(), C.byref(b), C.byref(t)) != 0:
            return None
        return b.value, t.value

    def kv_type(self, key: str):
        """(gguf value type, element type of an array or -1, item count) or None."""
        t, e, n = C.c_int(), C.c_int(), C.c_size_t()
        if lib().llr_gguf_kv_type(self._h, key.encode(), C.byref(t), C.byref(e), C.byref(n)) != 0:
            return None
        return t.value, e.value, n.value

    # --- weights ----------------------------------------------------------------------------------------------
    def upload(self, ex: Executor, name: str, part: int = 0, first_row: int = 0, n_rows: int = 0) -> Matrix:
        h = C.c_void_p()
        self._check(lib().llr_gguf_upload(ex._h, self._h, name.encode(), part, first_row, n_rows, C.byref(h)))
        return Matrix(ex, h.value)

    def matmul(self, ex: Executor, name: str, tokens: int, x, y: np.ndarray, part: int = 0, first_row: int = 0,
               n_rows: int = 0) -> None:
        xv = np.ascontiguousarray(x, np.float32).reshape(-1)
        rc = lib().llr_gguf_matmul(ex._h, self._h, name.encode(), part, first_row, n_rows, tokens, xv.ctypes.data, xv.size,
                                   y.ctypes.data, y.size)
        if rc != 0:
            msg = lib().llr_gguf_last_error(self._h).decode()
            ex._check(rc) if not msg else self._check(rc)

    def key(self, name: str, part: int = 0, first_row: int = 0, n_rows: int = 0) -> tuple[int, int]:
        hi, lo = C.c_uint64(), C.c_uint64()
        self._check(lib().llr_gguf_key(self._h, name.encode(), part, first_row, n_rows, C.byref(hi), C.byref(lo)))
        return hi.value, lo.value

    def f32s(self, name: str) -> np.ndarray:
        """A small F32 tensor (norm weights) read on the host (`f32s`, decode.rs)."""
        t = self.tensor(name)
        if t is None or t.ggml_type != 0:
            raise KeyError(name)
        return self.read(t.start, t.end).view(np.float32)

    def read(self, start: int, end: int) -> np.ndarray:
        out = np.empty(end - start, np.uint8)
        self._check(lib().llr_gguf_read(self._h, start, out.size, out.ctypes.data))
        return out


def llama_config(g: GgufFile, n_ctx: int | None = None) -> dict:
    """The hyper-parameters the walk needs, from `<arch>.*` metadata (decode.rs:1905-1930, 7461-7515)."""
    arch = g.kv_string("general.architecture") or "llama"

    def need(key):
        v = g.kv_u32(f"{arch}.{key}")
        if v is None or v == 0:
            raise GgufError(27, f"{arch}.{key}")
        return v
    n_embd, n_head = need("embedding_length"), need("attention.head_count")
    n_head_kv = g.kv_u32(f"{arch}.attention.head_count_kv") or n_head
    head_dim = g.kv_u32(f"{arch}.rope.dimension_count") or n_embd // n_head
    emb = g.tensor("token_embd.weight")
    if emb is None:
        raise KeyError("token_embd.weight")
    cfg = dict(n_layer=need("block_count"), n_embd=n_embd, n_head=n_head, n_head_kv=n_head_kv, head_dim=head_dim,
               n_ff=need("feed_forward_length"), n_vocab=emb.n_rows,
               n_ctx=n_ctx or g.kv_u32(f"{arch}.context_length") or 2048,
               rms_eps=g.kv_f32(f"{arch}.attention.layer_norm_rms_epsilon") or 1e-5,
               rope_base=g.kv_f32(f"{arch}.rope.freq_base") or 10000.0)
    n_expert = g.kv_u32(f"{arch}.expert_count") or 0
    if n_expert:  # architecture=llama with routed experts (llama.expert_count / llama.expert_used_count)
        n_used = g.kv_u32(f"{arch}.expert_used_count") or 0
        if not 0 < n_used <= n_expert:
            raise GgufError(27, f"{arch}.expert_used_count")
        cfg.update(n_expert=n_expert, n_expert_used=n_used)
    return cfg


def load_llama(ex: Executor, g: GgufFile, n_ctx: int | None = None, **session_args) -> Session:
    """Uploads every weight of a Llama-family file (dense, or with routed experts) packed and returns the device-resident session.  `output.weight`
    falls back to the token embedding when the file ties them (decode.rs:2069-2072)."""
    cfg = llama_config(g, n_ctx)
    token_embd = g.upload(ex, "token_embd.weight")
    output = g.upload(ex, "output.weight") if g.tensor("output.weight") is not None else None
    layers = []
    n_expert = cfg.get("n_expert", 0)
    for i in range(cfg["n_layer"]):
        L = {k: g.upload(ex, f"blk.{i}.{k}.weight") for k in ("attn_q", "attn_k", "attn_v", "attn_output")}
        if n_expert and g.tensor(f"blk.{i}.ffn_gate_inp.weight") is not None:
            # routed experts: the router and one resident matrix per expert part of the 3-D *_exps tensors
            L["ffn_gate_inp"] = g.upload(ex, f"blk.{i}.ffn_gate_inp.weight")
            L["n_expert_used"] = cfg["n_expert_used"]
            for k in ("ffn_gate_exps", "ffn_up_exps", "ffn_down_exps"):
                L[k] = [g.upload(ex, f"blk.{i}.{k}.weight", part=e) for e in range(n_expert)]
        else:
            L.update({k: g.upload(ex, f"blk.{i}.{k}.weight") for k in ("ffn_gate", "ffn_up", "ffn_down")})
        L["attn_norm"] = g.f32s(f"blk.{i}.attn_norm.weight")
        L["ffn_norm"] = g.f32s(f"blk.{i}.ffn_norm.weight")
        layers.append(L)
    s = Session(ex, cfg, token_embd, layers, output, g.f32s("output_norm.weight"), **session_args)
    s.weights = (token_embd, output, layers)  # keeps the matrices alive as long as the session
    return s
