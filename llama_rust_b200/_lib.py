"""Loads libllama_rust_b200.so (the C ABI of include/llama_rust_b200.h) through ctypes.

There is no fallback: if the shared library is missing or a symbol is absent,
importing fails with instructions to build it.
"""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libllama_rust_b200.so")

# every symbol include/llama_rust_b200.h declares
SYMBOLS = [
    "llr_exec_create", "llr_exec_destroy", "llr_exec_mem_info", "llr_exec_last_error",
    "llr_exec_counters", "llr_exec_set_path", "llr_row_bytes", "llr_matrix_upload",
    "llr_matrix_upload_device", "llr_matrix_free", "llr_matrix_info", "llr_gemv_resident",
    "llr_gemm_resident", "llr_matmul", "llr_matmul_device", "llr_exec_synchronize",
    "llr_dequant_rows", "llr_matrix_synth", "llr_matrix_download", "llr_program_create",
    "llr_program_run", "llr_program_free", "llr_gemm_device_noalloc", "llr_moe_ffn",
    "llr_shared_alloc", "llr_shared_open", "llr_shared_close", "llr_shared_free",
    "llr_program_create_sharded", "llr_program_create_ops", "llr_program_info", "llr_exec_set_wait_limit",
    "llr_session_create", "llr_session_prefill", "llr_session_decode", "llr_session_logits", "llr_session_position",
    "llr_session_reset", "llr_session_free", "llr_session_create_paged", "llr_session_batch", "llr_session_seq_position",
    "llr_session_seq_reset", "llr_session_seq_truncate", "llr_moe_route_device", "llr_moe_experts_device", "llr_matmul_keyed",
    "llr_exec_pin_key", "llr_plan_placement", "llr_gguf_open", "llr_gguf_open_bytes", "llr_gguf_close",
    "llr_gguf_last_error", "llr_gguf_info", "llr_gguf_tensor_at", "llr_gguf_find", "llr_gguf_read", "llr_gguf_kv_u32",
    "llr_gguf_kv_f32", "llr_gguf_kv_bits", "llr_gguf_kv_bool", "llr_gguf_kv_string", "llr_gguf_kv_i32s", "llr_gguf_kv_type",
    "llr_gguf_upload", "llr_gguf_matmul", "llr_gguf_key", "llr_moe_ep_arena_bytes", "llr_moe_ep_create", "llr_moe_ep_dispatch",
    "llr_moe_ep_serve", "llr_moe_ep_combine", "llr_moe_ep_run", "llr_moe_ep_free",
]
ARENA_HEADER_BYTES = 65536


class Counters(C.Structure):
    _fields_ = [(n, C.c_uint64) for n in (
        "launches", "uploads", "upload_bytes", "resident_bytes", "cache_limit", "cache_hits",
        "cache_misses", "evictions", "h2d_bytes", "d2h_bytes")]


class GgufTensor(C.Structure):
    _fields_ = [("name", C.c_void_p), ("ggml_type", C.c_int32), ("dtype", C.c_int32), ("n_dims", C.c_uint32),
                ("shape", C.c_uint64 * 4), ("start", C.c_uint64), ("end", C.c_uint64), ("name_len", C.c_uint64)]


class ProgramEntry(C.Structure):
    _fields_ = [("matrix", C.c_void_p), ("x_dev", C.c_void_p), ("y_dev", C.c_void_p),
                ("tokens", C.c_uint32), ("phase", C.c_uint32)]


class ProgramOp(C.Structure):
    _fields_ = [("matrix", C.c_void_p), ("x_dev", C.c_void_p), ("x2_dev", C.c_void_p), ("resid_dev", C.c_void_p),
                ("y_dev", C.c_void_p), ("y_ld", C.c_uint64), ("tokens", C.c_uint32), ("phase", C.c_uint32),
                ("x_op", C.c_uint32), ("eps", C.c_float)]


class ProgramShard(C.Structure):
    _fields_ = [("arena", C.c_void_p), ("arena_bytes", C.c_size_t), ("world", C.c_uint32), ("rank", C.c_uint32),
                ("peer_arenas", C.POINTER(C.c_void_p))]


class LlamaConfig(C.Structure):
    _fields_ = [(n, C.c_uint32) for n in ("n_layer", "n_embd", "n_head", "n_head_kv", "head_dim", "n_ff", "n_vocab", "n_ctx")] + \
               [("rms_eps", C.c_float), ("rope_base", C.c_float)]


class LlamaLayer(C.Structure):
    _fields_ = [(n, C.c_void_p) for n in ("attn_q", "attn_k", "attn_v", "attn_output", "ffn_gate", "ffn_up", "ffn_down",
                                          "attn_norm", "ffn_norm")] + \
               [("n_expert", C.c_uint32), ("n_expert_used", C.c_uint32), ("ffn_gate_inp", C.c_void_p),
                ("ffn_gate_exps", C.POINTER(C.c_void_p)), ("ffn_up_exps", C.POINTER(C.c_void_p)),
                ("ffn_down_exps", C.POINTER(C.c_void_p))]


class LlamaModel(C.Structure):
    _fields_ = [("cfg", LlamaConfig), ("token_embd", C.c_void_p), ("output", C.c_void_p), ("output_norm", C.c_void_p),
                ("layers", C.POINTER(LlamaLayer))]


class MoeLayer(C.Structure):
    _fields_ = [("n_expert", C.c_uint32), ("n_used", C.c_uint32), ("norm_w", C.c_uint32),
                ("router", C.c_void_p), ("gate", C.POINTER(C.c_void_p)), ("up", C.POINTER(C.c_void_p)),
                ("down", C.POINTER(C.c_void_p))]


def load() -> C.CDLL:
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m llama_rust_b200.build` "
            "(needs nvcc; there is no CPU fallback)")
    lib = C.CDLL(LIB_PATH)
    missing = [s for s in SYMBOLS if not hasattr(lib, s)]
    if missing:
        raise ImportError(f"{LIB_PATH} lacks symbols {missing}; rebuild it")
    vp, sz, u8 = C.c_void_p, C.c_size_t, C.c_uint8
    lib.llr_exec_create.argtypes = [C.c_int, C.POINTER(vp)]
    lib.llr_exec_destroy.argtypes = [vp]
    lib.llr_exec_mem_info.argtypes = [vp, C.POINTER(sz), C.POINTER(sz)]
    lib.llr_exec_last_error.argtypes = [vp]
    lib.llr_exec_last_error.restype = C.c_char_p
    lib.llr_exec_counters.argtypes = [vp, C.POINTER(Counters)]
    lib.llr_exec_set_path.argtypes = [vp, C.c_int]
    lib.llr_row_bytes.argtypes = [u8, sz, C.POINTER(sz)]
    lib.llr_matrix_upload.argtypes = [vp, u8, sz, sz, vp, sz, C.POINTER(vp)]
    lib.llr_matrix_upload_device.argtypes = [vp, u8, sz, sz, vp, sz, C.POINTER(vp)]
    lib.llr_matrix_free.argtypes = [vp]
    lib.llr_matrix_info.argtypes = [vp, C.POINTER(u8), C.POINTER(sz), C.POINTER(sz), C.POINTER(sz)]
    lib.llr_gemv_resident.argtypes = [vp, vp, vp, sz, vp, sz]
    lib.llr_gemm_resident.argtypes = [vp, vp, sz, vp, sz, vp, sz]
    lib.llr_matmul.argtypes = [vp, u8, sz, sz, sz, vp, sz, vp, sz, vp, sz]
    lib.llr_matmul_device.argtypes = [vp, vp, sz, vp, vp, vp]
    u64 = C.c_uint64
    lib.llr_matmul_keyed.argtypes = [vp, u64, u64, u8, sz, sz, sz, vp, sz, vp, sz, vp, sz]
    lib.llr_exec_pin_key.argtypes = [vp, u64, u64, C.c_int]
    lib.llr_plan_placement.argtypes = [u64, u64, u64, u64, u64]
    cp = C.c_char_p
    lib.llr_gguf_open.argtypes = [cp, C.POINTER(vp)]
    lib.llr_gguf_open_bytes.argtypes = [vp, sz, C.POINTER(vp)]
    lib.llr_gguf_close.argtypes = [vp]
    lib.llr_gguf_last_error.argtypes = [vp]
    lib.llr_gguf_info.argtypes = [vp, C.POINTER(sz), C.POINTER(sz), C.POINTER(sz)]
    lib.llr_gguf_tensor_at.argtypes = [vp, sz, C.POINTER(GgufTensor)]
    lib.llr_gguf_find.argtypes = [vp, cp, C.POINTER(GgufTensor)]
    lib.llr_gguf_read.argtypes = [vp, u64, sz, vp]
    lib.llr_gguf_kv_u32.argtypes = [vp, cp, C.POINTER(C.c_uint32)]
    lib.llr_gguf_kv_f32.argtypes = [vp, cp, C.POINTER(C.c_float)]
    lib.llr_gguf_kv_bits.argtypes = [vp, cp, C.POINTER(u64), C.POINTER(C.c_int)]
    lib.llr_gguf_kv_bool.argtypes = [vp, cp, C.POINTER(C.c_int)]
    lib.llr_gguf_kv_string.argtypes = [vp, cp, C.POINTER(cp), C.POINTER(sz)]
    lib.llr_gguf_kv_i32s.argtypes = [vp, cp, vp, sz, C.POINTER(sz)]
    lib.llr_gguf_kv_type.argtypes = [vp, cp, C.POINTER(C.c_int), C.POINTER(C.c_int), C.POINTER(sz)]
    lib.llr_gguf_upload.argtypes = [vp, vp, cp, sz, sz, sz, C.POINTER(vp)]
    lib.llr_gguf_matmul.argtypes = [vp, vp, cp, sz, sz, sz, sz, vp, sz, vp, sz]
    lib.llr_gguf_key.argtypes = [vp, cp, sz, sz, sz, C.POINTER(u64), C.POINTER(u64)]
    lib.llr_exec_synchronize.argtypes = [vp]
    lib.llr_dequant_rows.argtypes = [vp, vp, sz, sz, vp, sz]
    lib.llr_matrix_synth.argtypes = [vp, u8, sz, sz, C.c_uint64, C.POINTER(vp)]
    lib.llr_matrix_download.argtypes = [vp, vp, vp, sz]
    lib.llr_program_create.argtypes = [vp, C.POINTER(ProgramEntry), sz, C.POINTER(vp)]
    lib.llr_program_run.argtypes = [vp, vp, vp]
    lib.llr_program_free.argtypes = [vp]
    lib.llr_gemm_device_noalloc.argtypes = [vp, vp, sz, vp, vp, vp]
    lib.llr_moe_ffn.argtypes = [vp, C.POINTER(MoeLayer), sz, vp, sz, vp, sz, vp, vp]
    lib.llr_shared_alloc.argtypes = [vp, sz, C.POINTER(vp), C.c_char_p]
    lib.llr_shared_open.argtypes = [vp, C.c_char_p, C.POINTER(vp)]
    lib.llr_shared_close.argtypes = [vp, vp]
    lib.llr_shared_free.argtypes = [vp, vp]
    lib.llr_program_create_sharded.argtypes = [vp, C.POINTER(ProgramEntry), C.POINTER(C.c_uint64), sz, vp, sz,
                                               C.c_uint32, C.c_uint32, C.POINTER(vp), C.POINTER(vp)]
    lib.llr_program_create_ops.argtypes = [vp, C.POINTER(ProgramOp), sz, C.POINTER(ProgramShard), C.POINTER(vp)]
    lib.llr_program_info.argtypes = [vp, C.POINTER(C.c_uint32), C.POINTER(C.c_uint32), C.POINTER(C.c_uint32), C.POINTER(C.c_uint32)]
    lib.llr_exec_set_wait_limit.argtypes = [vp, C.c_uint32]
    lib.llr_moe_route_device.argtypes = [vp, C.POINTER(MoeLayer), sz, vp, vp, vp]
    lib.llr_moe_experts_device.argtypes = [vp, C.POINTER(MoeLayer), C.POINTER(C.c_uint32), vp, vp]
    lib.llr_moe_ep_arena_bytes.argtypes = [C.c_uint32, C.c_uint32, sz, C.c_uint32, sz]
    lib.llr_moe_ep_arena_bytes.restype = sz
    lib.llr_moe_ep_create.argtypes = [vp, C.POINTER(MoeLayer), C.c_uint32, C.c_uint32, sz, vp, sz, C.POINTER(vp), C.POINTER(vp)]
    lib.llr_moe_ep_dispatch.argtypes = [vp, sz, vp]
    lib.llr_moe_ep_serve.argtypes = [vp]
    lib.llr_moe_ep_combine.argtypes = [vp, vp, vp, vp]
    lib.llr_moe_ep_run.argtypes = [vp, sz, vp, vp, vp, vp]
    lib.llr_moe_ep_free.argtypes = [vp]
    lib.llr_session_create.argtypes = [vp, C.POINTER(LlamaModel), C.POINTER(vp)]
    lib.llr_session_create_paged.argtypes = [vp, C.POINTER(LlamaModel), sz, sz, sz, C.POINTER(vp)]
    lib.llr_session_batch.argtypes = [vp, sz, vp, vp, vp, vp, vp]
    lib.llr_session_seq_position.argtypes = [vp, sz, C.POINTER(sz)]
    lib.llr_session_seq_reset.argtypes = [vp, sz]
    lib.llr_session_seq_truncate.argtypes = [vp, sz, sz]
    lib.llr_session_prefill.argtypes = [vp, vp, sz, vp]
    lib.llr_session_decode.argtypes = [vp, sz, vp, vp]
    lib.llr_session_logits.argtypes = [vp, vp, sz]
    lib.llr_session_position.argtypes = [vp, C.POINTER(sz)]
    lib.llr_session_reset.argtypes = [vp]
    lib.llr_session_free.argtypes = [vp]
    for s in SYMBOLS:
        if s not in ("llr_exec_last_error", "llr_gguf_last_error", "llr_gguf_close"):
            getattr(lib, s).restype = C.c_int
    lib.llr_gguf_last_error.restype = C.c_char_p
    lib.llr_gguf_close.restype = None
    return lib
