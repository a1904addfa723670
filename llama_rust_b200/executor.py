"""Host-side mirror of the reference's executor types over the C ABI.

``Executor`` stands where ``llama_native_cuda::CudaGemv`` stands in the
reference (native-cuda/src/gpu.rs:139-418) and ``Matrix`` where ``CudaMatrix``
does (gpu.rs:126-130); method names, argument meaning and error behaviour follow
them, except that ``upload`` takes GGUF packed bytes and a dtype tag instead of
F32-expanded weights.  Errors surface as ``NativeCudaError`` carrying the status
code and the executor's message (the reference's ``Result<_, String>``).
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _lib

F16, BF16, F32, Q5_0, Q5_1, Q4_0, Q8_0, Q4_K, Q6_K = 0, 1, 2, 6, 7, 12, 13, 17, 19
Q4_1, Q5_K = 5, 18
DTYPES = {"F16": F16, "BF16": BF16, "F32": F32, "Q5_0": Q5_0, "Q5_1": Q5_1, "Q4_0": Q4_0,
          "Q8_0": Q8_0, "Q4_K": Q4_K, "Q6_K": Q6_K, "Q4_1": Q4_1, "Q5_K": Q5_K}
OK, ERR_INVALID, ERR_UNALIGNED, ERR_DTYPE, ERR_OVERFLOW, ERR_FOREIGN, ERR_CUDA, ERR_OOM, ERR_CONFIG = range(9)
PATH_AUTO, PATH_GENERIC, PATH_STAGED, PATH_MMA, PATH_TC = 0, 1, 2, 3, 4
XOP_NONE, XOP_RMSNORM, XOP_SWIGLU = 0, 1, 2

_cdll = None


def lib() -> C.CDLL:
    global _cdll
    if _cdll is None:
        _cdll = _lib.load()
    return _cdll


class NativeCudaError(Exception):
    """A failing executor call: ``code`` is the LLR_ERR_* status, ``args[0]`` the message."""

    def __init__(self, code: int, message: str):
        super().__init__(message)
        self.code = code


def row_bytes(dtype: int, cols: int) -> int:
    out = C.c_size_t(0)
    rc = lib().llr_row_bytes(dtype, cols, C.byref(out))
    if rc:
        raise NativeCudaError(rc, f"row_bytes(dtype={dtype}, cols={cols}) failed with status {rc}")
    return out.value


def _as_u8(a) -> np.ndarray:
    if isinstance(a, (bytes, bytearray, memoryview)):
        return np.frombuffer(a, dtype=np.uint8)
    return np.ascontiguousarray(a).view(np.uint8).reshape(-1)


def _as_f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32).reshape(-1)


class Matrix:
    """Immutable packed matrix resident on the device (CudaMatrix, gpu.rs:126)."""

    def __init__(self, executor: "Executor", handle: int):
        self._exec = executor
        self._h = handle
        dt, r, c, b = C.c_uint8(), C.c_size_t(), C.c_size_t(), C.c_size_t()
        lib().llr_matrix_info(handle, C.byref(dt), C.byref(r), C.byref(c), C.byref(b))
        self.dtype, self.rows, self.cols, self.packed_bytes = dt.value, r.value, c.value, b.value

    def free(self) -> None:
        if self._h:
            lib().llr_matrix_free(self._h)
            self._h = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


class Program:
    """A fixed list of decode products run by one persistent launch (llr_program_*)."""

    def __init__(self, executor: "Executor", handle: int, n_entries: int):
        self._exec, self._h, self.n_entries = executor, handle, n_entries

    def run(self, stream: int = 0) -> None:
        self._exec._check(lib().llr_program_run(self._exec._h, self._h, stream))

    def info(self) -> dict:
        """entries, phases, and how many phases synchronise through a counter instead of tagged results."""
        a, b, c, d = C.c_uint32(), C.c_uint32(), C.c_uint32(), C.c_uint32()
        self._exec._check(lib().llr_program_info(self._h, C.byref(a), C.byref(b), C.byref(c), C.byref(d)))
        return {"entries": a.value, "phases": b.value, "counter_phases": c.value, "ctas": d.value}

    def free(self) -> None:
        if self._h:
            lib().llr_program_free(self._h)
            self._h = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


class Session:
    """The device-resident Llama walk (llr_session_*): stands where the reference's ``Session`` stands
    (prefill / decode), with the element-wise steps, the KV cache and the greedy argmax on the device."""

    def __init__(self, executor: "Executor", cfg: dict, token_embd: Matrix, layers, output: Matrix | None = None,
                 output_norm=None, n_seq: int = 1, kv_blocks: int = 0, block_tokens: int = 16):
        """cfg: n_layer, n_embd, n_head, n_head_kv, head_dim, n_ff, n_vocab, n_ctx (+ rms_eps, rope_base);
        layers: per layer a dict attn_q, attn_k, attn_v, attn_output, ffn_gate, ffn_up, ffn_down (Matrix) and
        optionally attn_norm, ffn_norm (float32 arrays of n_embd; absent: all ones).  A layer with routed experts
        (architecture=llama, n_expert > 0) has ffn_gate_inp (Matrix, n_expert x n_embd), ffn_gate_exps, ffn_up_exps,
        ffn_down_exps (lists of n_expert matrices) and n_expert_used instead of ffn_gate, ffn_up, ffn_down."""
        self._exec = executor
        self._keep = []  # host arrays the C call reads during creation
        c = _lib.LlamaConfig(*(int(cfg[k]) for k in ("n_layer", "n_embd", "n_head", "n_head_kv", "head_dim", "n_ff",
                                                     "n_vocab", "n_ctx")),
                             float(cfg.get("rms_eps", 1e-5)), float(cfg.get("rope_base", 10000.0)))
        arr = (_lib.LlamaLayer * len(layers))()

        def norm(v):
            if v is None:
                return None
            a = np.ascontiguousarray(v, np.float32)
            self._keep.append(a)
            return a.ctypes.data
        for i, L in enumerate(layers):
            dense = [L[k]._h if L.get(k) is not None else None for k in ("attn_q", "attn_k", "attn_v", "attn_output", "ffn_gate",
                                                                          "ffn_up", "ffn_down")]
            arr[i] = _lib.LlamaLayer(*dense, norm(L.get("attn_norm")), norm(L.get("ffn_norm")))
            if L.get("ffn_gate_inp") is not None:
                n_expert = len(L["ffn_gate_exps"])
                exps = [(C.c_void_p * n_expert)(*[m._h for m in L[k]]) for k in ("ffn_gate_exps", "ffn_up_exps", "ffn_down_exps")]
                self._keep.extend(exps)
                arr[i].n_expert, arr[i].n_expert_used, arr[i].ffn_gate_inp = n_expert, int(L["n_expert_used"]), L["ffn_gate_inp"]._h
                arr[i].ffn_gate_exps, arr[i].ffn_up_exps, arr[i].ffn_down_exps = exps
        model = _lib.LlamaModel(c, token_embd._h, output._h if output is not None else None, norm(output_norm), arr)
        h = C.c_void_p()
        executor._check(lib().llr_session_create_paged(executor._h, C.byref(model), n_seq, kv_blocks, block_tokens, C.byref(h)))
        self._h = h.value
        self.n_seq = n_seq
        self.n_vocab = int(cfg["n_vocab"])
        self._keep = []
        self._model = (token_embd, output, layers)  # the device reads these matrices for as long as the session lives
        self._ids = [[] for _ in range(n_seq)]  # token ids whose keys and values each sequence's cache holds

    def prefill(self, tokens, want_logits: bool = False):
        t = np.ascontiguousarray(tokens, np.int32)
        out = np.empty(self.n_vocab, np.float32) if want_logits else None
        self._exec._check(lib().llr_session_prefill(self._h, t.ctypes.data, t.size, out.ctypes.data if want_logits else None))
        self._ids[0].extend(int(v) for v in t)
        return out

    def decode(self, n_gen: int):
        """Greedy tokens and each step's top-2 logit margin."""
        ids = np.empty(n_gen, np.int32)
        margin = np.empty(n_gen, np.float32)
        self._exec._check(lib().llr_session_decode(self._h, n_gen, ids.ctypes.data, margin.ctypes.data))
        self._ids[0].extend(int(v) for v in ids)
        return ids, margin

    def batch(self, groups, want_logits: bool = False):
        """groups: list of (sequence index, token ids): one ragged batch over several sequences (llr_session_batch).
        Returns (next_ids[n_groups], logits[n_groups, n_vocab] or None), in the order of `groups`."""
        seqs = np.array([g[0] for g in groups], np.uint32)
        counts = np.array([len(g[1]) for g in groups], np.uint32)
        toks = np.ascontiguousarray(np.concatenate([np.asarray(g[1], np.int32) for g in groups]), np.int32)
        nxt = np.empty(len(groups), np.int32)
        lg = np.empty((len(groups), self.n_vocab), np.float32) if want_logits else None
        self._exec._check(lib().llr_session_batch(self._h, len(groups), seqs.ctypes.data, counts.ctypes.data, toks.ctypes.data,
                                                  lg.ctypes.data if want_logits else None, nxt.ctypes.data))
        for q, t in groups:
            self._ids[q].extend(int(v) for v in t)
        return nxt, lg

    def cached_ids(self, seq: int = 0) -> list:
        return list(self._ids[seq])

    def seq_truncate(self, seq: int, n_keep: int) -> None:
        self._exec._check(lib().llr_session_seq_truncate(self._h, seq, n_keep))
        del self._ids[seq][n_keep:]

    def prompt_suffix(self, tokens, seq: int = 0, max_suffix: int = 0):
        """KvCache::prompt_suffix (langtax/src/decode.rs:1155-1195): keeps the longest common prefix of `tokens` and the
        cached ids, rewinds the cache to it and returns the tokens still to forward, at most max_suffix of them (0: all).
        When the whole prompt is cached the last token is forwarded again, so that its logits exist."""
        tokens = [int(v) for v in tokens]
        if not tokens:
            raise ValueError("prefill tokens")
        have = self._ids[seq]
        lcp = 0
        while lcp < len(have) and lcp < len(tokens) and have[lcp] == tokens[lcp]:
            lcp += 1
        keep = len(tokens) - 1 if lcp == len(tokens) else lcp
        self.seq_truncate(seq, keep)
        rest = tokens[keep:]
        return rest[:max_suffix] if max_suffix else rest

    def prompt(self, tokens, seq: int = 0):
        """Session::prompt: the logits after `tokens` as a full prompt, re-using what the cache already holds of it."""
        rest = self.prompt_suffix(tokens, seq)
        if self.n_seq == 1 and seq == 0:
            return self.prefill(rest, want_logits=True)
        return self.batch([(seq, rest)], want_logits=True)[1][0]

    def seq_position(self, seq: int) -> int:
        p = C.c_size_t()
        self._exec._check(lib().llr_session_seq_position(self._h, seq, C.byref(p)))
        return p.value

    def seq_reset(self, seq: int) -> None:
        self._exec._check(lib().llr_session_seq_reset(self._h, seq))
        self._ids[seq] = []

    def logits(self) -> np.ndarray:
        out = np.empty(self.n_vocab, np.float32)
        self._exec._check(lib().llr_session_logits(self._h, out.ctypes.data, out.size))
        return out

    @property
    def position(self) -> int:
        p = C.c_size_t()
        lib().llr_session_position(self._h, C.byref(p))
        return p.value

    def reset(self) -> None:
        self._exec._check(lib().llr_session_reset(self._h))
        self._ids = [[] for _ in range(self.n_seq)]

    def free(self) -> None:
        if self._h:
            lib().llr_session_free(self._h)
            self._h = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


MOVE_WEIGHTS, DISPATCH_ACTIVATIONS = 0, 1


def plan_placement(expert_bytes: int, activation_bytes: int, fan_in: int, reuse: int, link_bps: int) -> int:
    """Move an expert's weights once or ship activations on every use (expertvm/src/planner.rs:332-349)."""
    return lib().llr_plan_placement(expert_bytes, activation_bytes, fan_in, reuse, link_bps)


def moe_ep_arena_bytes(n_expert: int, n_used: int, n_embd: int, world: int, max_tokens: int) -> int:
    """Bytes of peer-writable arena one rank of an expert-parallel layer needs (llr_moe_ep_arena_bytes)."""
    n = int(lib().llr_moe_ep_arena_bytes(n_expert, n_used, n_embd, world, max_tokens))
    if n == 0:
        raise ValueError("expert-parallel layer: invalid shape")
    return n


class MoeEp:
    """Handle of llr_moe_ep_*: dispatch -> serve -> combine per run (run() makes the three calls); device pointers."""

    def __init__(self, ex: "Executor", h: int):
        self._ex, self._h = ex, h

    def dispatch(self, tokens: int, x_ptr: int) -> None:
        self._ex._check(lib().llr_moe_ep_dispatch(self._h, tokens, x_ptr))

    def serve(self) -> None:
        self._ex._check(lib().llr_moe_ep_serve(self._h))

    def combine(self, out_ptr: int, ids_ptr: int | None = None, w_ptr: int | None = None) -> None:
        self._ex._check(lib().llr_moe_ep_combine(self._h, out_ptr, ids_ptr, w_ptr))

    def run(self, tokens: int, x_ptr: int, out_ptr: int, ids_ptr: int | None = None, w_ptr: int | None = None) -> None:
        self._ex._check(lib().llr_moe_ep_run(self._h, tokens, x_ptr, out_ptr, ids_ptr, w_ptr))

    def free(self) -> None:
        if self._h:
            lib().llr_moe_ep_free(self._h)
            self._h = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


class Executor:
    """One device, one stream, scratch reuse and weight residency (CudaGemv, gpu.rs:139)."""

    def __init__(self, device: int = 0):
        h = C.c_void_p()
        rc = lib().llr_exec_create(device, C.byref(h))
        if rc:
            raise NativeCudaError(rc, lib().llr_exec_last_error(None).decode())
        self._h = h.value
        self.device = device

    # -- plumbing ---------------------------------------------------------
    def _check(self, rc: int) -> None:
        if rc:
            raise NativeCudaError(rc, lib().llr_exec_last_error(self._h).decode())

    def close(self) -> None:
        if self._h:
            lib().llr_exec_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    # -- CudaGemv surface ---------------------------------------------------
    def memory_info(self) -> tuple[int, int]:
        fr, tot = C.c_size_t(), C.c_size_t()
        self._check(lib().llr_exec_mem_info(self._h, C.byref(fr), C.byref(tot)))
        return fr.value, tot.value

    def upload(self, dtype: int, rows: int, cols: int, packed) -> Matrix:
        w = _as_u8(packed)
        h = C.c_void_p()
        self._check(lib().llr_matrix_upload(self._h, dtype, rows, cols, w.ctypes.data, w.size, C.byref(h)))
        return Matrix(self, h.value)

    def synth(self, dtype: int, rows: int, cols: int, seed: int) -> Matrix:
        h = C.c_void_p()
        self._check(lib().llr_matrix_synth(self._h, dtype, rows, cols, seed & (2 ** 64 - 1), C.byref(h)))
        return Matrix(self, h.value)

    def download(self, m: Matrix) -> np.ndarray:
        out = np.empty(m.packed_bytes, np.uint8)
        self._check(lib().llr_matrix_download(self._h, m._h, out.ctypes.data, out.size))
        return out

    def gemv_resident(self, m: Matrix, x, y: np.ndarray) -> None:
        xv = _as_f32(x)
        self._check(lib().llr_gemv_resident(self._h, m._h, xv.ctypes.data, xv.size, y.ctypes.data, y.size))

    def gemm_resident(self, m: Matrix, tokens: int, x, y: np.ndarray) -> None:
        xv = _as_f32(x)
        self._check(lib().llr_gemm_resident(self._h, m._h, tokens, xv.ctypes.data, xv.size,
                                            y.ctypes.data, y.size))

    def matmul(self, dtype: int, rows: int, cols: int, tokens: int, packed, x, y: np.ndarray) -> None:
        """native_gpu::matmul (langtax/src/native_gpu.rs:124): content-identity residency."""
        w, xv = _as_u8(packed), _as_f32(x)
        assert y.dtype == np.float32 and y.flags.c_contiguous
        self._check(lib().llr_matmul(self._h, dtype, rows, cols, tokens, w.ctypes.data, w.size,
                                     xv.ctypes.data, xv.size, y.ctypes.data, y.size))

    def matmul_keyed(self, key, dtype: int, rows: int, cols: int, tokens: int, packed, x, y: np.ndarray) -> None:
        """matmul for weights with a stable identity: key = (hi, lo), e.g. the blob range of an immutable model file
        (QuantMat.start..end, langtax/src/decode.rs:476-485).  A hit reads nothing but the key."""
        w, xv = _as_u8(packed), _as_f32(x)
        assert y.dtype == np.float32 and y.flags.c_contiguous
        self._check(lib().llr_matmul_keyed(self._h, key[0], key[1], dtype, rows, cols, tokens, w.ctypes.data, w.size,
                                           xv.ctypes.data, xv.size, y.ctypes.data, y.size))

    def pin_key(self, key, pinned: bool = True) -> None:
        """Keeps the keyed matrix out of eviction (pin_hot of the expert store, langtax/src/engine.rs:916-950)."""
        self._check(lib().llr_exec_pin_key(self._h, key[0], key[1], int(pinned)))

    def matmul_device(self, m: Matrix, tokens: int, x_ptr: int, y_ptr: int, stream: int = 0) -> None:
        self._check(lib().llr_matmul_device(self._h, m._h, tokens, x_ptr, y_ptr, stream))

    def program(self, entries) -> Program:
        """entries: iterable of (matrix, x_ptr, y_ptr, tokens, phase); see llr_program_create."""
        entries = list(entries)
        arr = (_lib.ProgramEntry * len(entries))()
        for i, (m, x, y, tokens, phase) in enumerate(entries):
            arr[i] = _lib.ProgramEntry(m._h, x, y, tokens, phase)
        h = C.c_void_p()
        self._check(lib().llr_program_create(self._h, arr, len(entries), C.byref(h)))
        return Program(self, h.value, len(entries))

    def program_ops(self, ops, shard=None) -> Program:
        """ops: iterable of dicts with keys matrix, x, y, tokens, phase and optionally x2, resid, y_ld, x_op, eps
        (llr_program_op).  shard: None, or (arena, arena_bytes, world, rank, peer_arenas) for one rank of a
        row-sharded program."""
        ops = list(ops)
        arr = (_lib.ProgramOp * len(ops))()
        for i, o in enumerate(ops):
            arr[i] = _lib.ProgramOp(o["matrix"]._h, o["x"], o.get("x2") or None, o.get("resid") or None, o["y"],
                                    int(o.get("y_ld", 0)), o["tokens"], o["phase"], int(o.get("x_op", 0)),
                                    float(o.get("eps", 0.0)))
        h = C.c_void_p()
        sh = None
        if shard is not None:
            arena, arena_bytes, world, rank, peer_arenas = shard
            peers = (C.c_void_p * world)(*[int(p) if p else None for p in peer_arenas])
            sh = C.byref(_lib.ProgramShard(arena, arena_bytes, world, rank, peers))
        self._check(lib().llr_program_create_ops(self._h, arr, len(ops), sh, C.byref(h)))
        return Program(self, h.value, len(ops))

    def set_wait_limit(self, polls: int) -> None:
        self._check(lib().llr_exec_set_wait_limit(self._h, polls))

    # -- row-sharded programs across GPUs (llr_shared_*, llr_program_create_sharded) ----
    def shared_alloc(self, nbytes: int) -> tuple[int, bytes]:
        """Zeroed device memory that other processes can open: (device address, 64-byte handle)."""
        dev = C.c_void_p()
        handle = C.create_string_buffer(64)
        self._check(lib().llr_shared_alloc(self._h, nbytes, C.byref(dev), handle))
        return dev.value, handle.raw

    def shared_open(self, handle: bytes) -> int:
        dev = C.c_void_p()
        self._check(lib().llr_shared_open(self._h, handle, C.byref(dev)))
        return dev.value

    def shared_close(self, dev: int) -> None:
        self._check(lib().llr_shared_close(self._h, dev))

    def shared_free(self, dev: int) -> None:
        self._check(lib().llr_shared_free(self._h, dev))

    def sharded_program(self, entries, y_ld, arena: int, arena_bytes: int, world: int, rank: int, peer_arenas) -> Program:
        """entries as for program(); y_ld[i] = full row count of result i; peer_arenas[g] = rank g's arena
        as opened in this process (own slot ignored)."""
        entries = list(entries)
        arr = (_lib.ProgramEntry * len(entries))()
        for i, (m, x, y, tokens, phase) in enumerate(entries):
            arr[i] = _lib.ProgramEntry(m._h, x, y, tokens, phase)
        ld = (C.c_uint64 * len(entries))(*[int(v) for v in y_ld])
        peers = (C.c_void_p * world)(*[int(p) if p else None for p in peer_arenas])
        h = C.c_void_p()
        self._check(lib().llr_program_create_sharded(self._h, arr, ld, len(entries), arena, arena_bytes, world, rank,
                                                     peers, C.byref(h)))
        return Program(self, h.value, len(entries))

    def moe_ffn(self, router: Matrix, gate, up, down, n_used: int, norm_w: bool, x, out=None):
        """One routed-expert FFN layer (llr_moe_ffn).  Returns (out, sel_ids, sel_w); `out` may be a
        caller-owned (e.g. pinned) float32 array of x's shape."""
        n_expert = len(gate)
        arrs = [(C.c_void_p * n_expert)(*[None if m is None else m._h for m in lst]) for lst in (gate, up, down)]  # None: expert resident on another rank
        layer = _lib.MoeLayer(n_expert, n_used, int(norm_w), router._h, arrs[0], arrs[1], arrs[2])
        xs = np.ascontiguousarray(x, np.float32).reshape(-1, router.cols)
        tokens = xs.shape[0]
        out = np.empty_like(xs) if out is None else out
        ids = np.empty((tokens, n_used), np.int32)
        w = np.empty((tokens, n_used), np.float32)
        self._check(lib().llr_moe_ffn(self._h, C.byref(layer), tokens, xs.ctypes.data, xs.size, out.ctypes.data,
                                      out.size, ids.ctypes.data, w.ctypes.data))
        return out, ids, w

    def _moe_layer(self, router, gate, up, down, n_used, norm_w):
        n_expert = len(gate)
        arrs = [(C.c_void_p * n_expert)(*[None if m is None else m._h for m in lst]) for lst in (gate, up, down)]
        return _lib.MoeLayer(n_expert, n_used, int(norm_w), router._h if router is not None else None, arrs[0], arrs[1], arrs[2]), arrs

    def moe_route_device(self, router: Matrix, n_expert: int, n_used: int, norm_w: bool, tokens: int, x_ptr: int, ids_ptr: int,
                         w_ptr: int) -> None:
        """Routing of `tokens` rows at x_ptr on the device (llr_moe_route_device); ids / weights go to device memory."""
        none = [None] * n_expert
        layer, keep = self._moe_layer(router, none, none, none, n_used, norm_w)
        self._check(lib().llr_moe_route_device(self._h, C.byref(layer), tokens, x_ptr, ids_ptr, w_ptr))

    def moe_experts_device(self, gate, up, down, counts, rows_ptr: int, y_ptr: int) -> None:
        """Expert products over packed rows grouped by expert (llr_moe_experts_device); counts[e] rows for expert e."""
        layer, keep = self._moe_layer(None, gate, up, down, 1, False)
        cnt = (C.c_uint32 * len(gate))(*[int(c) for c in counts])
        self._check(lib().llr_moe_experts_device(self._h, C.byref(layer), cnt, rows_ptr, y_ptr))

    def moe_ep(self, router: Matrix, gate, up, down, n_used: int, norm_w: bool, world: int, rank: int, max_tokens: int,
               arena: int, arena_bytes: int, peer_arenas) -> "MoeEp":
        """Expert-parallel layer with the exchange inside the library (llr_moe_ep_create); gate/up/down hold None for
        the experts of other ranks, peer_arenas[g] is rank g's arena as mapped here."""
        layer, keep = self._moe_layer(router, gate, up, down, n_used, norm_w)
        peers = (C.c_void_p * world)(*[None if g == rank else peer_arenas[g] for g in range(world)])
        h = C.c_void_p()
        self._check(lib().llr_moe_ep_create(self._h, C.byref(layer), world, rank, max_tokens, arena, arena_bytes, peers, C.byref(h)))
        return MoeEp(self, h.value)

    def dequant_rows(self, m: Matrix, row0: int = 0, n_rows: int | None = None) -> np.ndarray:
        n = m.rows - row0 if n_rows is None else n_rows
        out = np.empty((n, m.cols), np.float32)
        self._check(lib().llr_dequant_rows(self._h, m._h, row0, n, out.ctypes.data, out.size))
        return out

    def synchronize(self) -> None:
        self._check(lib().llr_exec_synchronize(self._h))

    def set_path(self, path: int) -> None:
        self._check(lib().llr_exec_set_path(self._h, path))

    def counters(self) -> dict:
        c = _lib.Counters()
        lib().llr_exec_counters(self._h, C.byref(c))
        return {n: getattr(c, n) for n, _ in c._fields_}
