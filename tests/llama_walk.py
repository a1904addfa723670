"""Test harness for benchmark config 3: the dense Llama walk of the reference (host code in the
oracle, langtax/src/decode.rs:2710-3097) driven either by the oracle's CPU matrix products or,
through callbacks, by the CUDA executor.  The host ops are literally the same code in both
runs, so any difference in tokens or logits comes from the matrix products alone."""
import ctypes as C

import numpy as np

from oracle import pyoracle as orc

Q4_K, Q6_K = 17, 19
LAYER_TENSORS = [("attn_q", Q4_K), ("attn_k", Q4_K), ("attn_v", Q6_K), ("attn_output", Q4_K),
                 ("ffn_gate", Q4_K), ("ffn_up", Q4_K), ("ffn_down", Q6_K)]  # Q4_K_M-style mix


class Cfg(C.Structure):
    _fields_ = [(n, C.c_int32) for n in ("n_layer", "n_embd", "n_head", "n_head_kv", "head_dim", "n_ff", "n_vocab", "n_ctx")] + \
               [("rms_eps", C.c_float), ("rope_base", C.c_float)]


MATMUL_CB = C.CFUNCTYPE(C.c_int, C.c_void_p, C.c_int, C.c_int64, C.c_void_p, C.c_void_p)
EMBD_CB = C.CFUNCTYPE(C.c_int, C.c_void_p, C.c_int32, C.c_void_p)
orc.lib.orc_llama_generate.argtypes = [C.POINTER(Cfg), C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int,
                                       C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_void_p,
                                       C.c_void_p, C.c_void_p, C.c_int]

class MoeCfg(C.Structure):
    _fields_ = [(n, C.c_int32) for n in ("n_expert", "n_used", "router_kind", "expert_kind")] + \
               [(n, C.c_void_p) for n in ("router", "gate", "up", "down")]


orc.lib.orc_llama_generate_moe.argtypes = [C.POINTER(Cfg), C.POINTER(MoeCfg)] + orc.lib.orc_llama_generate.argtypes[1:]

LLAMA3_8B = dict(n_layer=32, n_embd=4096, n_head=32, n_head_kv=8, head_dim=128, n_ff=14336, n_vocab=128256)


def tensor_list(cfg):
    """(name, dtype, rows, cols) in tensor-id order, then output; token_embd is separate."""
    E, QW, KVW, FF = cfg["n_embd"], cfg["n_head"] * cfg["head_dim"], cfg["n_head_kv"] * cfg["head_dim"], cfg["n_ff"]
    shapes = {"attn_q": (QW, E), "attn_k": (KVW, E), "attn_v": (KVW, E), "attn_output": (E, QW),
              "ffn_gate": (FF, E), "ffn_up": (FF, E), "ffn_down": (E, FF)}
    out = []
    for layer in range(cfg["n_layer"]):
        for name, dt in LAYER_TENSORS:
            out.append((f"blk.{layer}.{name}.weight", dt, *shapes[name]))
    out.append(("output.weight", Q6_K, cfg["n_vocab"], E))
    return out


def make_cfg(cfg, n_ctx):
    return Cfg(cfg["n_layer"], cfg["n_embd"], cfg["n_head"], cfg["n_head_kv"], cfg["head_dim"], cfg["n_ff"],
               cfg["n_vocab"], n_ctx, 1e-5, 10000.0)  # decode.rs:1958, :2053 defaults


def prompt_ids(n, vocab, seed):
    from llama_rust_b200 import synth
    return (synth.words(seed, 0, n) % np.uint64(vocab)).astype(np.int32)


def _generate(c, cb, tensors_ptr, kinds_ptr, embd_kind, embd_ptr, embd_cb, prompt, n_gen, threads, want_logits, moe=None):
    ids = np.zeros(n_gen, np.int32)
    margin = np.zeros(n_gen, np.float32)
    logits = np.zeros(c.n_vocab, np.float32) if want_logits else None
    p = np.ascontiguousarray(prompt, np.int32)
    rc = orc.lib.orc_llama_generate_moe(C.byref(c), C.byref(moe) if moe is not None else None, cb, None, tensors_ptr, kinds_ptr,
                                        embd_kind, embd_ptr, embd_cb, p.ctypes.data, p.size, n_gen, ids.ctypes.data,
                                        margin.ctypes.data, logits.ctypes.data if want_logits else None, threads)
    if rc:
        raise RuntimeError(f"walk failed with status {rc}")
    return ids, margin, logits


def run_cpu(cfg, n_ctx, weights, embd, prompt, n_gen, threads=0, want_logits=False, kinds=None, embd_kind=Q4_K, moe=None):
    """weights: packed numpy arrays in tensor_list order; embd: packed token_embd (Q4_K unless embd_kind says otherwise);
    kinds: dtype of each tensor when it is not tensor_list's mix.  moe (architecture=llama with routed experts): a dict
    n_used, router_kind, expert_kind, router[layer], gate / up / down[layer][expert] of packed arrays; the ffn entries of
    `weights` are then not read and may be None."""
    c = make_cfg(cfg, n_ctx)
    tl = tensor_list(cfg)
    ptrs = (C.c_void_p * len(tl))(*[None if w is None else w.ctypes.data for w in weights])
    kinds = (C.c_int * len(tl))(*(kinds if kinds is not None else [t[1] for t in tl]))
    m = None
    if moe is not None:
        n_expert = len(moe["gate"][0])
        flat = {k: (C.c_void_p * (cfg["n_layer"] * n_expert))(*[a.ctypes.data for per_layer in moe[k] for a in per_layer])
                for k in ("gate", "up", "down")}
        router = (C.c_void_p * cfg["n_layer"])(*[a.ctypes.data for a in moe["router"]])
        m = MoeCfg(n_expert, moe["n_used"], moe["router_kind"], moe["expert_kind"], C.cast(router, C.c_void_p),
                   C.cast(flat["gate"], C.c_void_p), C.cast(flat["up"], C.c_void_p), C.cast(flat["down"], C.c_void_p))
        m._keep = (flat, router)
    return _generate(c, None, ptrs, kinds, embd_kind, embd.ctypes.data, None, prompt, n_gen, threads, want_logits, moe=m)


def run_gpu(cfg, n_ctx, ex, mats, embd_mat, prompt, n_gen, want_logits=False):
    """mats: resident matrices in tensor_list order; every product goes through llr_gemm_resident."""
    from llama_rust_b200.executor import lib
    L = lib()
    c = make_cfg(cfg, n_ctx)
    tl = tensor_list(cfg)
    errors = []

    def matmul(user, tid, n, x, y):
        _, _, rows, cols = tl[tid]
        rc = L.llr_gemm_resident(ex._h, mats[tid]._h, n, x, n * cols, y, n * rows)
        if rc:
            errors.append(L.llr_exec_last_error(ex._h).decode())
        return rc

    def embd(user, token, row):
        rc = L.llr_dequant_rows(ex._h, embd_mat._h, token, 1, row, cfg["n_embd"])
        if rc:
            errors.append(L.llr_exec_last_error(ex._h).decode())
        return rc

    cb, ecb = MATMUL_CB(matmul), EMBD_CB(embd)
    try:
        return _generate(c, cb, None, None, Q4_K, None, ecb, prompt, n_gen, 1, want_logits)
    except RuntimeError as e:
        raise RuntimeError(f"{e}: {errors[:1]}")


def center_q4k(packed):
    """Rewrites, in place, the scale fields of Q4_K super-blocks so that the decoded weights are
    zero-mean: sc = old_sc % 5, m = 15*sc, dmin = d/2, hence w = d*sc*(q - 7.5).  The blocks stay
    valid Q4_K (quants and d untouched).  With the plain recipe (independent uniform scale and
    min fields) every Q4_K matrix has a large common offset and a random-init model emits one
    token with a margin of hundreds, which makes greedy identity vacuous; this recipe gives a
    model whose logits actually compete.  Field layout as get_scale_min_k4, quant.rs:7866."""
    b = packed.reshape(-1, 144)
    q = b[:, 4:16]
    sc = np.empty((b.shape[0], 8), np.uint8)
    sc[:, :4] = q[:, 0:4] & 63
    sc[:, 4:] = (q[:, 8:12] & 0xF) | ((q[:, 0:4] >> 6) << 4)
    sc %= 5
    m = sc * 15
    q[:, 0:4] = sc[:, :4]
    q[:, 4:8] = m[:, :4] | ((m[:, 4:] >> 4) << 6)
    q[:, 8:12] = sc[:, 4:] | ((m[:, 4:] & 0xF) << 4)
    d = b[:, 0:2].copy().view(np.float16).astype(np.float32)
    b[:, 2:4] = (d * 0.5).astype(np.float16).view(np.uint8)
    return packed


def centered_weights(cfg, base_seed):
    """Packed weights of tensor_list(cfg) plus token_embd, Q4_K tensors centred."""
    from llama_rust_b200 import synth
    out = []
    for name, dt, rows, cols in tensor_list(cfg):
        w = synth.packed_matrix(dt, rows, cols, synth.tensor_seed(base_seed, name))
        out.append(center_q4k(w) if dt == Q4_K else w)
    embd = center_q4k(synth.packed_matrix(Q4_K, cfg["n_vocab"], cfg["n_embd"], synth.tensor_seed(base_seed, "token_embd.weight")))
    return out, embd


def compared_prefix(ids_ref, margin_ref, logit_scale, tol=1e-3):
    """Number of leading generated tokens on which greedy identity is decidable: up to and
    excluding the first step whose reference top-2 margin is below tol*logit_scale (the
    reference's model-level logit tolerance) - past a genuine near-tie either argmax is a
    correct answer and the two runs may legitimately part."""
    near = np.nonzero(np.asarray(margin_ref) < tol * logit_scale)[0]
    return int(near[0]) if near.size else len(ids_ref)
