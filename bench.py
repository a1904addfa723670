#!/usr/bin/env python
"""Benchmark of the quantized matrix-product path on B200.

One "step" is the matmul sweep of one decode token of a Llama-3-8B-shaped model
in a Q4_K_M-style mix (benchmark configs 2 and 3): per layer attn_q/attn_k/
attn_output/ffn_gate/ffn_up as Q4_K and attn_v/ffn_down as Q6_K, 32 layers, plus
the Q6_K lm_head -- 225 decode GEMVs over 4 875 853 824 packed weight bytes, every
matrix distinct, so each step streams far more than the 126 MB L2 and no flush
is needed between steps.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--m M] [--impl ours|reference]

Prints one JSON line (rank 0).  `value` is the whole-job achieved HBM GB/s
(algorithmic bytes of the sweep / device time, inputs resident in HBM); `e2e`
is the same metric through the reference-facing host-pointer call
(llr_gemm_resident, 225 synchronous calls per step, pinned host buffers);
`e2e_program` is the same through the program API (one copy in, one launch,
one copy out per step; at N > 1 this is `e2e`);
`roofline` is the kernel the timed region consists of (the persistent program
kernel; the Q4_K single-product launches are reported beside it) against the
measured HBM peak; `cpu_baseline` is the CPU oracle (AVX2 row kernels, reference threading)
on a bounded sample of the same sweep.  `configs` holds the other benchmark configurations (1: the
single Q8_0 product; every format's decode kernel on one large matrix; 4: the chunk GEMM; 5: the
routed-expert layer, at N > 1 expert-parallel over peer stores beside the NCCL all-to-all form;
3: the walk on the device).  `--case gemv|moe|session` runs one small case for profiling.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

F32, Q4_K, Q6_K = 2, 17, 19
N_LAYER, D_MODEL, D_KV, D_FF, VOCAB = 32, 4096, 1024, 14336, 128256
LAYER = [  # (name, dtype, rows, cols)  -- decode.rs:2737-3057 call order
    ("attn_q", Q4_K, D_MODEL, D_MODEL), ("attn_k", Q4_K, D_KV, D_MODEL), ("attn_v", Q6_K, D_KV, D_MODEL),
    ("attn_output", Q4_K, D_MODEL, D_MODEL), ("ffn_gate", Q4_K, D_FF, D_MODEL),
    ("ffn_up", Q4_K, D_FF, D_MODEL), ("ffn_down", Q6_K, D_MODEL, D_FF),
]
METRIC = "Q4_K/Q6_K decode GEMV HBM GB/s over the 8B decode-step matmul sweep"
WORKLOAD = ("llama3-8b-shaped decode-step matmul sweep: 32x(q,k,o,gate,up Q4_K; v,down Q6_K) + lm_head Q6_K, "
            "225 GEMVs, 4875853824 packed bytes")


def model_matrices():
    mats = []
    for layer in range(N_LAYER):
        for name, dt, rows, cols in LAYER:
            mats.append((f"blk.{layer}.{name}.weight", dt, rows, cols))
    mats.append(("output.weight", Q6_K, VOCAB, D_MODEL))
    return mats


def row_bytes(dt, cols):
    return {Q4_K: 144, Q6_K: 210}[dt] * (cols // 256)


def algorithmic_bytes(dt, rows, cols, m):
    """Algorithmic bytes of one product: the packed weights once + 4*M*(cols+rows) of activations and results."""
    return rows * row_bytes(dt, cols) + 4 * m * (cols + rows)


def load_peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


class ClockSampler:
    """nvidia-smi clocks and throttle reasons sampled while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.rows, self.proc, self.index = [], None, index

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        self.t.join(timeout=2)
        sm = [float(r[1]) for r in self.rows if len(r) >= 9 and r[1].replace(".", "").isdigit()]
        mx = [float(r[2]) for r in self.rows if len(r) >= 9 and r[2].replace(".", "").isdigit()]
        reasons = set()
        for r in self.rows:
            if len(r) >= 9:
                for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[5:9]):
                    if v.lower().startswith("active"):
                        reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


# ---------------------------------------------------------------------------- CPU arm
def cpu_sweep(threads: int, seconds_budget: float = 20.0):
    """Times the CPU oracle (AVX2 restatement of the reference row kernels, reference
    threading) on a bounded sample: layer 0's seven matrices plus the first 8016 rows
    (1/16) of the lm_head, weights from the host generator with the bench's seeds."""
    from llama_rust_b200 import synth
    from oracle import pyoracle as orc
    sample = [(f"blk.0.{n}.weight", dt, r, c) for n, dt, r, c in LAYER] + [("output.weight", Q6_K, VOCAB // 16, D_MODEL)]
    mats, nbytes = [], 0
    for name, dt, rows, cols in sample:
        w = synth.packed_matrix(dt, rows, cols, synth.tensor_seed(0, name))
        x = synth.activations(cols, synth.tensor_seed(0, name + ".x"))
        mats.append((dt, rows, cols, w, x))
        nbytes += algorithmic_bytes(dt, rows, cols, 1)

    def sweep():
        for dt, rows, cols, w, x in mats:
            orc.gemv(dt, cols, w, x, rows, simd=True, threads=threads)
    sweep()  # warm-up, as kernel_throughput does (simd/tests.rs:1845-1906)
    t0 = time.perf_counter()
    reps = 0
    while True:
        sweep()
        reps += 1
        dt_s = time.perf_counter() - t0
        if reps >= 4 and (dt_s > seconds_budget or reps >= 64):
            break
    gbs = nbytes * reps / dt_s / 1e9
    cores = min(os.cpu_count() or 1, 10) if threads == 0 else threads
    return {"value": gbs, "unit": "GB/s", "cores": cores, "kind": "port",
            "sample": f"layer 0 (7 matrices) + 1/16 of lm_head = {nbytes} B per sweep, {reps} timed sweeps after 1 warm-up; "
                      "oracle = C++ restatement of the reference's AVX2 row kernels (no Rust toolchain here)",
            "ms_per_sweep": dt_s / reps * 1e3,
            "tok_s_equiv": gbs * 1e9 / sum(algorithmic_bytes(dt, r, c, 1) for _, dt, r, c in model_matrices())}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    t0 = time.perf_counter()
    res = cpu_sweep(0, seconds_budget=max(2.0, 1.5 * (args.steps + args.warmup)))
    total = sum(algorithmic_bytes(dt, r, c, 1) for _, dt, r, c in model_matrices())
    ms = total / (res["value"] * 1e9) * 1e3
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": res["value"], "unit": "GB/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "m": 1, "note": "CPU row kernels on the host cores; ms_per_step extrapolated from the sample"},
        "cpu_baseline": res,
        "e2e": {"value": res["value"], "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "tok_s": res["tok_s_equiv"], "wall_s": time.perf_counter() - t0}))


# ---------------------------------------------------------------------------- GPU arm
def decode_step_ops(mat_of, addr_of, h0, ones, M):
    """The 225 products of one decode step as a data-flow chain (llr_program_op), in the walk's order
    (decode.rs:2737-3097): rmsnorm(h) -> q|k|v; o (+ h); rmsnorm -> gate|up; silu(gate)*up -> down (+ h').
    The attention itself is not a matrix product and not part of this sweep: attn_output reads the q
    result in its place.  mat_of(name) -> resident matrix (this rank's rows), addr_of(name) -> device
    address of that product's full-width result."""
    from llama_rust_b200 import XOP_NONE, XOP_RMSNORM, XOP_SWIGLU
    ops, phase = [], 0
    h = h0
    for layer in range(N_LAYER):
        n = lambda t: f"blk.{layer}.{t}.weight"  # noqa: E731
        for t in ("attn_q", "attn_k", "attn_v"):
            ops.append(dict(name=n(t), x=h, x2=ones, x_op=XOP_RMSNORM, eps=1e-5, phase=phase))
        phase += 1
        ops.append(dict(name=n("attn_output"), x=addr_of(n("attn_q")), resid=h, x_op=XOP_NONE, phase=phase))
        phase += 1
        h1 = addr_of(n("attn_output"))
        for t in ("ffn_gate", "ffn_up"):
            ops.append(dict(name=n(t), x=h1, x2=ones, x_op=XOP_RMSNORM, eps=1e-5, phase=phase))
        phase += 1
        ops.append(dict(name=n("ffn_down"), x=addr_of(n("ffn_gate")), x2=addr_of(n("ffn_up")), resid=h1,
                        x_op=XOP_SWIGLU, phase=phase))
        phase += 1
        h = addr_of(n("ffn_down"))
    ops.append(dict(name="output.weight", x=h, x2=ones, x_op=XOP_RMSNORM, eps=1e-5, phase=phase))
    for o in ops:
        o["matrix"] = mat_of(o["name"])
        o["tokens"] = M
    return ops


def timed(stream, fn, reps):
    """Average device time of fn() in ms over reps calls on `stream` (CUDA events on that stream)."""
    import torch
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(reps):
        fn()
    e1.record(stream)
    e1.synchronize()
    return e0.elapsed_time(e1) / reps


def session_leg(ex, mats, specs_all):
    """benchmark config 3 as one sequence on the device-resident walk (llr_session_*): 512 random prompt tokens, then
    128 greedy tokens.  Wall time through the C ABI with host token ids in and out; prefill with the automatic kernel
    choice (tensor-core GEMM for the 512-row chunk), decode with the f32-faithful decode kernels."""
    from llama_rust_b200 import Session, synth
    cfg = dict(n_layer=N_LAYER, n_embd=D_MODEL, n_head=32, n_head_kv=8, head_dim=128, n_ff=D_FF, n_vocab=VOCAB, n_ctx=640)
    embd = ex.synth(Q4_K, VOCAB, D_MODEL, synth.tensor_seed(0, "token_embd.weight"))
    layers = [{t: mats[f"blk.{li}.{t}.weight"] for t, *_ in LAYER} for li in range(N_LAYER)]
    s = Session(ex, cfg, embd, layers, output=mats["output.weight"])
    prompt = (synth.words(7, 0, 512) % np.uint64(VOCAB)).astype(np.int32)
    s.prefill(prompt[:8])  # warm-up of both phases
    s.decode(4)
    s.reset()
    t0 = time.perf_counter()
    s.prefill(prompt)
    t1 = time.perf_counter()
    ids, _ = s.decode(128)
    t2 = time.perf_counter()
    out = {"prefill_ms_512_tokens": (t1 - t0) * 1e3, "prefill_tok_s": 512 / (t1 - t0), "decode_ms_per_token": (t2 - t1) / 128 * 1e3,
           "decode_tok_s": 128 / (t2 - t1), "distinct_tokens": int(len(set(ids.tolist()))),
           "what": "llr_session_prefill + llr_session_decode: embedding, RMSNorm, RoPE, KV cache, attention, SwiGLU, argmax and the "
                   "225 products per token on the device; one host synchronization per call"}
    s.free()
    embd.free()
    return out


def config_legs(ex, stream, peak_hbm, peaks):
    """Driver-visible numbers for benchmark configs 1, 4 and 5 on one GPU (device time, CUDA events):
    config 1 the single Q8_0 product, every format's decode kernel on one large matrix, config 4 the chunk GEMM (tensor-core path, 16-bit operands) for
    four formats at three batch sizes, config 5 the routed-expert layer at 64 and 512 tokens."""
    import torch
    from llama_rust_b200 import DTYPES
    out = {}
    sptr = stream.cuda_stream
    Q8_0, Q5_0, Q5_1 = DTYPES["Q8_0"], DTYPES["Q5_0"], DTYPES["Q5_1"]
    rb = lambda dt, cols: {Q4_K: 144 * (cols // 256), Q6_K: 210 * (cols // 256), Q8_0: 34 * (cols // 32),  # noqa: E731
                           Q5_0: 22 * (cols // 32), Q5_1: 24 * (cols // 32)}[dt]
    # config 1: 4096 x 4096 Q8_0, one activation row, 8 distinct matrices round-robin (142 MB > L2)
    mats = [ex.synth(Q8_0, 4096, 4096, 500 + i) for i in range(8)]
    x = torch.randn(4096, device="cuda")
    y = torch.empty(4096, device="cuda")
    it = [0]

    def one():
        ex.matmul_device(mats[it[0] % 8], 1, x.data_ptr(), y.data_ptr(), sptr)
        it[0] += 1
    timed(stream, one, 16)
    ms = timed(stream, one, 64)
    nbytes = 4096 * rb(Q8_0, 4096) + 4 * 2 * 4096
    out["config1_q8_0_4096x4096_m1"] = {"us_per_product": ms * 1e3, "GB_per_s": nbytes / ms / 1e6, "frac_of_hbm_peak": nbytes / ms / 1e6 / peak_hbm,
                                       "algorithmic_bytes": nbytes, "launch": "one PDL launch per product, 8 distinct matrices"}
    for m in mats:
        m.free()
    # every format's decode kernel on one large matrix (65536 x 4096, one activation row, 4 distinct matrices round-robin:
    # 0.6-4.3 GB, far beyond L2): what a format's kernel sustains when the launch is long enough to stream
    from llama_rust_b200 import row_bytes as lib_row_bytes
    fm = {}
    for name in ("Q4_K", "Q5_K", "Q6_K", "Q8_0", "Q4_0", "Q4_1", "Q5_0", "Q5_1", "F16", "BF16", "F32"):
        dt, rows, cols = DTYPES[name], 65536, 4096
        mats = [ex.synth(dt, rows, cols, 700 + i) for i in range(4)]
        x = torch.randn(cols, device="cuda")
        y = torch.empty(rows, device="cuda")
        it = [0]

        def one():
            ex.matmul_device(mats[it[0] % 4], 1, x.data_ptr(), y.data_ptr(), sptr)
            it[0] += 1
        timed(stream, one, 4)
        ms = timed(stream, one, 24)
        nbytes = rows * lib_row_bytes(dt, cols) + 4 * (rows + cols)
        fm[name] = {"us_per_product": ms * 1e3, "GB_per_s": nbytes / ms / 1e6, "frac_of_hbm_peak": nbytes / ms / 1e6 / peak_hbm}
        for m in mats:
            m.free()
    out["decode_formats_65536x4096_m1"] = fm
    # config 4
    burst, sustained = peaks.get("bf16_tflops", 1619.1), peaks.get("bf16_tflops_sustained", 1354.7)
    c4 = {}
    for name, dt, rows, cols in (("q4_k_14336x4096", Q4_K, 14336, 4096), ("q8_0_4096x14336", Q8_0, 4096, 14336),
                                 ("q5_0_4096x4096", Q5_0, 4096, 4096), ("q5_1_4096x4096", Q5_1, 4096, 4096)):
        mats = [ex.synth(dt, rows, cols, 600 + i) for i in range(6)]
        for M in (64, 256, 1024):
            x = torch.randn(M, cols, device="cuda")
            y = torch.empty(M, rows, device="cuda")
            it = [0]

            def one():
                ex.matmul_device(mats[it[0] % 6], M, x.data_ptr(), y.data_ptr(), sptr)
                it[0] += 1
            timed(stream, one, 6)
            ms = timed(stream, one, 30)
            flops = 2.0 * M * rows * cols
            nbytes = rows * rb(dt, cols) + 4 * M * (rows + cols)
            floor_us = max(nbytes / (peak_hbm * 1e9), flops / (sustained * 1e12)) * 1e6
            c4[f"{name}_m{M}"] = {"us_per_call": ms * 1e3, "TFLOP_per_s": flops / ms / 1e9, "frac_of_burst": flops / ms / 1e9 / burst,
                                  "frac_of_sustained": flops / ms / 1e9 / sustained, "roofline_us": floor_us,
                                  "frac_of_roofline": floor_us / (ms * 1e3)}
        for m in mats:
            m.free()
    out["config4_chunk_gemm"] = c4
    # config 5
    out["config5_moe_layer"] = moe_leg(ex, None, 0, 1, peak_hbm, sustained)
    return out


def moe_leg(ex, group, rank, world, peak_hbm, sustained, token_counts=(64, 512)):
    """Routed-expert layer of benchmark config 5 (8 experts, top-2, 4096 / 14336, Q4_K experts, F32 router) through
    the host-buffer entry point with pinned buffers: wall ms per layer call.  world > 1: experts striped e % world, tokens
    sharded on the device, routed rows and results exchanged by peer stores inside the library (llr_moe_ep_*); the same
    layer over NCCL all-to-all is timed beside it; every rank compares its tokens' outputs bit for bit with the
    single-device layer."""
    import torch
    import torch.distributed as dist
    from llama_rust_b200 import DTYPES
    n_exp, d_model, d_ff = 8, 4096, 14336
    gate = [ex.synth(Q4_K, d_ff, d_model, 100 + e) for e in range(n_exp)]
    up = [ex.synth(Q4_K, d_ff, d_model, 200 + e) for e in range(n_exp)]
    down = [ex.synth(Q4_K, d_model, d_ff, 300 + e) for e in range(n_exp)]
    rng = np.random.default_rng(1)
    w = (rng.standard_normal((n_exp, d_model)) * 0.05).astype(np.float32)
    router = ex.upload(DTYPES["F32"], n_exp, d_model, w.view(np.uint8).reshape(-1))
    res = {}
    layer = nccl_layer = None
    if world > 1:
        from llama_rust_b200.sharding import ExpertParallelLayer, PeerExpertParallelLayer, home_rank
        keep = [home_rank(e, world) == rank for e in range(n_exp)]
        mine = [[m if k else None for m, k in zip(lst, keep)] for lst in (gate, up, down)]
        layer = PeerExpertParallelLayer(ex, router, mine[0], mine[1], mine[2], 2, True, max(token_counts) // world + 1, group=group)
        route, experts = ExpertParallelLayer.cuda_backend(ex, router, mine[0], mine[1], mine[2], 2, True)
        nccl_layer = ExpertParallelLayer(n_exp, 2, route, experts, group=group)

    def timed(call, n=5):
        for _ in range(2):
            call()
        torch.cuda.synchronize()  # also keeps torch's one-time CUDA set-up out of the timed region
        if world > 1:
            dist.barrier()
        t0 = time.perf_counter()
        for _ in range(n):
            call()
        torch.cuda.synchronize()
        ms = (time.perf_counter() - t0) / n * 1e3
        if world > 1:
            tt = torch.tensor([ms], device="cuda")
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
            ms = float(tt.item())
        return ms
    for tokens in token_counts:
        xs = np.random.default_rng(tokens).standard_normal((tokens, d_model)).astype(np.float32)
        x = torch.from_numpy(xs).pin_memory().numpy()
        out = torch.empty(tokens, d_model).pin_memory().numpy()
        if layer is not None:
            # tokens sharded over the ranks: device tensors in, device tensors out
            lo, hi = tokens * rank // world, tokens * (rank + 1) // world
            xl = torch.from_numpy(np.ascontiguousarray(xs[lo:hi])).cuda()
            ms = timed(lambda: layer(xl))
            ms_nccl = timed(lambda: nccl_layer(xl))
        else:
            ms = timed(lambda: ex.moe_ffn(router, gate, up, down, 2, True, x, out))
            # the same layer with the tokens already on the device and the output left there (the expert-parallel entry
            # points with a world of one rank): what the N > 1 figures, whose tokens live on the device, compare with
            from llama_rust_b200.executor import moe_ep_arena_bytes
            nb = moe_ep_arena_bytes(n_exp, 2, d_model, 1, tokens)
            arena = ex.shared_alloc(nb)[0]
            ep = ex.moe_ep(router, gate, up, down, 2, True, 1, 0, tokens, arena, nb, [arena])
            xd, od = torch.from_numpy(xs).cuda(), torch.empty(tokens, d_model, device="cuda")

            def on_device():
                ep.run(tokens, xd.data_ptr(), od.data_ptr())
                ex.synchronize()
            ms_dev = timed(on_device)
            ep.free()
            ex.shared_free(arena)
        flops = 2.0 * tokens * 2 * 3 * d_model * d_ff
        nbytes = n_exp * 3 * d_ff * 144 * (d_model // 256)
        floor_ms = max(nbytes / world / (peak_hbm * 1e9), flops / world / (sustained * 1e12)) * 1e3
        rec = {"ms_per_layer_call": ms, "TFLOP_per_s": flops / ms / 1e9, "roofline_ms": floor_ms, "frac_of_roofline": floor_ms / ms}
        if world == 1:
            rec["tokens_on_device_ms_per_layer_call"] = ms_dev
        if world > 1:
            # untimed check with the f32-faithful products, whose rows do not depend on their batch: same bits as the
            # single-device layer on this rank's tokens (the automatic choice picks kernels by the number of rows)
            ex.set_path(3)
            full = ex.moe_ffn(router, gate, up, down, 2, True, xs[lo:hi])[0]
            dist.barrier()
            chk = layer(xl)[0].cpu().numpy()
            chk_nccl = nccl_layer(xl)[0].cpu().numpy()
            ex.set_path(0)
            same = torch.tensor([1 if np.array_equal(chk, full) and np.array_equal(chk_nccl, full) else 0], device="cuda")
            dist.all_reduce(same, op=dist.ReduceOp.MIN)
            rec["bit_identical_to_single_device"] = bool(same.item())
            rec["layout"] = (f"tokens/{world} per rank on the device, experts e % {world}, routed rows and results exchanged by peer "
                             "stores from the library's gather / scatter kernels")
            rec["same_layer_over_nccl_all_to_all_ms"] = ms_nccl
        res[f"tokens_{tokens}"] = rec
    if layer is not None:
        dist.barrier()
        layer.close()
    for m in gate + up + down + [router]:
        m.free()
    return res


def run_ours(args):
    import torch
    import torch.distributed as dist
    from llama_rust_b200 import Executor, synth

    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback)")
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    M = args.m
    torch.manual_seed(1234)  # the step's input is replicated: the same values on every rank
    ex = Executor(local)
    stream = torch.cuda.Stream(device=local)
    sptr = stream.cuda_stream
    peak, peak_kind = load_peaks()
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            peaks = json.load(f)
    except Exception:
        peaks = {}

    # every matrix sharded by output rows (all row counts divide by 8)
    specs_all = model_matrices()
    mats = {}
    for name, dt, rows, cols in specs_all:
        assert rows % world == 0
        # each rank generates its own shard from its own stream: rank r's rows are blocks of stream (name, r)
        mats[name] = ex.synth(dt, rows // world, cols, synth.tensor_seed(rank, name))
    shape_of = {name: (dt, rows, cols) for name, dt, rows, cols in specs_all}
    total_bytes = sum(algorithmic_bytes(dt, rows, cols, M) for _, dt, rows, cols in specs_all)
    h0 = torch.randn(M, D_MODEL, device="cuda", dtype=torch.float32)
    ones = torch.ones(D_MODEL, device="cuda", dtype=torch.float32)
    # independent inputs for the one-launch-per-product legs
    xin = {cols: torch.randn(M, cols, device="cuda") for cols in (D_MODEL, D_FF)}
    torch.cuda.synchronize()

    prog = sharded = ybig = chain = None
    offs = {}
    PHASE = {"attn_q": 0, "attn_k": 0, "attn_v": 0, "attn_output": 1, "ffn_gate": 2, "ffn_up": 2, "ffn_down": 3}

    def phase_of(name):
        parts = name.split(".")
        return 4 * int(parts[1]) + PHASE[parts[2]] if parts[0] == "blk" else 4 * N_LAYER
    if args.mode == "program":
        # One persistent launch per rank and step.  Phases follow the model's dependency structure: {q,k,v} -> {o} ->
        # {gate,up} -> {down} per layer, then the lm_head; a phase starts only when the previous one is completely
        # written (strict phases: one counter per phase).
        if world == 1:
            cur = 0
            for name, dt, rows, cols in specs_all:
                offs[name] = cur
                cur += M * rows
            ybig = torch.empty(cur, device="cuda", dtype=torch.float32)
            prog = ex.program([(mats[n], xin[cols].data_ptr(), ybig.data_ptr() + 4 * offs[n], M, phase_of(n))
                               for n, dt, rows, cols in specs_all])
            # the same step as a data-flow chain: results travel from product to product inside the launch, RMSNorm /
            # SwiGLU / residual adds applied by the readers and writers (reported beside the headline, see `fused_chain`)
            ops = decode_step_ops(lambda n: mats[n], lambda n: ybig.data_ptr() + 4 * offs[n], h0.data_ptr(), ones.data_ptr(), M)
            for o in ops:
                o["y"] = ybig.data_ptr() + 4 * offs[o["name"]]
            chain = ex.program_ops(ops)
        else:
            from llama_rust_b200.sharding import ShardedDecodeProgram, arena_layout
            order = [n for n, *_ in specs_all]
            aoffs, _ = arena_layout([shape_of[n][1] for n in order], M)
            offs = dict(zip(order, aoffs))
            sharded = ShardedDecodeProgram(ex, [(mats[n], xin[cols].data_ptr(), rows, phase_of(n)) for n, dt, rows, cols in specs_all], M)
            prog = sharded.program
        info = prog.info()

    def step():
        if prog is not None:
            prog.run(sptr)
            return
        for name, dt, rows, cols in specs_all:  # --mode calls: one launch per product, independent inputs
            ex.matmul_device(mats[name], M, xin[cols].data_ptr(), ycall.data_ptr(), sptr)
            if world > 1:  # the library baseline: a NCCL all-gather after every product
                with torch.cuda.stream(stream):
                    dist.all_gather_into_tensor(ygather[:world * M * (rows // world)], ycall[:M * (rows // world)])
    ycall = torch.empty(M * VOCAB, device="cuda")
    ygather = torch.empty(M * VOCAB, device="cuda") if world > 1 else None

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    clocks = ClockSampler(local)
    if rank == 0:
        clocks.start()  # sampled from warm-up to the end of the roofline pass
    for _ in range(max(args.warmup, 3)):
        step()
    barrier()
    ex.synchronize()

    # ---- untimed check of the sharded program: every rank compares the first layers' full-width results in its
    # arena, bit for bit, with the same products run unsharded on its own GPU
    sharded_check = None
    if sharded is not None:
        sharded_check = check_sharded(ex, sharded, offs, shape_of, xin, phase_of, M, world, rank, sptr, stream)
        flag = torch.tensor([1 if sharded_check["bit_identical"] else 0], device="cuda")
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        sharded_check["bit_identical"] = bool(flag.item())
        sharded_check["ranks"] = world
        barrier()

    launches0 = ex.counters()["launches"]
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record(stream)
    for _ in range(args.steps):
        step()
    e1.record(stream)
    barrier()
    ms_total = e0.elapsed_time(e1)
    launches = ex.counters()["launches"] - launches0
    per_rank_ms = [ms_total / args.steps]
    if world > 1:
        t = torch.tensor([ms_total], device="cuda")
        allt = [torch.zeros_like(t) for _ in range(world)]
        dist.all_gather(allt, t)
        per_rank_ms = [float(v.item()) / args.steps for v in allt]
        ms_total = max(float(v.item()) for v in allt)
        launches *= world
    ms_step = ms_total / args.steps
    value = total_bytes / (ms_step * 1e-3) / 1e9

    # Q4_K decode products one per launch (57% of the sweep's bytes), back to back on the same stream with
    # programmatic dependent launch, every matrix distinct (2.8 GB per pass, no L2 reuse)
    dom = [(n, dt, rows, cols) for n, dt, rows, cols in specs_all if dt == Q4_K]
    reps = max(3, min(args.steps, 20))

    def dom_pass():
        for n, dt, rows, cols in dom:
            ex.matmul_device(mats[n], M, xin[cols].data_ptr(), ycall.data_ptr(), sptr)
    barrier()
    dom_ms = timed(stream, dom_pass, reps) * reps
    torch.cuda.synchronize()
    dom_bytes = reps * sum((rows // world) * row_bytes(dt, cols) + 4 * M * (cols + rows // world) for _, dt, rows, cols in dom)
    clock_rec = clocks.stop() if rank == 0 else None
    achieved = dom_bytes / (dom_ms * 1e-3) / 1e9
    single = {"kernel": "gemv_stream_kernel<M, Q4_K> (one product per launch, programmatic dependent launch)",
              "achieved": achieved, "frac": achieved / peak, "launches_timed": reps * len(dom),
              "avg_launch_us": dom_ms * 1e3 / (reps * len(dom)), "avg_bytes_per_launch": dom_bytes / (reps * len(dom))}
    if prog is not None:
        # The timed region consists of launches of one kernel, the persistent program kernel (one per
        # rank and step): its average launch duration is ms_step, its algorithmic bytes per launch are
        # this rank's share of the sweep.  traffic: ncu dram bytes of the streaming kernel equal the
        # algorithmic bytes within 0.03 % (profiles/gemv_stream_q4k_65536x4096_m1.md); not re-measured here.
        per_rank = total_bytes / world
        ach = per_rank / (ms_step * 1e-3) / 1e9
        roofline = {"bound": "hbm", "achieved": ach, "peak": peak, "unit": "GB/s", "frac": ach / peak, "traffic": None,
                    "kernel": "gemv_sharded_program_kernel<M>" if world > 1 else "gemv_program_kernel<M>",
                    "peak_kind": peak_kind, "launches_timed": args.steps, "avg_launch_us": ms_step * 1e3,
                    "avg_bytes_per_launch": per_rank, "frac_of_8tbs_nominal": ach / 8000.0,
                    "single_product_launches": single}
    else:
        roofline = {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                    "traffic": None, "kernel": single["kernel"], "peak_kind": peak_kind,
                    "launches_timed": single["launches_timed"], "avg_launch_us": single["avg_launch_us"],
                    "avg_bytes_per_launch": single["avg_bytes_per_launch"], "frac_of_8tbs_nominal": achieved / 8000.0}

    # end to end through the reference-facing call: host buffers, copies inside the timed region
    e2e_calls = None
    if world == 1:
        hx = {cols: torch.randn(M, cols).pin_memory() for cols in (D_MODEL, D_FF)}
        hy = torch.empty(M, VOCAB).pin_memory()
        from llama_rust_b200.executor import lib
        L, h = lib(), ex._h

        # the arguments of the 225 calls are put together once: what is timed is the library call, as a compiled caller
        # makes it, not the interpreter's attribute look-ups
        call, y_ptr = L.llr_gemm_resident, hy.data_ptr()
        calls = [(h, mats[name]._h, M, hx[cols].data_ptr(), hx[cols].numel(), y_ptr, M * rows) for name, dt, rows, cols in specs_all]

        def e2e_step():
            for a in calls:
                if call(*a):
                    raise RuntimeError(L.llr_exec_last_error(h).decode())
        for _ in range(2):
            e2e_step()
        torch.cuda.synchronize()
        n_e2e = max(2, min(args.steps, 10))
        t0 = time.perf_counter()
        for _ in range(n_e2e):
            e2e_step()
        torch.cuda.synchronize()
        dt_s = (time.perf_counter() - t0) / n_e2e
        e2e_calls = {"value": total_bytes / dt_s / 1e9, "unit": "GB/s",
                     "h2d_bytes_per_step": sum(4 * M * cols for _, _, _, cols in specs_all),
                     "d2h_bytes_per_step": sum(4 * M * rows for _, _, rows, _ in specs_all),
                     "ms_per_step": dt_s * 1e3, "tok_s": M / dt_s,
                     "api": "llr_gemm_resident with pinned host buffers, 225 synchronous calls per step: H2D copy of x, kernel, the kernel stores y into the pinned host buffer and raises a completion word the call polls"}

    e2e_program = None
    if prog is not None:
        # End to end through the program API (llr_program_run): per rank and step the step's input (the hidden state,
        # pinned host memory) goes host -> device, one program launch, the step's result (the logits) comes device ->
        # host, synchronize.  Everything between the 225 products stays on the device.
        import ctypes as C
        rt = C.CDLL("libcudart.so.12")
        rt.cudaMemcpyAsync.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t, C.c_int, C.c_void_p]
        hxb = torch.randn(M, D_MODEL).pin_memory()
        h0 = xin[D_MODEL]  # the hidden state of the step: what attn_q/k/v, attn_output, ffn_gate/up and the lm_head read
        logits_dev = (sharded.arena + offs["output.weight"]) if sharded is not None else ybig.data_ptr() + 4 * offs["output.weight"]
        hyb = torch.empty(M, VOCAB).pin_memory()

        def e2e_prog_step():
            assert rt.cudaMemcpyAsync(h0.data_ptr(), hxb.data_ptr(), 4 * hxb.numel(), 1, sptr) == 0
            prog.run(sptr)
            assert rt.cudaMemcpyAsync(hyb.data_ptr(), logits_dev, 4 * hyb.numel(), 2, sptr) == 0
            stream.synchronize()
        barrier()  # rank 0 has just stopped its clock sampler: the ranks enter the exchange of the next launch together
        ex.synchronize()  # raises if a bounded device-side wait gave up in anything above
        for _ in range(2):
            e2e_prog_step()
        barrier()
        n_e2e = max(2, min(args.steps, 10))
        t0 = time.perf_counter()
        for _ in range(n_e2e):
            e2e_prog_step()
        barrier()
        dt_s = (time.perf_counter() - t0) / n_e2e
        if world > 1:
            tt = torch.tensor([dt_s], device="cuda")
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
            dt_s = float(tt.item())
        e2e_program = {"value": total_bytes / dt_s / 1e9, "unit": "GB/s",
                       "h2d_bytes_per_step": world * 4 * hxb.numel(), "d2h_bytes_per_step": world * 4 * hyb.numel(),
                       "ms_per_step": dt_s * 1e3, "tok_s": M / dt_s,
                       "api": "per rank and step: the step's input (hidden state) H2D from pinned memory, llr_program_run (225 products), "
                              "the step's result (logits) D2H, synchronize; intermediate results stay on the device"}
    # `e2e`: the reference-facing per-product call on one GPU; a row-sharded product per call would need a collective
    # per product, so on several GPUs it is the program API.  `e2e_program` is the series that is comparable over N.
    e2e = e2e_calls if world == 1 else e2e_program
    if e2e is not None:
        e2e = dict(e2e, kind="per-product calls (reference call contract)" if world == 1 else "program API")

    def secondary(leg):
        # the legs beside the headline must not cost the headline line (measured above) if one of them fails
        try:
            return leg()
        except Exception as exc:  # noqa: BLE001
            return {"error": f"{type(exc).__name__}: {exc}"}

    def chain_leg():
        for _ in range(3):
            chain.run(sptr)
        cms = timed(stream, lambda: chain.run(sptr), max(3, min(args.steps, 20)))
        ex.synchronize()
        ci = chain.info()
        rec = {"ms_per_step": cms, "GB_per_s": total_bytes / cms / 1e6, "frac_of_hbm_peak": total_bytes / cms / 1e6 / peak,
               "phases": ci["phases"], "counter_phases": ci["counter_phases"], "ctas": ci["ctas"],
               "what": "the same 225 products as a data-flow program (llr_program_create_ops): each product reads earlier results as tagged "
                       "pairs, RMSNorm / SwiGLU / residual adds run inside the launch, attn_output reads the q result in place of the attention output"}
        chain.free()
        return rec
    fused_chain = secondary(chain_leg) if chain is not None else None
    configs = None
    if not args.no_configs and args.mode == "program":
        if world == 1:
            configs = secondary(lambda: config_legs(ex, stream, peak, peaks))
            configs["config3_device_resident_walk"] = secondary(lambda: session_leg(ex, mats, specs_all))
        else:
            sustained = peaks.get("bf16_tflops_sustained", 1354.7)
            configs = {"config5_moe_layer_striped": moe_leg(ex, None, rank, world, peak, sustained)}

    out = None
    if rank == 0:
        cpu = secondary(lambda: cpu_sweep(0, seconds_budget=15.0)) if world == 1 and not args.no_cpu else None
        out = {
            "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": WORKLOAD, "m": M,
                       "launch": (f"one persistent program launch per rank and step, {info['phases']} dependent phases "
                                  f"(a phase starts when the previous one is completely written), {info['ctas']} CTAs"
                                  if prog is not None else "one PDL launch per matmul"),
                       "l2": "inputs larger than L2: every step streams 4.9 GB of distinct weights",
                       "parallelism": ("single GPU" if world == 1 else
                                       f"rows/{world} per GPU; result slices exchanged inside the kernel (peer stores over NVLink + phase counters over all ranks)"
                                       if sharded is not None else f"rows/{world} per GPU + NCCL all-gather of output slices after every product")},
            "tok_s": M / (ms_step * 1e-3), "frac_of_measured_hbm": value / peak, "frac_of_8tbs_nominal": value / 8000.0,
            "roofline": roofline, "cpu_baseline": cpu, "e2e": e2e, "e2e_program": e2e_program, "gpu_launches": int(launches),
            "per_rank_ms_per_step": per_rank_ms, "sharded_check": sharded_check, "fused_chain": fused_chain, "configs": configs,
            "clocks": clock_rec,
        }
        print(json.dumps(out))
    if sharded is not None:
        sharded.close()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if sharded_check is not None and not sharded_check["bit_identical"]:
        raise SystemExit("sharded program results differ from the unsharded program")
    return out


def check_sharded(ex, sharded, offs, shape_of, xin, phase_of, M, world, rank, sptr, stream, layers=2):
    """Runs the first `layers` layers unsharded on this GPU (full matrices rebuilt from every rank's shard stream)
    with the same input and compares their results, bit for bit, with what the sharded program left in this
    rank's arena (this rank's rows and the rows the peers stored)."""
    import ctypes as C

    import torch
    import torch.distributed as dist
    from llama_rust_b200 import synth
    rt = C.CDLL("libcudart.so.12")
    rt.cudaMemcpy.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t, C.c_int]
    names = [f"blk.{layer}.{t}.weight" for layer in range(layers) for t, *_ in LAYER]
    full = {}
    for n in names:
        dt, rows, cols = shape_of[n]
        parts = []
        for g in range(world):
            m = ex.synth(dt, rows // world, cols, synth.tensor_seed(g, n))
            parts.append(ex.download(m))
            m.free()
        full[n] = ex.upload(dt, rows, cols, np.concatenate(parts))
    cur, roffs = 0, {}
    for n in names:
        roffs[n] = cur
        cur += M * shape_of[n][1]
    yref = torch.full((cur,), float("nan"), device="cuda")
    ref = ex.program([(full[n], xin[shape_of[n][2]].data_ptr(), yref.data_ptr() + 4 * roffs[n], M, phase_of(n)) for n in names])
    dist.barrier()
    sharded.run(sptr)
    ref.run(sptr)
    ex.synchronize()
    stream.synchronize()
    dist.barrier()  # the peers' stores into this arena are complete as well
    ok, n_bad = True, 0
    host = yref.cpu().numpy()
    for n in names:
        rows = shape_of[n][1]
        got = np.empty(M * rows, np.float32)
        assert rt.cudaMemcpy(got.ctypes.data, sharded.arena + offs[n], 4 * M * rows, 2) == 0
        want = host[roffs[n]:roffs[n] + M * rows]
        same = np.array_equal(got.view(np.uint32), want.view(np.uint32))
        ok = ok and same
        n_bad += 0 if same else 1
    ref.free()
    for m in full.values():
        m.free()
    return {"bit_identical": ok, "entries": len(names), "entries_differing_on_rank0": n_bad, "layers": layers,
            "how": "first layers of the sharded program vs the same products unsharded on each rank's own GPU, all rows, uint32 compare"}


def run_case(args):
    """One small case for profiling (the full sweep holds 5 GB): prints one JSON line.
      --case gemv    --dtype D --rows R --cols C --m M --reps N --copies K [--path P]   device-pointer products round-robin over K matrices
      --case moe     --tokens T                                                        the routed-expert layer of benchmark config 5 (2 warm-up + 5 timed calls)
      --case session --prompt P --gen G [--layers L] [--experts E]                     the device-resident walk on an 8B-shaped model of L layers
                                                                                       (E routed experts per layer, two per token, instead of the dense FFN)"""
    import torch
    from llama_rust_b200 import DTYPES, Executor, row_bytes as lib_row_bytes, synth
    ex = Executor(0)
    if args.path is not None:
        ex.set_path(args.path)
    stream = torch.cuda.Stream()
    sptr = stream.cuda_stream
    if args.case == "gemv":
        dt = DTYPES[args.dtype]
        mats = [ex.synth(dt, args.rows, args.cols, 1000 + i) for i in range(args.copies)]
        x = torch.randn(args.m, args.cols, device="cuda")
        y = torch.empty(args.m, args.rows, device="cuda")
        it = [0]

        def one():
            ex.matmul_device(mats[it[0] % args.copies], args.m, x.data_ptr(), y.data_ptr(), sptr)
            it[0] += 1
        timed(stream, one, min(args.reps, 3))
        ms = timed(stream, one, args.reps)
        nbytes = args.rows * lib_row_bytes(dt, args.cols) + 4 * args.m * (args.cols + args.rows)
        out = {"case": "gemv", "dtype": args.dtype, "rows": args.rows, "cols": args.cols, "m": args.m, "us_per_launch": ms * 1e3,
               "algorithmic_bytes": nbytes, "GB_per_s": nbytes / ms / 1e6, "TFLOP_per_s": 2.0 * args.m * args.rows * args.cols / ms / 1e9,
               "launches": ex.counters()["launches"]}
    elif args.case == "moe":
        peak, _ = load_peaks()
        out = {"case": "moe", **moe_leg(ex, None, 0, 1, peak, 1354.7, token_counts=(args.tokens,))}
    else:
        cfg = dict(n_layer=args.layers, n_embd=D_MODEL, n_head=32, n_head_kv=8, head_dim=128, n_ff=D_FF, n_vocab=VOCAB, n_ctx=max(args.ctx, args.prompt + args.gen + 8))
        from llama_rust_b200 import Session
        embd = ex.synth(Q4_K, VOCAB, D_MODEL, 1)
        one = DTYPES[args.dtype] if args.dtype != "Q4_K" else None  # --dtype D: every layer matrix in that format instead of the Q4_K / Q6_K mix
        layers = [{t: ex.synth(one if one is not None else dt, r, c, 10 * li + j) for j, (t, dt, r, c) in enumerate(LAYER)} for li in range(args.layers)]
        if args.experts:  # config 5's experts in every layer (Mixtral-shaped: routed experts where the dense FFN stands)
            rng = np.random.default_rng(3)
            for li, L in enumerate(layers):
                for t in ("ffn_gate", "ffn_up", "ffn_down"):
                    L.pop(t).free()
                L["n_expert_used"] = 2
                L["ffn_gate_inp"] = ex.upload(DTYPES["F32"], args.experts, D_MODEL,
                                              (rng.standard_normal((args.experts, D_MODEL)) * 0.05).astype(np.float32).view(np.uint8).reshape(-1))
                L["ffn_gate_exps"] = [ex.synth(Q4_K, D_FF, D_MODEL, 1000 * li + e) for e in range(args.experts)]
                L["ffn_up_exps"] = [ex.synth(Q4_K, D_FF, D_MODEL, 1000 * li + 100 + e) for e in range(args.experts)]
                L["ffn_down_exps"] = [ex.synth(Q4_K, D_MODEL, D_FF, 1000 * li + 200 + e) for e in range(args.experts)]
        head = ex.synth(Q6_K, VOCAB, D_MODEL, 2)
        s = Session(ex, cfg, embd, layers, output=head)
        prompt = (synth.words(7, 0, args.prompt) % np.uint64(VOCAB)).astype(np.int32)
        t0 = time.perf_counter()
        s.prefill(prompt)
        t1 = time.perf_counter()
        ids, _ = s.decode(args.gen)
        t2 = time.perf_counter()
        out = {"case": "session", "layers": args.layers, "experts": args.experts, "prefill_ms": (t1 - t0) * 1e3, "decode_ms_per_token": (t2 - t1) / args.gen * 1e3,
               "launches": ex.counters()["launches"]}
    print(json.dumps(out))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--m", type=int, default=1, help="activation rows per matmul (1..8)")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu", action="store_true", help="skip the cpu_baseline leg")
    ap.add_argument("--no-configs", action="store_true", help="skip the legs for benchmark configs 1, 4 and 5")
    ap.add_argument("--mode", default="program", choices=["program", "calls"],
                    help="program: the sweep as one persistent launch; calls: one launch per matmul")
    ap.add_argument("--case", default=None, choices=["gemv", "moe", "session"], help="run one small case instead of the sweep (for profiling)")
    ap.add_argument("--dtype", default="Q4_K")
    ap.add_argument("--rows", type=int, default=65536)
    ap.add_argument("--cols", type=int, default=4096)
    ap.add_argument("--reps", type=int, default=20)
    ap.add_argument("--copies", type=int, default=6)
    ap.add_argument("--path", type=int, default=None, help="kernel path of llr_exec_set_path")
    ap.add_argument("--tokens", type=int, default=64)
    ap.add_argument("--prompt", type=int, default=64)
    ap.add_argument("--gen", type=int, default=4)
    ap.add_argument("--layers", type=int, default=4)
    ap.add_argument("--ctx", type=int, default=0, help="--case session: context length of the session (default: prompt + gen + 8)")
    ap.add_argument("--experts", type=int, default=0, help="--case session: routed experts per layer (0: dense FFN)")
    args = ap.parse_args()
    if args.case:
        return run_case(args)
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
