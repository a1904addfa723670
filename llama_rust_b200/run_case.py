"""Runs one matrix-product case on the GPU: the small driver used for profiling.

  python -m llama_rust_b200.run_case --dtype Q4_K --rows 14336 --cols 4096 --m 1 --reps 20 --copies 8

Generates `copies` distinct synthetic matrices on the device (so that repeated
launches stream from HBM rather than L2), runs `reps` device-pointer launches
round-robin over them on one stream and prints the average launch time measured
with CUDA events, plus the achieved bytes/s against the algorithmic byte count
(packed weights once + 4*M*(cols+rows)).

  python -m llama_rust_b200.run_case --moe 64 --reps 5

runs the routed-expert layer of BASELINE config 5 instead (8 experts, top-2, 4096 / 14336,
Q4_K experts, F32 router; `--moe` = tokens per call) through the host-buffer entry point
with pinned buffers and prints the wall time per layer call.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json

from . import DTYPES, Executor, row_bytes
from .executor import lib


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--dtype", default="Q4_K", choices=sorted(DTYPES))
    ap.add_argument("--rows", type=int, default=14336)
    ap.add_argument("--cols", type=int, default=4096)
    ap.add_argument("--m", type=int, default=1)
    ap.add_argument("--reps", type=int, default=20)
    ap.add_argument("--copies", type=int, default=8)
    ap.add_argument("--path", type=int, default=0, help="0 auto, 1 shape-agnostic, 2 staged FMA, 3 tensor core")
    ap.add_argument("--moe", type=int, default=0, help="tokens per routed-expert layer call (0: matrix-product case)")
    args = ap.parse_args()
    if args.moe:
        return moe_case(args.moe, max(args.reps, 1))

    rt = C.CDLL("libcudart.so.12")
    rt.cudaMalloc.argtypes = [C.POINTER(C.c_void_p), C.c_size_t]
    rt.cudaMemset.argtypes = [C.c_void_p, C.c_int, C.c_size_t]
    rt.cudaEventCreate.argtypes = [C.POINTER(C.c_void_p)]
    rt.cudaEventRecord.argtypes = [C.c_void_p, C.c_void_p]
    rt.cudaEventSynchronize.argtypes = [C.c_void_p]
    rt.cudaEventElapsedTime.argtypes = [C.POINTER(C.c_float), C.c_void_p, C.c_void_p]
    rt.cudaStreamCreate.argtypes = [C.POINTER(C.c_void_p)]

    dt = DTYPES[args.dtype]
    with Executor(0) as ex:
        ex.set_path(args.path)
        mats = [ex.synth(dt, args.rows, args.cols, 1000 + i) for i in range(args.copies)]
        x, y, stream, e0, e1 = (C.c_void_p() for _ in range(5))
        assert rt.cudaMalloc(C.byref(x), 4 * args.m * args.cols) == 0
        assert rt.cudaMalloc(C.byref(y), 4 * args.m * args.rows) == 0
        rt.cudaMemset(x, 0, 4 * args.m * args.cols)
        assert rt.cudaStreamCreate(C.byref(stream)) == 0
        rt.cudaEventCreate(C.byref(e0))
        rt.cudaEventCreate(C.byref(e1))
        L, h = lib(), ex._h
        for i in range(min(args.reps, 3)):  # warm-up
            assert L.llr_matmul_device(h, mats[i % args.copies]._h, args.m, x, y, stream) == 0
        rt.cudaEventRecord(e0, stream)
        for i in range(args.reps):
            assert L.llr_matmul_device(h, mats[i % args.copies]._h, args.m, x, y, stream) == 0
        rt.cudaEventRecord(e1, stream)
        rt.cudaEventSynchronize(e1)
        ms = C.c_float()
        rt.cudaEventElapsedTime(C.byref(ms), e0, e1)
        us = ms.value * 1e3 / args.reps
        nbytes = args.rows * row_bytes(dt, args.cols) + 4 * args.m * (args.cols + args.rows)
        print(json.dumps({"dtype": args.dtype, "rows": args.rows, "cols": args.cols, "m": args.m,
                          "us_per_launch": us, "algorithmic_bytes": nbytes, "GB_per_s": nbytes / us / 1e3,
                          "launches": ex.counters()["launches"]}))
        for m in mats:
            m.free()


def moe_case(tokens: int, reps: int) -> None:
    import time

    import numpy as np
    import torch  # pinned host buffers only

    n_exp, d_model, d_ff, q4k, f32 = 8, 4096, 14336, DTYPES["Q4_K"], DTYPES["F32"]
    with Executor(0) as ex:
        gate = [ex.synth(q4k, d_ff, d_model, 100 + e) for e in range(n_exp)]
        up = [ex.synth(q4k, d_ff, d_model, 200 + e) for e in range(n_exp)]
        down = [ex.synth(q4k, d_model, d_ff, 300 + e) for e in range(n_exp)]
        rng = np.random.default_rng(1)
        w = (rng.standard_normal((n_exp, d_model)) * 0.05).astype(np.float32)
        router = ex.upload(f32, n_exp, d_model, w.view(np.uint8).reshape(-1))
        x = torch.randn(tokens, d_model).pin_memory().numpy()
        out = torch.empty(tokens, d_model).pin_memory().numpy()
        for _ in range(2):
            ex.moe_ffn(router, gate, up, down, 2, True, x, out)
        t0 = time.perf_counter()
        for _ in range(reps):
            _, ids, _ = ex.moe_ffn(router, gate, up, down, 2, True, x, out)
        ms = (time.perf_counter() - t0) / reps * 1e3
        flops = 2 * tokens * 2 * 3 * d_model * d_ff
        print(json.dumps({"moe_tokens": tokens, "ms_per_layer_call": ms, "TFLOP_per_s": flops / ms / 1e9,
                          "rows_per_expert": np.bincount(np.asarray(ids).reshape(-1), minlength=n_exp).tolist(),
                          "launches": ex.counters()["launches"]}))


if __name__ == "__main__":
    main()
