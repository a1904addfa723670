"""The allocation-free chunk GEMM (llr_gemm_device_noalloc) against the regular device-pointer
entry point (llr_matmul_device) on the same kernel: identical results on two calls in a row.

The point of the entry point is that a caller whose GPU memory is already spoken for (KV pool
plus weights filling the device, or a region where cudaMalloc's implicit synchronization is not
allowed) can still run prefill chunks: the bf16 staging buffer is a fixed array inside the
library.  This file sorts last on purpose, so a run that stops at the first failure has
already run every other test."""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

Q4_K, Q8_0, TC = 17, 13, 4


def test_noalloc_gemm_matches_regular_entry_point_twice():
    import torch
    from llama_rust_b200 import Executor
    from llama_rust_b200.executor import lib
    L = lib()
    ex = Executor(0)
    ex.set_path(TC)
    rows, cols = 384, 2048
    for dtype, seed in ((Q4_K, 11), (Q8_0, 12)):
        m = ex.synth(dtype, rows, cols, seed)
        for call, tokens in enumerate((96, 200)):  # two calls in a row, the second larger than the first
            g = torch.Generator(device="cuda").manual_seed(100 * seed + call)
            x = torch.randn(tokens, cols, device="cuda", generator=g)
            y_ref = torch.full((tokens, rows), float("nan"), device="cuda")
            y_new = torch.full((tokens, rows), float("nan"), device="cuda")
            torch.cuda.synchronize()
            ex.matmul_device(m, tokens, x.data_ptr(), y_ref.data_ptr(), 0)
            rc = L.llr_gemm_device_noalloc(ex._h, m._h, tokens, x.data_ptr(), y_new.data_ptr(), None)
            assert rc == 0, L.llr_exec_last_error(ex._h).decode()
            ex.synchronize()
            assert torch.isfinite(y_new).all()
            # same kernels, same arithmetic: bit-identical (the GEMM's own tolerance against the
            # CPU reference is asserted in tests/test_gpu_gemm.py)
            assert torch.equal(y_new, y_ref), f"dtype {dtype} call {call}"
        m.free()
    # the call path allocates nothing: free device memory is the same after two more calls of a new, larger shape
    m = ex.synth(Q4_K, 512, 4096, 13)
    x = torch.randn(300, 4096, device="cuda")
    y = torch.empty(300, 512, device="cuda")
    torch.cuda.synchronize()
    free0 = torch.cuda.mem_get_info()[0]
    for _ in range(2):
        assert L.llr_gemm_device_noalloc(ex._h, m._h, 300, x.data_ptr(), y.data_ptr(), None) == 0
    ex.synchronize()
    assert torch.cuda.mem_get_info()[0] == free0
    m.free()
    # columns that are not a multiple of 256 are rejected
    odd = ex.synth(Q8_0, 128, 2048 + 32, 14)
    xo = torch.zeros(64, 2048 + 32, device="cuda")
    yo = torch.full((64, 128), 7.0, device="cuda")
    assert L.llr_gemm_device_noalloc(ex._h, odd._h, 64, xo.data_ptr(), yo.data_ptr(), None) == 1
    ex.synchronize()
    assert bool((yo == 7.0).all())
    odd.free()
    # beyond the built-in staging area: a clear error, nothing launched, output untouched
    big = ex.synth(Q4_K, 128, 16384, 5)
    tokens = 1100  # 1100 * 16384 * 2 = 36 MB > 32 MiB
    x = torch.zeros(tokens, 16384, device="cuda")
    y = torch.full((tokens, 128), 7.0, device="cuda")
    rc = L.llr_gemm_device_noalloc(ex._h, big._h, tokens, x.data_ptr(), y.data_ptr(), None)
    assert rc == 1 and "exceeds the built-in staging area" in L.llr_exec_last_error(ex._h).decode()
    ex.synchronize()
    assert bool((y == 7.0).all())
    # formats the tensor-core GEMM does not take are rejected, not rerouted
    f16 = ex.synth(0, 128, 2048, 6)  # F16 weights have no tensor-core routine
    rc = L.llr_gemm_device_noalloc(ex._h, f16._h, 64, x.data_ptr(), y.data_ptr(), None)
    assert rc == 1
    big.free()
    f16.free()
    ex.close()
