"""Programs: a list of decode products, phases chained through device buffers, run by one
persistent launch (llr_program_*).  Every product is checked against the CPU row kernels
applied to the activations the device actually used."""
import numpy as np
import pytest

from helpers import Q4_K, Q6_K, Q8_0, check_gemv, gemv_references

pytestmark = pytest.mark.gpu


def _chain(ex, torch, tokens, seeds):
    from llama_rust_b200 import synth
    shapes = [  # name, dtype, rows, cols, phase, input
        ("q", Q4_K, 512, 4096, 0, "x0"), ("k", Q4_K, 136, 4096, 0, "x0"), ("v", Q6_K, 128, 4096, 0, "x0"),
        ("o", Q4_K, 4096, 512, 1, "q"),
        ("gate", Q4_K, 2048, 4096, 2, "o"), ("up", Q8_0, 1000, 4096, 2, "o"),
        ("down", Q6_K, 4096, 2048, 3, "gate"),
        ("head", Q8_0, 777, 4096, 4, "down"),
    ]
    mats, bufs = {}, {"x0": torch.zeros(tokens, 4096, device="cuda")}
    for name, dt, rows, cols, phase, src in shapes:
        mats[name] = ex.synth(dt, rows, cols, seeds + hash(name) % 1000)
        bufs[name] = torch.full((tokens, rows), float("nan"), device="cuda")
    entries = [(mats[n], bufs[src].data_ptr(), bufs[n].data_ptr(), tokens, ph) for n, _, _, _, ph, src in shapes]
    return shapes, mats, bufs, entries


@pytest.mark.parametrize("tokens", [1, 2, 5])
def test_program_matches_cpu_row_kernels_stage_by_stage(orc, tokens):
    import torch
    from llama_rust_b200 import Executor, synth
    ex = Executor(0)
    shapes, mats, bufs, entries = _chain(ex, torch, tokens, 4000)
    prog = ex.program(entries)
    stream = torch.cuda.Stream()
    for run in range(3):  # the phase counters carry over from run to run
        x0 = synth.activations(tokens * 4096, 100 + run).reshape(tokens, 4096) * np.float32(0.05)
        bufs["x0"].copy_(torch.from_numpy(x0))
        torch.cuda.synchronize()
        prog.run(stream.cuda_stream)
        ex.synchronize()
        stream.synchronize()
        for name, dt, rows, cols, phase, src in shapes:
            x = bufs[src].cpu().numpy().reshape(-1)
            y = bufs[name].cpu().numpy().reshape(-1)
            w = ex.download(mats[name])
            cpu, exact, abs_sum = gemv_references(dt, rows, cols, w, x, tokens)
            check_gemv(y, cpu, exact, abs_sum, cols, f"program {name} M={tokens} run {run}")
    # the same products through single calls give the same bits (same kernels' arithmetic)
    y_single = torch.empty_like(bufs["q"])
    ex.matmul_device(mats["q"], tokens, bufs["x0"].data_ptr(), y_single.data_ptr(), stream.cuda_stream)
    stream.synchronize()
    assert torch.equal(y_single, bufs["q"])
    prog.free()
    ex.close()


def test_program_rejects_what_it_cannot_run():
    import torch
    from llama_rust_b200 import Executor, NativeCudaError
    from helpers import F32
    ex = Executor(0)
    m = ex.synth(Q4_K, 64, 4096, 1)
    f = ex.synth(F32, 64, 4096, 1)
    x = torch.zeros(4096, device="cuda")
    y = torch.zeros(64, device="cuda")
    with pytest.raises(NativeCudaError):
        ex.program([(f, x.data_ptr(), y.data_ptr(), 1, 0)])
    with pytest.raises(NativeCudaError):
        ex.program([(m, x.data_ptr(), y.data_ptr(), 9, 0)])
    with pytest.raises(NativeCudaError):
        ex.program([(m, x.data_ptr(), y.data_ptr(), 1, 1), (m, x.data_ptr(), y.data_ptr(), 1, 0)])
    other = Executor(0)
    with pytest.raises(NativeCudaError) as e:
        other.program([(m, x.data_ptr(), y.data_ptr(), 1, 0)])
    assert e.value.code == 5
    other.close()
    ex.close()


def test_sharded_program_validation_on_one_gpu():
    """The argument checks of llr_program_create_sharded and the shared-arena calls need no second GPU."""
    import torch
    from llama_rust_b200 import Executor, NativeCudaError
    from llama_rust_b200._lib import ARENA_HEADER_BYTES
    from llama_rust_b200.sharding import arena_layout
    ex = Executor(0)
    m = ex.synth(Q4_K, 64, 4096, 1)          # this rank's 64 rows of a 128-row matrix
    x = torch.zeros(4096, device="cuda")
    _, arena_bytes = arena_layout([128])     # header | results | tagged copies
    arena, handle = ex.shared_alloc(arena_bytes)
    assert len(handle) == 64 and arena % 256 == 0
    other, _ = ex.shared_alloc(arena_bytes)  # stands in for the peer's arena (same process: no IPC open needed)
    y = arena + ARENA_HEADER_BYTES
    ok = ex.sharded_program([(m, x.data_ptr(), y, 1, 0)], [128], arena, arena_bytes, 2, 0, [None, other])
    ok.free()
    bad = [
        dict(world=1, rank=0, peers=[None]),                       # a sharded program needs at least two ranks
        dict(world=9, rank=0, peers=[None] + [other] * 8),         # at most eight
        dict(world=2, rank=2, peers=[None, other]),                # rank out of range
        dict(world=2, rank=0, peers=[None, None]),                 # missing peer arena
    ]
    for kw in bad:
        with pytest.raises(NativeCudaError):
            ex.sharded_program([(m, x.data_ptr(), y, 1, 0)], [128], arena, arena_bytes, kw["world"], kw["rank"], kw["peers"])
    with pytest.raises(NativeCudaError):  # result slice outside the arena
        ex.sharded_program([(m, x.data_ptr(), arena + arena_bytes - 64, 1, 0)], [128], arena, arena_bytes, 2, 0, [None, other])
    with pytest.raises(NativeCudaError):  # result slice in the part of the arena that holds the tagged copies
        ex.sharded_program([(m, x.data_ptr(), y + 512, 1, 0)], [128], arena, arena_bytes, 2, 0, [None, other])
    with pytest.raises(NativeCudaError):  # result slice inside the library's header
        ex.sharded_program([(m, x.data_ptr(), arena, 1, 0)], [128], arena, arena_bytes, 2, 0, [None, other])
    with pytest.raises(NativeCudaError):  # leading dimension smaller than the shard
        ex.sharded_program([(m, x.data_ptr(), y, 1, 0)], [32], arena, arena_bytes, 2, 0, [None, other])
    ex.shared_free(other)
    ex.shared_free(arena)
    ex.close()


def _model_chain(ex, torch, tokens, seed, n_embd=4096, n_kv=256, n_ff=4096):
    """Two transformer-shaped blocks as the walk chains its products (decode.rs:2737-3097), attention replaced by
    the q result as a stand-in: rmsnorm(h) -> q|k|v; q -> o, + h; rmsnorm -> gate|up; silu(gate)*up -> down, + h'."""
    from llama_rust_b200 import XOP_NONE, XOP_RMSNORM, XOP_SWIGLU
    rng = np.random.default_rng(seed)
    bufs = {"h0": torch.zeros(tokens, n_embd, device="cuda")}
    norm = {}
    ops, meta = [], []
    phase = 0
    h = "h0"

    def add(name, dt, rows, cols, x, x_op=XOP_NONE, x2=None, resid=None, w=None):
        m = ex.synth(dt, rows, cols, seed + len(meta))
        bufs[name] = torch.full((tokens, rows), float("nan"), device="cuda")
        ops.append(dict(matrix=m, x=bufs[x].data_ptr(), x2=(w.data_ptr() if w is not None else (bufs[x2].data_ptr() if x2 else None)),
                        resid=bufs[resid].data_ptr() if resid else None, y=bufs[name].data_ptr(), tokens=tokens, phase=phase,
                        x_op=x_op, eps=1e-5))
        meta.append((name, dt, rows, cols, x, x_op, x2, resid, w, m))
    for layer in range(2):
        wa = torch.from_numpy((1.0 + 0.1 * rng.standard_normal(n_embd)).astype(np.float32)).cuda()
        wf = None if layer == 0 else torch.from_numpy((1.0 + 0.1 * rng.standard_normal(n_embd)).astype(np.float32)).cuda()
        norm[layer] = (wa, wf)
        for nm, dt, rows in (("q", Q4_K, n_embd), ("k", Q4_K, n_kv), ("v", Q6_K, n_kv)):
            add(f"{nm}{layer}", dt, rows, n_embd, h, XOP_RMSNORM, w=wa)
        phase += 1
        add(f"o{layer}", Q4_K, n_embd, n_embd, f"q{layer}", resid=h)
        phase += 1
        add(f"gate{layer}", Q4_K, n_ff, n_embd, f"o{layer}", XOP_RMSNORM, w=wf)
        add(f"up{layer}", Q8_0, n_ff, n_embd, f"o{layer}", XOP_RMSNORM, w=wf)
        phase += 1
        add(f"down{layer}", Q6_K, n_embd, n_ff, f"gate{layer}", XOP_SWIGLU, x2=f"up{layer}", resid=f"o{layer}")
        phase += 1
        h = f"down{layer}"
    return bufs, ops, meta


@pytest.mark.parametrize("tokens", [1, 3])
def test_program_with_fused_rmsnorm_swiglu_residual_matches_cpu(orc, tokens):
    """Every product of a chain whose element-wise steps run inside the launch is checked against the CPU:
    the reference's rmsnorm / silu (oracle) applied to the buffers the device produced, then the CPU row kernels."""
    import torch
    from llama_rust_b200 import Executor, synth, XOP_RMSNORM, XOP_SWIGLU
    ex = Executor(0)
    bufs, ops, meta = _model_chain(ex, torch, tokens, 7000)
    prog = ex.program_ops(ops)
    info = prog.info()
    assert info["counter_phases"] == 0 and info["phases"] == 8, info
    stream = torch.cuda.Stream()
    for run in range(2):
        h0 = synth.activations(tokens * 4096, 300 + run).reshape(tokens, 4096)
        bufs["h0"].copy_(torch.from_numpy(h0))
        torch.cuda.synchronize()
        prog.run(stream.cuda_stream)
        ex.synchronize()
        stream.synchronize()
        host = {k: v.cpu().numpy() for k, v in bufs.items()}
        for name, dt, rows, cols, x, x_op, x2, resid, w, m in meta:
            xin = host[x].astype(np.float32)
            if x_op == XOP_RMSNORM:
                wv = np.ones(cols, np.float32) if w is None else w.cpu().numpy()
                xin = np.stack([orc.rmsnorm(xin[t], wv, 1e-5) for t in range(tokens)])
            elif x_op == XOP_SWIGLU:
                xin = np.stack([orc.silu(xin[t]) * host[x2][t] for t in range(tokens)]).astype(np.float32)
            wp = ex.download(m)
            cpu, exact, abs_sum = gemv_references(dt, rows, cols, wp, xin.reshape(-1), tokens)
            if resid:
                r = host[resid].astype(np.float64)
                cpu = (cpu.reshape(tokens, rows) + host[resid]).astype(np.float32)
                exact = exact + r
                abs_sum = abs_sum + np.abs(r)
            check_gemv(host[name].reshape(-1), cpu, exact, abs_sum, cols, f"fused {name} M={tokens} run {run}")
    prog.free()
    ex.close()


def test_strict_program_falls_back_to_phase_counters_for_inputs_it_cannot_trace(orc):
    """llr_program_create: an input that is only part of an earlier result with several activation rows cannot
    travel as tagged pairs; its phase then waits for the previous phase's counter and the results are the same."""
    import torch
    from llama_rust_b200 import Executor, synth
    tokens = 2
    ex = Executor(0)
    a = ex.synth(Q4_K, 512, 1024, 1)
    b = ex.synth(Q8_0, 64, 256, 2)
    x0 = torch.from_numpy(synth.activations(tokens * 1024, 5).reshape(tokens, 1024) * np.float32(0.1)).cuda()
    ya = torch.full((tokens, 512), float("nan"), device="cuda")
    yb = torch.full((tokens, 64), float("nan"), device="cuda")
    # b reads 2 x 256 consecutive floats starting at ya: for two activation rows that is not a result's layout
    prog = ex.program([(a, x0.data_ptr(), ya.data_ptr(), tokens, 0), (b, ya.data_ptr(), yb.data_ptr(), tokens, 1)])
    assert prog.info()["counter_phases"] == 1
    for run in range(3):
        prog.run()
        ex.synchronize()
        xa = ya.cpu().numpy().reshape(-1)[: tokens * 256]
        cpu, exact, abs_sum = gemv_references(Q8_0, 64, 256, ex.download(b), xa, tokens)
        check_gemv(yb.cpu().numpy().reshape(-1), cpu, exact, abs_sum, 256, f"counter phase run {run}")
    prog.free()
    ex.close()


def test_wait_that_runs_out_is_reported_and_the_executor_stays_usable(orc):
    """A sharded program whose peer never runs: the reader's bounded wait for the peer's half of a result runs out,
    the launch still finishes, llr_exec_synchronize reports it, and the executor then serves a normal product
    (native-cuda/src/main.rs:48-66: the executor stays usable after an error).  Nothing faults or hangs: the
    wait is a bounded poll of device memory that nobody writes."""
    import time
    import torch
    from llama_rust_b200 import Executor, NativeCudaError, synth
    from llama_rust_b200.sharding import arena_layout
    ex = Executor(0)
    ex.set_wait_limit(2000)
    a = ex.synth(Q4_K, 128, 1024, 1)   # this rank's half of a 256-row product
    b = ex.synth(Q4_K, 64, 256, 2)     # reads all 256 values: half of them would come from the peer
    c = ex.synth(Q4_K, 64, 256, 3)     # a later phase: its wait must return at once
    x0 = torch.from_numpy(synth.activations(1024, 5) * np.float32(0.1)).cuda()
    offs, arena_bytes = arena_layout([256, 128, 128])
    arena, _ = ex.shared_alloc(arena_bytes)
    absent, _ = ex.shared_alloc(arena_bytes)  # stands in for the arena of a rank that never launches
    ops = [dict(matrix=a, x=x0.data_ptr(), y=arena + offs[0], y_ld=256, tokens=1, phase=0),
           dict(matrix=b, x=arena + offs[0], y=arena + offs[1], y_ld=128, tokens=1, phase=1),
           dict(matrix=c, x=arena + offs[0], y=arena + offs[2], y_ld=128, tokens=1, phase=2)]
    prog = ex.program_ops(ops, (arena, arena_bytes, 2, 0, [None, absent]))
    t0 = time.perf_counter()
    prog.run()
    with pytest.raises(NativeCudaError) as e:
        ex.synchronize()
    assert e.value.code == 6 and "wait" in str(e.value)
    assert time.perf_counter() - t0 < 5.0
    prog.free()
    ex.shared_free(absent)
    ex.shared_free(arena)
    # the executor still works
    x = synth.activations(1024, 9)
    y = np.empty(128, np.float32)
    ex.gemm_resident(a, 1, x, y)
    cpu, exact, abs_sum = gemv_references(Q4_K, 128, 1024, ex.download(a), x, 1)
    check_gemv(y, cpu, exact, abs_sum, 1024, "after a failed wait")
    ex.synchronize()
    ex.close()


def test_program_recreated_on_a_used_arena_starts_clean(orc):
    """A second program on an arena that an earlier program ran on must not take the earlier program's tags for
    its own.  One rank of a two-rank layout whose reader needs only this rank's half of the result, so that no peer
    has to run; the input changes between runs, so a stale value that passed for a new one would show."""
    import ctypes as C
    import torch
    from llama_rust_b200 import Executor, synth
    from llama_rust_b200.sharding import arena_layout
    rt = C.CDLL("libcudart.so.12")
    rt.cudaMemcpy.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t, C.c_int]
    ex = Executor(0)
    a = ex.synth(Q4_K, 256, 1024, 1)   # rows 0..255 of a 512-row product
    b = ex.synth(Q4_K, 64, 256, 2)     # reads values 0..255: all produced here
    x0 = torch.zeros(1024, device="cuda")
    offs, arena_bytes = arena_layout([512, 128, 128])
    arena, _ = ex.shared_alloc(arena_bytes)
    other, _ = ex.shared_alloc(arena_bytes)
    seed = 0
    for generation in range(3):  # same arena, three programs one after the other, a different number of phases each
        ops = [dict(matrix=a, x=x0.data_ptr(), y=arena + offs[0], y_ld=512, tokens=1, phase=0)]
        for k in range(1 + generation):
            ops.append(dict(matrix=b, x=arena + offs[0], y=arena + offs[1 + k % 2], y_ld=128, tokens=1, phase=1 + k))
        prog = ex.program_ops(ops, (arena, arena_bytes, 2, 0, [None, other]))
        assert prog.info()["counter_phases"] == 0
        for run in range(2):
            seed += 1
            x0.copy_(torch.from_numpy(synth.activations(1024, seed) * np.float32(0.1)))
            torch.cuda.synchronize()
            prog.run()
            ex.synchronize()
            xa, yb = np.empty(256, np.float32), np.empty(64, np.float32)
            assert rt.cudaMemcpy(xa.ctypes.data, arena + offs[0], 1024, 2) == 0
            cpu, exact, abs_sum = gemv_references(Q4_K, 256, 1024, ex.download(a), x0.cpu().numpy(), 1)
            check_gemv(xa, cpu, exact, abs_sum, 1024, f"generation {generation} run {run} first product")
            for k in range(1 + generation):
                assert rt.cudaMemcpy(yb.ctypes.data, arena + offs[1 + k % 2], 256, 2) == 0
                cpu, exact, abs_sum = gemv_references(Q4_K, 64, 256, ex.download(b), xa, 1)
                check_gemv(yb, cpu, exact, abs_sum, 256, f"generation {generation} run {run} reader {k}")
        prog.free()
    ex.shared_free(other)
    ex.shared_free(arena)
    ex.close()
