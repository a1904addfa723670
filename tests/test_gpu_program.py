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
    ex = Executor(0)
    m = ex.synth(Q4_K, 64, 4096, 1)          # this rank's 64 rows of a 128-row matrix
    x = torch.zeros(4096, device="cuda")
    arena_bytes = ARENA_HEADER_BYTES + 4 * 128
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
    with pytest.raises(NativeCudaError):  # result slice inside the library's header
        ex.sharded_program([(m, x.data_ptr(), arena, 1, 0)], [128], arena, arena_bytes, 2, 0, [None, other])
    with pytest.raises(NativeCudaError):  # leading dimension smaller than the shard
        ex.sharded_program([(m, x.data_ptr(), y, 1, 0)], [32], arena, arena_bytes, 2, 0, [None, other])
    ex.shared_free(other)
    ex.shared_free(arena)
    ex.close()
