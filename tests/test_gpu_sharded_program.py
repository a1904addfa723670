"""Row-sharded programs on two GPUs (one process per GPU): the reducer's peer stores and the
phase counters counted over both ranks replace the all-gather.  Every rank must end up with
the complete result vectors, bit-identical to the unsharded program on one GPU, also for
phases whose input is a vector that the other rank helped to write.  Skipped with fewer than
two GPUs.  The control plane (exchange of memory handles, barriers) is a gloo group."""
import ctypes as C
import os
import socket

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

Q4_K, Q6_K, Q8_0 = 17, 19, 13
SHAPES = [  # name, dtype, full rows, cols, phase, input (None = x0)
    ("a", Q4_K, 2048, 1024, 0, None), ("b", Q8_0, 1024, 1024, 0, None),
    ("c", Q6_K, 512, 2048, 1, "a"),
    ("d", Q4_K, 1024, 512, 2, "c"), ("e", Q8_0, 256, 512, 2, "c"),
]


def _d2h(ptr, n_floats):
    rt = C.CDLL("libcudart.so.12")
    rt.cudaMemcpy.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t, C.c_int]
    out = np.empty(n_floats, np.float32)
    assert rt.cudaMemcpy(out.ctypes.data, ptr, 4 * n_floats, 2) == 0
    return out


def _worker(rank, world, port, tokens, ret):
    try:
        import torch
        import torch.distributed as dist
        from llama_rust_b200 import Executor, synth
        from llama_rust_b200.sharding import ShardedDecodeProgram, shard_packed
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
        dist.init_process_group("gloo", rank=rank, world_size=world)
        torch.cuda.set_device(rank)
        ex = Executor(rank)
        packed = {n: synth.packed_matrix(dt, rows, cols, 900 + i) for i, (n, dt, rows, cols, _, _) in enumerate(SHAPES)}
        x0 = torch.from_numpy(synth.activations(tokens * 1024, 7).reshape(tokens, 1024) * np.float32(0.05)).cuda()
        # unsharded reference on this GPU
        full = {n: ex.upload(dt, rows, cols, packed[n]) for n, dt, rows, cols, _, _ in SHAPES}
        ref = {n: torch.full((tokens, rows), float("nan"), device="cuda") for n, _, rows, _, _, _ in SHAPES}
        prog1 = ex.program([(full[n], (x0 if src is None else ref[src]).data_ptr(), ref[n].data_ptr(), tokens, ph)
                            for n, _, _, _, ph, src in SHAPES])
        # sharded
        shards = {}
        for n, dt, rows, cols, _, _ in SHAPES:
            b, r = shard_packed(packed[n], rows, world, rank)
            shards[n] = ex.upload(dt, r, cols, np.ascontiguousarray(b))
        idx = {n: i for i, (n, *_rest) in enumerate(SHAPES)}
        from llama_rust_b200.sharding import arena_layout
        offs, _ = arena_layout([rows for _, _, rows, _, _, _ in SHAPES], tokens)
        # inputs: x0, or the producing entry's full-width buffer in the local arena
        specs2 = [(shards[n], (lambda arena, src=src: x0.data_ptr() if src is None else arena + offs[idx[src]]), rows, ph)
                  for n, _, rows, _, ph, src in SHAPES]
        sp = ShardedDecodeProgram(ex, specs2, tokens)
        stream = torch.cuda.Stream()
        ok = True
        for run in range(3):
            x0.copy_(torch.from_numpy(synth.activations(tokens * 1024, 7 + run).reshape(tokens, 1024) * np.float32(0.05)))
            torch.cuda.synchronize()
            dist.barrier()
            prog1.run(stream.cuda_stream)
            sp.run(stream.cuda_stream)
            ex.synchronize()
            stream.synchronize()
            dist.barrier()  # the other rank's stores into this arena are complete as well
            for i, (n, _, rows, _, _, _) in enumerate(SHAPES):
                got = _d2h(sp.y_ptr(i), tokens * rows)
                want = ref[n].cpu().numpy().reshape(-1)
                if not np.array_equal(got, want):
                    ok = False
                    ret[rank] = f"run {run} result {n}: {int((got != want).sum())} of {got.size} differ"
                    break
            if not ok:
                break
        sp.close()
        prog1.free()
        ex.close()
        dist.destroy_process_group()
        if ok:
            ret[rank] = "ok"
    except Exception as e:  # noqa: BLE001
        import traceback
        ret[rank] = f"{type(e).__name__}: {e}\n{traceback.format_exc()}"


@pytest.mark.parametrize("tokens", [1, 3])
def test_sharded_program_equals_unsharded_on_every_rank(tokens):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, tokens, ret)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(300)
    for p in procs:
        if p.is_alive():
            p.terminate()
    assert dict(ret) == {0: "ok", 1: "ok"}, dict(ret)


def _moe_worker(rank, world, port, ret):
    try:
        import torch
        import torch.distributed as dist
        from llama_rust_b200 import Executor
        from llama_rust_b200.sharding import ExpertParallelLayer, home_rank
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
        torch.cuda.set_device(rank)
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
        ex = Executor(rank)
        F32 = 2
        n_expert, n_used, n_embd, n_ff = 8, 2, 1024, 2048
        # every rank builds all experts here (to have the single-device answer); a deployment keeps only its own
        gate = [ex.synth(Q4_K, n_ff, n_embd, 10 + e) for e in range(n_expert)]
        up = [ex.synth(Q4_K, n_ff, n_embd, 30 + e) for e in range(n_expert)]
        down = [ex.synth(Q4_K, n_embd, n_ff, 50 + e) for e in range(n_expert)]
        rng = np.random.default_rng(3)
        router = ex.upload(F32, n_expert, n_embd, (rng.standard_normal((n_expert, n_embd)) * 0.05).astype(np.float32).view(np.uint8).reshape(-1))
        keep = [home_rank(e, world) == rank for e in range(n_expert)]
        route, experts = ExpertParallelLayer.cuda_backend(ex, router, [m if k else None for m, k in zip(gate, keep)],
                                                          [m if k else None for m, k in zip(up, keep)],
                                                          [m if k else None for m, k in zip(down, keep)], n_used, True)
        layer = ExpertParallelLayer(n_expert, n_used, route, experts)
        ok = "ok"
        # f32-faithful products (path 3): a row's result does not depend on its batch, so the outputs must be the same
        # bits.  Automatic choice (path 0): the kernel family follows the number of rows an expert gets, which differs
        # between the sharded and the single-device call, so the 16-bit tensor-core tolerance applies.
        for path, tokens in ((3, 7), (3, 128), (3, 600), (0, 128), (0, 600)):
            ex.set_path(path)
            x = rng.standard_normal((tokens, n_embd)).astype(np.float32)      # the same on every rank (same seed)
            lo, hi = tokens * rank // world, tokens * (rank + 1) // world    # this rank's tokens
            full, ids, w = ex.moe_ffn(router, gate, up, down, n_used, True, x[lo:hi])  # single-device answer for them
            out, ids_s, w_s = layer(torch.from_numpy(np.ascontiguousarray(x[lo:hi])).cuda())
            torch.cuda.synchronize()
            got = out.cpu().numpy()
            if not (np.array_equal(ids_s.cpu().numpy(), ids) and np.array_equal(w_s.cpu().numpy(), w)):
                ok = f"path {path} tokens={tokens}: routing differs"
                break
            if path == 3 and not np.array_equal(got, full):
                ok = f"path {path} tokens={tokens}: expert-parallel result differs in {int((got != full).sum())} of {got.size} values, max {np.abs(got - full).max()}"
                break
            if path == 0 and not np.abs(got - full).max() <= 2e-2 * max(1.0, np.abs(full).max()):
                ok = f"path {path} tokens={tokens}: outside the tensor-core tolerance, max {np.abs(got - full).max()}"
                break
        ex.close()
        dist.barrier()
        dist.destroy_process_group()
        ret[rank] = ok
    except Exception as e:  # noqa: BLE001
        import traceback
        ret[rank] = f"{type(e).__name__}: {e}\n{traceback.format_exc()}"


def _moe_ep_worker(rank, world, port, ret):
    """The expert-parallel layer whose exchange is peer stores inside the library (llr_moe_ep_*)."""
    try:
        import torch
        import torch.distributed as dist
        from llama_rust_b200 import Executor
        from llama_rust_b200.sharding import PeerExpertParallelLayer, home_rank
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
        torch.cuda.set_device(rank)
        dist.init_process_group("gloo", rank=rank, world_size=world)
        ex = Executor(rank)
        F32 = 2
        n_expert, n_used, n_embd, n_ff = 8, 2, 1024, 2048
        gate = [ex.synth(Q4_K, n_ff, n_embd, 10 + e) for e in range(n_expert)]
        up = [ex.synth(Q4_K, n_ff, n_embd, 30 + e) for e in range(n_expert)]
        down = [ex.synth(Q4_K, n_embd, n_ff, 50 + e) for e in range(n_expert)]
        rng = np.random.default_rng(3)
        router = ex.upload(F32, n_expert, n_embd, (rng.standard_normal((n_expert, n_embd)) * 0.05).astype(np.float32).view(np.uint8).reshape(-1))
        keep = [home_rank(e, world) == rank for e in range(n_expert)]
        layer = PeerExpertParallelLayer(ex, router, [m if k else None for m, k in zip(gate, keep)],
                                        [m if k else None for m, k in zip(up, keep)],
                                        [m if k else None for m, k in zip(down, keep)], n_used, True, 320)
        ok = "ok"
        for path, tokens in ((3, 7), (3, 128), (3, 600), (0, 128), (0, 600), (3, 9)):
            ex.set_path(path)
            x = rng.standard_normal((tokens, n_embd)).astype(np.float32)      # the same on every rank (same seed)
            lo, hi = tokens * rank // world, tokens * (rank + 1) // world    # this rank's tokens
            full, ids, w = ex.moe_ffn(router, gate, up, down, n_used, True, x[lo:hi])  # single-device answer for them
            dist.barrier()  # ranks enter a run together: the device-side waits are bounded
            out, ids_s, w_s = layer(torch.from_numpy(np.ascontiguousarray(x[lo:hi])).cuda())
            got = out.cpu().numpy()
            if not (np.array_equal(ids_s.cpu().numpy(), ids) and np.array_equal(w_s.cpu().numpy(), w)):
                ok = f"path {path} tokens={tokens}: routing differs"
                break
            if path == 3 and not np.array_equal(got, full):
                ok = f"path {path} tokens={tokens}: expert-parallel result differs in {int((got != full).sum())} of {got.size} values, max {np.abs(got - full).max()}"
                break
            if path == 0 and not np.abs(got - full).max() <= 2e-2 * max(1.0, np.abs(full).max()):
                ok = f"path {path} tokens={tokens}: outside the tensor-core tolerance, max {np.abs(got - full).max()}"
                break
        dist.barrier()
        layer.close()
        ex.close()
        dist.barrier()
        dist.destroy_process_group()
        ret[rank] = ok
    except Exception as e:  # noqa: BLE001
        import traceback
        ret[rank] = f"{type(e).__name__}: {e}\n{traceback.format_exc()}"


def _spawn(world, target, *args):
    import torch.multiprocessing as mp
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    procs = [ctx.Process(target=target, args=(r, world, port, *args, ret)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(300)
    for p in procs:
        if p.is_alive():
            p.terminate()
    return dict(ret)


def test_expert_parallel_layer_over_two_gpus_equals_the_single_device_layer():
    """Tokens sharded, experts striped e % 2, routed rows exchanged with NCCL all-to-all."""
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    assert _spawn(2, _moe_worker) == {0: "ok", 1: "ok"}


def test_expert_parallel_layer_on_one_rank_equals_the_layer_call():
    """The same code path with a group of one rank: no second GPU needed (the all-to-all is then a local copy)."""
    assert _spawn(1, _moe_worker) == {0: "ok"}


def test_expert_parallel_layer_with_peer_stores_over_two_gpus():
    """Tokens sharded, experts striped e % 2, routed rows and results moved by peer stores from the library's own
    kernels; bit-identical to the single-device layer on the f32-faithful path."""
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    assert _spawn(2, _moe_ep_worker) == {0: "ok", 1: "ok"}


def test_one_process_drives_executors_on_two_devices():
    """Executors of two devices in ONE process (one thread driving several ranks, as the expert-parallel stages allow):
    kernels are set up per device (shared-memory limits and occupancy belong to a device's context), so the second
    device runs every kernel family and returns the same bits as the first."""
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    from helpers import random_packed
    from llama_rust_b200 import Executor
    rng = np.random.default_rng(2024)
    cases = []  # path, kind, rows, cols, tokens, packed weights, activations
    for path, kind, rows, cols, tokens in ((3, Q4_K, 64, 4096, 1), (3, Q6_K, 32, 2048, 3), (3, Q8_0, 48, 2048, 1), (2, Q4_K, 64, 4096, 1),
                                           (2, Q8_0, 48, 2048, 3), (1, Q6_K, 32, 2048, 1), (0, Q4_K, 128, 4096, 64), (0, Q8_0, 128, 2048, 64)):
        cases.append((path, kind, rows, cols, tokens, random_packed(rng, kind, rows, cols),
                      rng.standard_normal(tokens * cols).astype(np.float32)))
    got = []
    for dev in (0, 1):
        with Executor(dev) as ex:
            mine = []
            for path, kind, rows, cols, tokens, w, x in cases:
                ex.set_path(path)
                m = ex.upload(kind, rows, cols, w)
                y = np.full(rows * tokens, np.nan, np.float32)
                ex.gemm_resident(m, tokens, x, y)
                assert np.all(np.isfinite(y)), (dev, path, kind)
                mine.append(y)
                m.free()
            got.append(mine)
    for a, b, case in zip(got[0], got[1], cases):
        assert np.array_equal(a.view(np.uint32), b.view(np.uint32)), case[:5]
