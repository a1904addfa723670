"""Host logic of the sharding layer on CPU: two gloo ranks, the oracle standing in for the
device executor.  Row-sharded products must reproduce the unsharded result bit for bit
(rows are independent), and the expert-parallel layer (tokens sharded, routed rows exchanged with
all-to-all) must match the single-process MoE walk."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from helpers import F32, Q4_K, Q6_K, random_packed


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, fn, args, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        ret[rank] = fn(rank, world, *args)
    finally:
        dist.destroy_process_group()


def _run(world, fn, *args):
    ctx = mp.get_context("spawn")
    mgr = ctx.Manager()
    ret = mgr.dict()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, fn, args, ret)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    return [ret[r] for r in range(world)]


def _dense_rank(rank, world, kind, rows, cols, w, x):
    from llama_rust_b200 import sharding
    from oracle import pyoracle as orc
    shard, local_rows = sharding.shard_packed(w, rows, world, rank)
    tokens = x.shape[0]
    mm = sharding.RowShardedMatmul(rows, lambda xt: torch.from_numpy(
        orc.gemm(kind, cols, tokens, shard, xt.numpy(), local_rows, simd=True, threads=1)))
    return mm(torch.from_numpy(x)).numpy()


@pytest.mark.parametrize("kind,rows,cols", [(Q4_K, 64, 512), (Q6_K, 48, 2048)])
def test_row_sharded_product_is_bit_identical_to_unsharded(orc, kind, rows, cols):
    rng = np.random.default_rng(77)
    w = random_packed(rng, kind, rows, cols)
    x = rng.standard_normal((3, cols)).astype(np.float32)
    full = orc.gemm(kind, cols, 3, w, x, rows, simd=True, threads=1)
    for y in _run(2, _dense_rank, kind, rows, cols, w, x):
        assert np.array_equal(y.view(np.uint32), full.view(np.uint32))


def test_row_ranges_cover_baseline_shapes():
    from llama_rust_b200 import sharding
    for rows in (4096, 1024, 14336, 128256):
        for world in (1, 2, 4, 8):
            spans = [sharding.row_range(rows, world, r) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == rows
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            assert len({b - a for a, b in spans}) == 1
    assert [sharding.home_rank(e, 4) for e in range(8)] == [0, 1, 2, 3, 0, 1, 2, 3]  # place.rs:71-75


def _moe_rank(rank, world, n_used, gate, up, down, n_embd, n_ff, x, ids, wts):
    """One rank of the expert-parallel layer on CPU tensors: the oracle stands in for the device executor."""
    from llama_rust_b200 import sharding
    from oracle import pyoracle as orc
    tokens = x.shape[0]
    lo, hi = tokens * rank // world, tokens * (rank + 1) // world  # this rank's tokens

    def route(xt):
        return torch.from_numpy(ids[lo:hi].astype(np.int32)), torch.from_numpy(wts[lo:hi])

    def experts(counts, rows):
        out, r0 = [], 0
        for e, n in enumerate(counts):
            n = int(n)
            if n == 0:
                continue
            assert sharding.home_rank(e, world) == rank  # only rows of this rank's experts arrive
            r = rows[r0:r0 + n].numpy()
            g = orc.gemm(Q4_K, n_embd, n, gate[e], r, n_ff, simd=True, threads=1)
            u = orc.gemm(Q4_K, n_embd, n, up[e], r, n_ff, simd=True, threads=1)
            a = np.array([orc.lib.orc_silu(float(v)) for v in g.ravel()], np.float32).reshape(g.shape) * u
            out.append(torch.from_numpy(orc.gemm(Q4_K, n_ff, n, down[e], a, n_embd, simd=True, threads=1)))
            r0 += n
        return torch.cat(out) if out else torch.zeros(0, n_embd)

    layer = sharding.ExpertParallelLayer(len(gate), n_used, route, experts)
    out, _, _ = layer(torch.from_numpy(np.ascontiguousarray(x[lo:hi])))
    return lo, hi, out.numpy()


@pytest.mark.parametrize("tokens", [7, 12])
def test_expert_parallel_layer_matches_single_process_walk(orc, tokens):
    """Tokens sharded over two ranks, experts striped e % 2, routed rows exchanged with all-to-all (gloo): every rank's
    outputs for its own tokens are bit-identical to the single-process layer."""
    rng = np.random.default_rng(5)
    n_expert, n_used, n_embd, n_ff = 4, 2, 256, 256
    router_w = (rng.standard_normal((n_expert, n_embd)) * 0.05).astype(np.float32)
    gate = [random_packed(rng, Q4_K, n_ff, n_embd) for _ in range(n_expert)]
    up = [random_packed(rng, Q4_K, n_ff, n_embd) for _ in range(n_expert)]
    down = [random_packed(rng, Q4_K, n_embd, n_ff) for _ in range(n_expert)]
    x = rng.standard_normal((tokens, n_embd)).astype(np.float32)
    ref, ids, wts = orc.moe_ffn(n_used, True, F32, router_w.view(np.uint8), Q4_K, gate, up, down, n_embd, n_ff, x)
    for lo, hi, out in _run(2, _moe_rank, n_used, gate, up, down, n_embd, n_ff, x, ids, wts):
        # same products per row, same ascending-expert accumulation: identical bits for any number of ranks
        assert np.array_equal(out.view(np.uint32), ref[lo:hi].view(np.uint32))


def test_dispatch_plans_are_consistent():
    from llama_rust_b200 import sharding
    rng = np.random.default_rng(9)
    n_expert, k, world = 8, 2, 4
    per_rank = []
    for r in range(world):
        tokens = 5 + r
        ids = np.stack([rng.permutation(n_expert)[:k] for _ in range(tokens)])
        per_rank.append((ids, *sharding.plan_dispatch(ids, n_expert, world)))
    counts_all = np.stack([p[4] for p in per_rank])
    for r, (ids, src_t, src_j, send_counts, expert_counts) in enumerate(per_rank):
        assert send_counts.sum() == ids.size and np.array_equal(ids[src_t, src_j] % world, np.repeat(np.arange(world), send_counts))
        perm, per_expert = sharding.plan_regroup(counts_all, r, world)
        mine = [e for e in range(n_expert) if e % world == r]
        assert sorted(perm.tolist()) == list(range(int(counts_all[:, mine].sum())))
        assert per_expert.sum() == perm.size and all(per_expert[e] == 0 for e in range(n_expert) if e % world != r)


def _gate_rank(rank, world, port, leave_after, silent):
    """Steps of a two-rank job whose rank 1 leaves between steps (announced, or silently)."""
    import datetime
    from llama_rust_b200.sharding import RankLeft, StepGate
    store = dist.TCPStore("127.0.0.1", port, world, rank == 0, timeout=datetime.timedelta(seconds=30))
    gate = StepGate(store, rank, world, timeout_s=1.0)
    launched = []
    out = None
    for step in range(6):
        if rank == 1 and step == leave_after:
            if not silent:
                gate.leave()
            break
        try:
            gate.enter(step)
        except RankLeft as e:
            out = (e.step, e.left, e.missing)
            break
        launched.append(step)   # the launch of the peer-waiting kernel would stand here
    if rank == 0:
        store.set("done", b"1")
    else:
        store.wait(["done"])     # the store's host outlives its clients
    return launched, out


@pytest.mark.parametrize("silent", [False, True])
def test_a_rank_that_leaves_between_steps_is_seen_before_the_next_launch(silent):
    port = _free_port()
    res = _run(2, _gate_rank, port, 3, silent)
    assert res[1] == ([0, 1, 2], None)
    launched, err = res[0]
    assert launched == [0, 1, 2]                      # no step is launched that the peer does not launch too
    assert err == ((3, [], [1]) if silent else (3, [1], []))
