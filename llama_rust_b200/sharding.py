"""Sharding layer for one multi-GPU box: one process per GPU over torch.distributed.

The reference has no multi-device execution (its only notions are simulated:
`home_gpu = expert % n_gpus`, expertvm/src/place.rs:71-75); this layer is new.

* Dense products shard by OUTPUT ROWS: rows are independent and a row range of a packed
  matrix is a contiguous byte range (langtax/src/decode.rs:10876-10879, `quant_mat_rows`
  :9680-9713), so rank g holds rows [g*R/G, (g+1)*R/G) of every matrix, activations are
  replicated, and the exchange is an all-gather of M x R/G result slices.
* Routed experts stripe as `e % G` and tokens are sharded over the ranks; routed rows travel
  to the expert's rank and back with all-to-all (`ExpertParallelLayer`), and a token's output
  is summed over its experts in ascending expert id (the reference's accumulation order,
  decode.rs:10006-10290), so results do not depend on G.

The compute is a callable, so the same code runs on NCCL with the CUDA executor and on
gloo with any CPU stand-in (that is how the host logic is tested without GPUs).

`ShardedDecodeProgram` is the path that matters for decode: the exchange of result slices is
done by the kernel itself (peer stores + phase counters counted over all ranks), one launch
per rank and step, no collective call between products.  torch.distributed only carries
the 64-byte memory handles at set-up time.
"""
from __future__ import annotations

from typing import Callable, Sequence

import numpy as np
import torch
import torch.distributed as dist


def row_range(rows: int, world: int, rank: int) -> tuple[int, int]:
    """Contiguous, balanced row range of `rank`; exact for every benchmark shape (rows % 8 == 0)."""
    return rows * rank // world, rows * (rank + 1) // world


def shard_packed(packed, rows: int, world: int, rank: int):
    """The byte range of a packed matrix that holds this rank's rows."""
    rb = len(packed) // rows
    r0, r1 = row_range(rows, world, rank)
    return packed[r0 * rb:r1 * rb], r1 - r0


def home_rank(expert: int, world: int) -> int:
    """expertvm/src/place.rs:71-75"""
    return expert % world


class RowShardedMatmul:
    """y[t, :] = W x[t] with W sharded by rows: local product + all-gather of the slices."""

    def __init__(self, rows: int, local_matmul: Callable[[torch.Tensor], torch.Tensor], group=None):
        self.rows, self.local, self.group = rows, local_matmul, group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        if rows % self.world:
            raise ValueError(f"{rows} rows do not split evenly over {self.world} ranks")
        self.local_rows = rows // self.world

    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        y_local = self.local(x)  # [tokens, rows / G]
        tokens = y_local.shape[0]
        gathered = torch.empty(self.world * tokens, self.local_rows, dtype=y_local.dtype, device=y_local.device)
        dist.all_gather_into_tensor(gathered, y_local.contiguous(), group=self.group)
        return gathered.view(self.world, tokens, self.local_rows).permute(1, 0, 2).reshape(tokens, self.rows)


def arena_layout(row_counts: Sequence[int], tokens: int = 1) -> tuple[list[int], int]:
    """Byte offsets of the full-width result buffers inside a rank's arena (behind the library's
    header, 256-byte aligned) and the arena size: header | results | twice as much for the tagged
    copies of the results (see llr_program_create_sharded).  Identical on every rank."""
    from ._lib import ARENA_HEADER_BYTES
    offs, cur = [], ARENA_HEADER_BYTES
    for rows in row_counts:
        offs.append(cur)
        cur += (4 * rows * tokens + 255) // 256 * 256
    return offs, ARENA_HEADER_BYTES + 3 * (cur - ARENA_HEADER_BYTES)


class RankLeft(RuntimeError):
    """A peer announced that it leaves, or did not reach the step in time; nothing was launched."""

    def __init__(self, step: int, left: list[int], missing: list[int]):
        super().__init__(f"step {step}: ranks {left} left, ranks {missing} did not arrive")
        self.step, self.left, self.missing = step, left, missing


class StepGate:
    """Host-side agreement of all ranks before each launch of a kernel that waits on its peers.

    The sharded program's CTAs spin (bounded) on values that peer GPUs store, so a launch must not start unless every
    peer launches the same step.  Each rank posts `step` to a key-value store (torch.distributed's TCPStore or any
    object with set/check) and polls until every rank has posted it; a rank that leaves between steps posts a
    departure mark first, which the others see before their next launch.  A rank that is silent for `timeout_s`
    counts as missing.  Either way `enter` raises RankLeft and the caller still owns a usable executor: no kernel
    of the step ran on this rank."""

    def __init__(self, store, rank: int, world: int, timeout_s: float = 5.0, poll_s: float = 0.002, name: str = "gate"):
        self.store, self.rank, self.world = store, rank, world
        self.timeout_s, self.poll_s, self.name = timeout_s, poll_s, name

    def _key(self, what, rank):
        return f"{self.name}/{what}/{rank}"

    def enter(self, step: int) -> None:
        import time
        self.store.set(self._key(step, self.rank), b"1")
        others = [g for g in range(self.world) if g != self.rank]
        deadline = time.monotonic() + self.timeout_s
        while True:
            waiting = [g for g in others if not self.store.check([self._key(step, g)])]
            if not waiting:
                return
            left = [g for g in waiting if self.store.check([self._key("left", g)])]
            if left or time.monotonic() > deadline:
                raise RankLeft(step, left, [g for g in waiting if g not in left])
            time.sleep(self.poll_s)

    def leave(self) -> None:
        """Call between steps, with none of this rank's kernels in flight."""
        self.store.set(self._key("left", self.rank), b"1")


class ShardedDecodeProgram:
    """One decode step of row-sharded products as a single launch per rank.

    specs: list of (shard_matrix, x, full_rows, phase) or dicts with those keys plus the optional
    x2, resid, x_op, eps of llr_program_op, in execution order; shard_matrix is this rank's resident
    row slice (rows = full_rows / world); x (x2, resid) is a device address, or a callable taking the
    arena's base address (for an input that is an earlier result: arena + its offset from
    arena_layout).  Tuples create a program with strict phases, dicts one whose inputs are either
    results of the program or ready at launch.  Result i lives full width in every rank's arena at
    `self.y_ptr(i)`; after `run()` + a device synchronize on EVERY rank and a host barrier it holds
    the complete vector on every rank."""

    def __init__(self, ex, specs, tokens: int = 1, group=None):
        self.ex, self.group = ex, group
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        as_ops = len(specs) > 0 and isinstance(specs[0], dict)
        if not as_ops:
            specs = [dict(matrix=m, x=x, full_rows=r, phase=p) for m, x, r, p in specs]
        self.offsets, self.arena_bytes = arena_layout([s["full_rows"] for s in specs], tokens)
        self.arena, handle = ex.shared_alloc(self.arena_bytes)
        handles = [None] * self.world
        dist.all_gather_object(handles, handle, group=group)
        self.peers = [None if g == self.rank else ex.shared_open(handles[g]) for g in range(self.world)]

        def addr(v):
            return v(self.arena) if callable(v) else v
        ops = []
        for s, off in zip(specs, self.offsets):
            mat, full_rows = s["matrix"], s["full_rows"]
            r0, r1 = row_range(full_rows, self.world, self.rank)
            if r1 - r0 != mat.rows:
                raise ValueError(f"shard has {mat.rows} rows, rank {self.rank} of {self.world} owns {r1 - r0} of {full_rows}")
            ops.append(dict(matrix=mat, x=addr(s["x"]), x2=addr(s.get("x2")), resid=addr(s.get("resid")),
                            y=self.arena + off + 4 * r0, y_ld=full_rows, tokens=tokens, phase=s["phase"],
                            x_op=s.get("x_op", 0), eps=s.get("eps", 0.0)))
        if as_ops:
            self.program = ex.program_ops(ops, (self.arena, self.arena_bytes, self.world, self.rank, self.peers))
        else:
            self.program = ex.sharded_program([(o["matrix"], o["x"], o["y"], tokens, o["phase"]) for o in ops],
                                              [o["y_ld"] for o in ops], self.arena, self.arena_bytes, self.world,
                                              self.rank, self.peers)
        dist.barrier(group=group)  # every rank has opened every arena and created its program before anybody runs

    def y_ptr(self, i: int) -> int:
        return self.arena + self.offsets[i]

    def run(self, stream: int = 0, gate: StepGate | None = None, step: int = 0) -> None:
        """With a gate, the launch happens only after every rank has reached `step` (else RankLeft, nothing launched)."""
        if gate is not None:
            gate.enter(step)
        self.program.run(stream)

    def close(self) -> None:
        if self.program is not None:
            self.ex.synchronize()
            dist.barrier(group=self.group)  # nobody still stores into an arena that is about to go
            self.program.free()
            self.program = None
            for p in self.peers:
                if p:
                    self.ex.shared_close(p)
            dist.barrier(group=self.group)
            self.ex.shared_free(self.arena)


def plan_dispatch(ids, n_expert: int, world: int):
    """Host side of the token-row exchange.  ids: [T, k] expert ids of this rank's tokens (numpy).  Rows travel to the
    rank that owns their expert (home_rank) ordered by (destination, expert, token), which is also the order they come
    back in.  Returns (src_token[n_rows], src_slot[n_rows], send_counts[world], expert_counts[n_expert])."""
    ids = np.asarray(ids)
    tokens, k = ids.shape
    flat_e = ids.reshape(-1).astype(np.int64)
    flat_t = np.repeat(np.arange(tokens, dtype=np.int64), k)
    flat_j = np.tile(np.arange(k, dtype=np.int64), tokens)
    dest = flat_e % world
    order = np.lexsort((flat_t, flat_e, dest))  # by destination, then expert, then token
    send_counts = np.bincount(dest, minlength=world).astype(np.int64)
    expert_counts = np.bincount(flat_e, minlength=n_expert).astype(np.int64)
    return flat_t[order], flat_j[order], send_counts, expert_counts


def plan_regroup(counts_all, rank: int, world: int):
    """counts_all[src, e]: rows rank src sends for expert e.  The rows this rank receives lie [src][expert][token];
    the expert products want them [expert][src][token].  Returns (perm, rows_per_expert[n_expert]) with
    grouped = received[perm] (and received = grouped[inverse of perm])."""
    counts_all = np.asarray(counts_all, np.int64)
    n_expert = counts_all.shape[1]
    mine = [e for e in range(n_expert) if home_rank(e, world) == rank]
    start = {}
    off = 0
    for src in range(world):
        for e in mine:
            start[(src, e)] = off
            off += int(counts_all[src, e])
    perm = []
    per_expert = np.zeros(n_expert, np.int64)
    for e in mine:
        for src in range(world):
            n = int(counts_all[src, e])
            perm.extend(range(start[(src, e)], start[(src, e)] + n))
            per_expert[e] += n
    return np.asarray(perm, np.int64), per_expert


class ExpertParallelLayer:
    """Routed-expert FFN layer with the experts striped over the ranks (expert e on rank e % G, expertvm/src/place.rs:
    71-75) and the TOKENS sharded too: every rank routes its own tokens, sends each routed row to the rank that owns
    its expert (all-to-all), runs its experts on what it received, sends the results back (all-to-all) and adds a token's
    rows in ascending expert id (the accumulation order of scatter_expert_rows, decode.rs:10263).  A row's expert output
    does not depend on which other rows share its batch, so the layer's output is bit-identical to the single-device
    layer on the same tokens.

    route(x) -> (ids[T, k] int32, w[T, k] float32) and experts(counts[n_expert], rows[n, d]) -> y[n, d] are callables on
    torch tensors of the group's device type (`cuda_backend` builds them for the CUDA executor); the exchange is
    torch.distributed all_to_all_single, i.e. NCCL over NVLink for CUDA tensors."""

    def __init__(self, n_expert: int, n_used: int, route, experts, group=None):
        self.n_expert, self.n_used, self.route, self.experts, self.group = n_expert, n_used, route, experts, group
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)

    @staticmethod
    def cuda_backend(ex, router, gate, up, down, n_used: int, norm_w: bool):
        """(route, experts) over the CUDA executor; gate/up/down hold None for experts that live on other ranks."""
        n_expert = len(gate)

        def route(x):
            ids = torch.empty(x.shape[0], n_used, dtype=torch.int32, device=x.device)
            w = torch.empty(x.shape[0], n_used, dtype=torch.float32, device=x.device)
            torch.cuda.current_stream().synchronize()  # x is ready before the executor's stream reads it
            ex.moe_route_device(router, n_expert, n_used, norm_w, x.shape[0], x.data_ptr(), ids.data_ptr(), w.data_ptr())
            ex.synchronize()
            return ids, w

        def experts(counts, rows):
            y = torch.empty_like(rows)
            if rows.shape[0]:
                torch.cuda.current_stream().synchronize()
                ex.moe_experts_device(gate, up, down, counts, rows.data_ptr(), y.data_ptr())
                ex.synchronize()
            return y
        return route, experts

    def __call__(self, x: torch.Tensor):
        """x: this rank's tokens [T, n_embd] (float32, contiguous).  Returns (out[T, n_embd], ids, w)."""
        dev = x.device
        ids, w = self.route(x)
        src_t, src_j, send_counts, expert_counts = plan_dispatch(ids.cpu().numpy(), self.n_expert, self.world)
        # who sends how many rows for which expert: one small all-gather
        mine = torch.tensor(expert_counts, dtype=torch.int64, device=dev)
        gathered = [torch.empty_like(mine) for _ in range(self.world)]
        dist.all_gather(gathered, mine, group=self.group)
        counts_all = torch.stack(gathered).cpu().numpy()
        recv_counts = [int(sum(counts_all[src, e] for e in range(self.n_expert) if home_rank(e, self.world) == self.rank))
                       for src in range(self.world)]
        t_idx = torch.from_numpy(src_t).to(dev)
        send = x.index_select(0, t_idx).contiguous()
        recv = torch.empty(sum(recv_counts), x.shape[1], dtype=x.dtype, device=dev)
        dist.all_to_all_single(recv, send, output_split_sizes=recv_counts, input_split_sizes=[int(c) for c in send_counts],
                               group=self.group)
        perm, per_expert = plan_regroup(counts_all, self.rank, self.world)
        perm_t = torch.from_numpy(perm).to(dev)
        y_grouped = self.experts(per_expert, recv.index_select(0, perm_t).contiguous())
        y_recv = torch.empty_like(recv)
        y_recv.index_copy_(0, perm_t, y_grouped)
        back = torch.empty_like(send)
        dist.all_to_all_single(back, y_recv, output_split_sizes=[int(c) for c in send_counts], input_split_sizes=recv_counts,
                               group=self.group)
        # combine: a token's rows in ascending expert id, each multiplied by its router weight, added from zero
        tokens = x.shape[0]
        row_of = np.empty((tokens, self.n_used), np.int64)
        row_of[src_t, src_j] = np.arange(src_t.size)
        ids_np = ids.cpu().numpy()
        slot_order = np.argsort(ids_np, axis=1, kind="stable")  # slots by ascending expert id
        out = torch.zeros_like(x)
        for s in range(self.n_used):
            j = slot_order[:, s]
            rows = torch.from_numpy(row_of[np.arange(tokens), j]).to(dev)
            wj = w.gather(1, torch.from_numpy(j).to(dev).unsqueeze(1))
            term = back.index_select(0, rows) * wj  # product rounded, then added: no fused multiply-add
            out = out + term
        return out, ids, w


class PeerExpertParallelLayer:
    """The expert-parallel layer with the exchange inside the library (llr_moe_ep_*): same layout as
    ExpertParallelLayer (expert e on rank e % G, tokens sharded), but routed rows and their results move between the
    GPUs as peer stores issued by the gather and scatter kernels, with no collective call and no host hop for rows.
    The process group only carries the memory handles at construction (any backend).  gate/up/down hold None for
    the experts of other ranks; max_tokens bounds this rank's tokens per call.  Every rank makes the same sequence
    of calls; a rank must pass at least one token."""

    def __init__(self, ex, router, gate, up, down, n_used: int, norm_w: bool, max_tokens: int, group=None):
        from .executor import moe_ep_arena_bytes
        self.ex, self.n_used, self.n_embd = ex, n_used, router.cols
        world, rank = dist.get_world_size(group), dist.get_rank(group)
        self.nbytes = moe_ep_arena_bytes(len(gate), n_used, router.cols, world, max_tokens)
        self.arena, handle = ex.shared_alloc(self.nbytes)
        handles = [None] * world
        dist.all_gather_object(handles, handle, group=group)
        self.peers = [self.arena if g == rank else ex.shared_open(handles[g]) for g in range(world)]
        self.ep = ex.moe_ep(router, gate, up, down, n_used, norm_w, world, rank, max_tokens, self.arena, self.nbytes, self.peers)
        self.rank = rank
        dist.barrier(group=group)  # every rank's layer exists before anybody's first run stores into a peer

    def __call__(self, x: torch.Tensor, synchronize: bool = True):
        """x: this rank's tokens [T, n_embd] (float32, contiguous, on the executor's GPU).  Returns (out, ids, w)."""
        tokens = x.shape[0]
        out = torch.empty_like(x)
        ids = torch.empty(tokens, self.n_used, dtype=torch.int32, device=x.device)
        w = torch.empty(tokens, self.n_used, dtype=torch.float32, device=x.device)
        torch.cuda.current_stream().synchronize()  # x is ready before the executor's stream reads it
        self.ep.run(tokens, x.data_ptr(), out.data_ptr(), ids.data_ptr(), w.data_ptr())
        if synchronize:
            self.ex.synchronize()
        return out, ids, w

    def close(self) -> None:
        self.ep.free()
        for g, p in enumerate(self.peers):
            if g != self.rank:
                self.ex.shared_close(p)
        self.ex.shared_free(self.arena)
