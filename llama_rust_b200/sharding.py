"""Sharding layer for one multi-GPU box: one process per GPU over torch.distributed.

The reference has no multi-device execution (its only notions are simulated:
`home_gpu = expert % n_gpus`, expertvm/src/place.rs:71-75); this layer is new.

* Dense products shard by OUTPUT ROWS: rows are independent and a row range of a packed
  matrix is a contiguous byte range (langtax/src/decode.rs:10876-10879, `quant_mat_rows`
  :9680-9713), so rank g holds rows [g*R/G, (g+1)*R/G) of every matrix, activations are
  replicated, and the exchange is an all-gather of M x R/G result slices.
* Routed experts stripe as `e % G`; token rows travel to the expert's rank and back with
  all-to-all, and a token's output is summed over its experts in ascending expert id
  (the reference's accumulation order, decode.rs:10006-10290), so results do not depend
  on G.

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
    """Contiguous, balanced row range of `rank`; exact for every BASELINE shape (rows % 8 == 0)."""
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


class ExpertParallelFFN:
    """Routed-expert FFN with experts striped over ranks.

    `route(x) -> (ids[T, k], w[T, k])` is replicated (every rank routes every token);
    `expert_ffn(e, rows[n, d]) -> rows[n, d]` runs one local expert on a packed batch.
    Tokens are replicated too (the usual data layout after attention), so the dispatch
    all-to-all only moves the rows a rank does NOT own... every rank could gather its own
    rows locally; the exchange that cannot be avoided is the combine: each rank returns the
    expert outputs of its experts for all tokens, and every rank sums a token's k rows in
    ascending expert id.
    """

    def __init__(self, n_expert: int, route, expert_ffn, group=None):
        self.n_expert, self.route, self.expert_ffn, self.group = n_expert, route, expert_ffn, group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)

    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        ids, w = self.route(x)
        tokens, k = ids.shape
        d = x.shape[1]
        # rows in (expert ascending, token ascending) order, as grouped_routed_ffn builds them
        flat_e = ids.reshape(-1)
        flat_t = torch.arange(tokens, device=x.device).repeat_interleave(k)
        order = torch.argsort(flat_e * tokens + flat_t, stable=True)
        e_sorted, t_sorted = flat_e[order], flat_t[order]
        counts = torch.bincount(e_sorted, minlength=self.n_expert)
        starts = torch.cumsum(counts, 0) - counts
        y_rows = torch.zeros(tokens * k, d, dtype=x.dtype, device=x.device)
        # per-rank row counts are known everywhere (routing is replicated): all-to-all sizes
        per_rank = [int(sum(int(counts[e]) for e in range(self.n_expert) if home_rank(e, self.world) == r))
                    for r in range(self.world)]
        mine = []
        for e in range(self.n_expert):
            if home_rank(e, self.world) != self.rank or int(counts[e]) == 0:
                continue
            s, n = int(starts[e]), int(counts[e])
            out = self.expert_ffn(e, x[t_sorted[s:s + n]])
            mine.append((s, out))
        send = torch.cat([o for _, o in mine]) if mine else torch.zeros(0, d, dtype=x.dtype, device=x.device)
        # every rank needs every row: all-gather of ragged blocks via all_to_all_single with
        # identical payload to each peer (the combine step of expert parallelism)
        recv = torch.empty(sum(per_rank), d, dtype=x.dtype, device=x.device)
        dist.all_to_all_single(recv, send.repeat(self.world, 1), output_split_sizes=per_rank,
                               input_split_sizes=[send.shape[0]] * self.world, group=self.group)
        # place the received blocks: rank r's block lists its experts ascending
        off = 0
        for r in range(self.world):
            for e in range(self.n_expert):
                if home_rank(e, self.world) != r or int(counts[e]) == 0:
                    continue
                s, n = int(starts[e]), int(counts[e])
                y_rows[s:s + n] = recv[off:off + n]
                off += n
        # combine: ascending expert id per token, starting from zero
        out = torch.zeros_like(x)
        w_sorted = w.reshape(-1)[order]
        # slot j of token t = its j-th expert in ascending id
        slot = torch.zeros(tokens, dtype=torch.long, device=x.device)
        rows_of_tok = torch.zeros(tokens, k, dtype=torch.long, device=x.device)
        for i in range(tokens * k):  # routing tables are tiny (T*k entries)
            t = int(t_sorted[i])
            rows_of_tok[t, int(slot[t])] = i
            slot[t] += 1
        for j in range(k):
            idx = rows_of_tok[:, j]
            out = out + y_rows[idx] * w_sorted[idx].unsqueeze(1)
        return out


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

    def run(self, stream: int = 0) -> None:
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


class StripedExperts:
    """Routed-expert FFN layer with the experts striped over the ranks (expert e on rank e % G,
    expertvm/src/place.rs:71-75), on the CUDA executor.  Every rank routes every token (the router
    is replicated) and runs llr_moe_ffn with only its own experts resident; the exchange step is one
    sum of the ranks' partial outputs (NCCL all-reduce, or gloo).  With two experts per token at most
    two terms of that sum are non-zero for any element, so the result is bit-identical to the
    single-device layer whatever order the collective adds in."""

    def __init__(self, ex, router, gate, up, down, n_used: int, norm_w: bool, group=None):
        self.ex, self.router, self.n_used, self.norm_w, self.group = ex, router, n_used, norm_w, group
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        keep = [home_rank(e, self.world) == self.rank for e in range(len(gate))]
        self.gate = [m if k else None for m, k in zip(gate, keep)]
        self.up = [m if k else None for m, k in zip(up, keep)]
        self.down = [m if k else None for m, k in zip(down, keep)]

    def __call__(self, x, device=None):
        """x: [tokens, n_embd] float32 numpy array (host).  Returns (out, ids, weights) as numpy arrays
        (out is a view of a pinned buffer that the next call reuses)."""
        shape = tuple(np.asarray(x).reshape(-1, self.router.cols).shape)
        if getattr(self, "_pin", None) is None or tuple(self._pin.shape) != shape:
            self._pin = torch.empty(shape, dtype=torch.float32)
            if device is not None:
                self._pin = self._pin.pin_memory()  # the executor writes its partial sums straight into it
        partial, ids, w = self.ex.moe_ffn(self.router, self.gate, self.up, self.down, self.n_used, self.norm_w, x,
                                          out=self._pin.numpy())
        if device is None:
            dist.all_reduce(self._pin, op=dist.ReduceOp.SUM, group=self.group)
        else:
            t = self._pin.to(device, non_blocking=True)
            dist.all_reduce(t, op=dist.ReduceOp.SUM, group=self.group)
            self._pin.copy_(t, non_blocking=True)
            torch.cuda.current_stream().synchronize()
        return self._pin.numpy(), ids, w
