"""Row-sharded Q4_K matmul over several GPUs, one process per GPU.

The reference is single-GPU; this layer is what the multi-GPU configurations add.  Output
rows are independent and a row range of the packed weight is a contiguous byte range
(rows are `rowStrideWords*4` bytes apart, runtime/gguf_loader.cpp:367-378), so rank g keeps
rows [g*Ns, (g+1)*Ns) resident, every rank holds the (small) activations, and the output
slices are exchanged with one all-gather (`torch.distributed`, NCCL on GPUs).

    M = 1   slices are contiguous pieces of Y[N]: all-gather straight into Y.
    M > 1   slices are column blocks of row-major Y[M, N]: all-gather into [G][M][Ns],
            then one strided copy into [M][N].

When N is not a multiple of the world size every rank takes ceil(N/G) rows and the last
rank's shard is zero-padded (a padded row decodes to weight 0 and is cut off after the gather).

`matmul_fn(x, shard) -> y` does the local product.  By default it is the CUDA path of this
package; tests of the partitioning logic on CPU ranks pass their own.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Optional

import numpy as np

from .synth import BLOCK_BYTES, QK_K


def shard_rows(N: int, world: int) -> int:
    """Rows per rank (the last rank may own fewer real rows)."""
    return (N + world - 1) // world


def shard_range(N: int, world: int, rank: int) -> tuple[int, int]:
    ns = shard_rows(N, world)
    return min(rank * ns, N), min((rank + 1) * ns, N)


def shard_raw(raw: np.ndarray, N: int, K: int, world: int, rank: int, block_bytes: int = BLOCK_BYTES) -> np.ndarray:
    """This rank's rows of a raw [N, K/256*block_bytes] weight (144-byte Q4_K blocks unless told otherwise),
    zero-padded to shard_rows(N, world) rows."""
    rb = (K // QK_K) * block_bytes
    raw = np.ascontiguousarray(raw).view(np.uint8).reshape(N, rb)
    n0, n1 = shard_range(N, world, rank)
    ns = shard_rows(N, world)
    out = np.zeros((ns, rb), np.uint8)
    out[: n1 - n0] = raw[n0:n1]
    return out


@dataclass
class ShardedQ4KLinear:
    """One projection, N-sharded.  `shard` is whatever `matmul_fn` understands as a weight."""
    N: int
    K: int
    world: int
    rank: int
    shard: object
    matmul_fn: Callable
    group: Optional[object] = None

    @property
    def Ns(self) -> int:
        return shard_rows(self.N, self.world)

    def local(self, x, out=None):
        """This rank's slice Y[:, n0:n0+Ns] (padded rows included)."""
        return self.matmul_fn(x, self.shard, out)

    def forward(self, x, gathered=None):
        """Full Y[M, N] on every rank.  x: [M, K] float32, replicated."""
        import torch
        import torch.distributed as dist

        M = x.shape[0]
        Ns, G = self.Ns, self.world
        if G == 1:
            return self.local(x)[:, : self.N]
        if gathered is None:
            gathered = torch.empty((G, M, Ns), dtype=torch.float32, device=x.device)
        # the local product is written straight into this rank's slot of the gather buffer
        self.local(x, gathered[self.rank])
        dist.all_gather_into_tensor(gathered.view(-1), gathered[self.rank].reshape(-1), group=self.group)
        if M == 1:
            return gathered.view(1, G * Ns)[:, : self.N]
        return gathered.permute(1, 0, 2).reshape(M, G * Ns)[:, : self.N]


def make_cuda_linear(ctx, raw: np.ndarray, N: int, K: int, world: int, rank: int, group=None) -> ShardedQ4KLinear:
    """Upload this rank's rows and bind the CUDA matmul of `ctx` (a Q4KContext)."""
    from . import pack_q4k

    ns = shard_rows(N, world)
    w = ctx.upload(pack_q4k(shard_raw(raw, N, K, world, rank), ns, K))

    def fn(x, shard, out=None):
        import torch

        if out is None:
            out = torch.empty((x.shape[0], shard.N), dtype=torch.float32, device=x.device)
        ctx.matmul(x, shard, out=out)
        return out

    return ShardedQ4KLinear(N, K, world, rank, w, fn, group)


class PeerGather:
    """Fused all-gather over peer-mapped memory for a set of projections.

    One symmetric allocation per rank holds, for every projection, the gather buffer [world][M][Ns] -- twice
    (`double_buffer`, the default): the matmul kernel of rank g stores its slice into slot g of EVERY rank's
    buffer (plain stores over NVLink), steps alternate between the two halves, and ONE bounded flag barrier per
    step makes the slices visible.  With two halves a rank that runs ahead stores the next step's slices into the
    half nobody reads; a rank that has passed barrier t+1 knows that every peer queued its reads of step t ahead
    of that barrier, so step t+2 may overwrite step t's half.  With `double_buffer=False` there is one half and a
    consumer that reads the buffer must put a second barrier after its reads.
    Replaces the per-projection NCCL all-gather of `ShardedQ4KLinear.forward`.
    """

    def __init__(self, ctx, world: int, rank: int, slots: dict, group=None, timeout_ms: int = 1000,
                 double_buffer: bool = True):
        import ctypes as C

        import torch
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm

        self.ctx, self.world, self.rank, self.timeout_ms = ctx, world, rank, timeout_ms
        group = group or dist.group.WORLD
        dev = torch.device(f"cuda:{ctx.device}")
        self.offsets, total = {}, 0
        for name, (M, Ns) in slots.items():
            self.offsets[name] = (total, M, Ns)
            total += world * M * Ns
            total = (total + 63) // 64 * 64
        self.half = max(total, 64)
        self.halves = 2 if double_buffer else 1
        self.buf = symm.empty(self.half * self.halves, dtype=torch.float32, device=dev)
        self.flags = symm.empty(64, dtype=torch.int32, device=dev)
        self.buf.zero_()
        self.flags.zero_()
        hb = symm.rendezvous(self.buf, group.group_name)
        hf = symm.rendezvous(self.flags, group.group_name)
        torch.cuda.synchronize()
        dist.barrier(group=group)          # every rank's flags are zero before anyone signals
        order = [rank] + [p for p in range(world) if p != rank]
        self.slot_ptrs = {}
        for name, (off, M, Ns) in self.offsets.items():
            arr = (C.c_void_p * world)(*[int(hb.buffer_ptrs[p]) + (off + rank * M * Ns) * 4 for p in order])
            self.slot_ptrs[name] = arr
        self.flag_ptrs = (C.c_void_p * world)(*[int(hf.buffer_ptrs[p]) for p in range(world)])
        self._handles = (hb, hf)
        self.steps = 0                     # barriers enqueued so far (every rank enqueues the same ones)
        # word 63 of the own flag array is the step counter the barrier kernel keeps
        ctx.peer_double_buffer(int(hf.buffer_ptrs[rank]) + 63 * 4 if double_buffer else 0, self.half)

    def close(self) -> None:
        self.ctx.peer_double_buffer(0, 0)

    def gathered(self, name: str, step: int | None = None):
        """[world, M, Ns] view of this rank's gather buffer for one projection: the slices of step `step`
        (0-based count of barriers; default: the last one enqueued)."""
        off, M, Ns = self.offsets[name]
        step = self.steps - 1 if step is None else step
        base = (step % self.halves) * self.half if self.halves == 2 else 0
        return self.buf[base + off: base + off + self.world * M * Ns].view(self.world, M, Ns)

    def matmul(self, name: str, x, shard, bias=None) -> None:
        self.ctx.matmul_allgather(x, shard, self.slot_ptrs[name], bias)

    def barrier(self, replays: int = 1) -> None:
        """Epoch 0 = self-advancing (the count lives in the flag array), so this call can be captured
        into a CUDA graph and replayed.  `note_replays` keeps the host-side step count right for replays."""
        self.ctx.peer_barrier(self.flag_ptrs, self.rank, 0, self.timeout_ms)
        self.steps += 1

    def note_replays(self, n: int = 1) -> None:
        """A CUDA graph holding one step (matmuls + barrier) was replayed n times."""
        self.steps += n
