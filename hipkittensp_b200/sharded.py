"""Column-parallel MX-FP6 GEMM over the GPUs of one box.

B[N,K] (and its scales) is split along N into `world` contiguous row blocks, A is replicated, rank r
computes C[:, r*N/g:(r+1)*N/g] with the single-GPU kernel and the shards are all-gathered so that every
rank ends with the full row-major C[M,N].  The reference's only multi-GPU GEMM shards A by rows and has
no exchange step (distributed-kernels/bf16_gemm/example.py:70,112); the column-parallel split with a
gather is this path's own multi-GPU form.

Two exchanges:

* `gather="fused"` (default on GPUs): the full C of every rank lives in symmetric memory (peer-mapped over
  NVLink); the GEMM kernel's epilogue stores each finished 128x64 piece by TMA into the right column window of
  the local C and of every peer's C (`mxfp6_gemm_multi`), so the gather overlaps the remaining tiles and no
  re-layout pass exists.  A cross-GPU barrier on the stream closes the step.  Ordering between steps: a peer's
  pushes of the next step must not land in a C this rank is still reading.  With `depth=2` (the default) the
  operator owns two full-size C buffers and alternates between them, so the C a call returns stays untouched
  until the call after the next one: by then every rank has passed the barrier that closed the next call, which
  on each rank's stream lies behind its own readers of this C.  With `depth=1` there is one C, and every call
  opens with a second cross-GPU barrier on the stream (all ranks' queued readers of the previous C are done)
  before any tile is pushed.  Either way the reader's work must be queued on the same stream before the next call.
* `gather="copy"`: the same symmetric C buffers, but the kernel writes only the local C and raises a flag per finished
  block of it; side streams wait for the flags (stream memory operations) and the GPU's copy engines carry the blocks
  to the peers (`mxfp6_gemm_copy_gather`).  The GEMM is not slowed by pushing, but nothing leaves before a whole block
  is finished, the copy engines want few large copies, and copies and GEMM compete for HBM: measured on 4 GPUs this
  exchange is slower than "fused" (3.3 ms per step of 16384 x 57344 x 8192 against 2.3).  The same ordering rules as
  "fused".
* `gather="nccl"`: one NCCL (or gloo, on CPU) all-gather of the contiguous [M, N/g] shards into a [g, M, N/g]
  buffer followed by a strided copy into row-major C.  The baseline, and the path the CPU tests use.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from ._lib import E2M3
from .gemm import dispatch_micro


def shard_bounds(N: int, world: int, rank: int) -> tuple[int, int]:
    """Rows [lo, hi) of B (columns of C) owned by `rank`.  N must divide evenly into 128-row blocks per rank
    only loosely: any N % world == 0 is accepted."""
    if N % world:
        raise ValueError(f"N={N} is not divisible by the number of ranks {world}")
    per = N // world
    return rank * per, (rank + 1) * per


def shard_rows(t: torch.Tensor, world: int, rank: int) -> torch.Tensor:
    """The contiguous row block of a [N, *] operand that `rank` owns."""
    lo, hi = shard_bounds(t.shape[0], world, rank)
    return t[lo:hi].contiguous()


def assemble_columns(gathered: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """[g, M, N/g] (shard-major, as an all-gather of [M, N/g] shards produces) -> row-major [M, N]."""
    g, M, per = gathered.shape
    out.view(M, g, per).copy_(gathered.permute(1, 0, 2))
    return out


class ColumnParallelGemm:
    """Holds the communicator and the reusable buffers of one sharded GEMM shape."""

    def __init__(self, M: int, N: int, K: int, group=None, device=None, fmt: int = E2M3, gather: str | None = None,
                 depth: int = 2, strip_tiles: int | None = None, streams_per_peer: int = 1):
        if depth not in (1, 2):
            raise ValueError("depth must be 1 or 2")
        self.depth, self.calls = depth, 0
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.M, self.N, self.K, self.fmt = M, N, K, fmt
        self.lo, self.hi = shard_bounds(N, self.world, self.rank)
        self.device = device
        on_gpu = device is not None and torch.device(device).type == "cuda"
        if gather is None:
            gather = "fused" if (on_gpu and self.world > 1) else "nccl"
        if gather not in ("fused", "copy", "nccl"):
            raise ValueError(gather)
        if gather == "copy" and self.world > 1:
            from ._lib import debug_plan

            # per-block flags exist in the CTA-pair kernel only: smaller shards keep the pushes from the epilogue
            sms = torch.cuda.get_device_properties(device).multi_processor_count
            if not debug_plan(M, self.hi - self.lo, K, sm_count=sms)["pair"] or (self.hi - self.lo) % 8 or N % 8:
                gather = "fused"
        self.mode = gather
        self.symm = None
        # copy engines are at their best with few large copies: by default a block is a whole row group of the tile order
        # (4096 rows of the window) and every peer has one copy stream
        if strip_tiles is None:
            strip_tiles = max(1, (self.hi - self.lo + 255) // 256)
        self.copy_streams, self.copy_scratch, self.strip_tiles = [], None, strip_tiles
        if self.mode == "copy" and self.world > 1:
            from .gemm import copy_gather_scratch_bytes

            with torch.cuda.device(device):
                self.copy_streams = [torch.cuda.Stream(device=device) for _ in range(streams_per_peer * (self.world - 1))]
            nbytes = copy_gather_scratch_bytes(M, self.hi - self.lo, strip_tiles)
            self.copy_scratch = torch.zeros(max(nbytes // 4, 1), dtype=torch.int32, device=device)
        if self.mode in ("fused", "copy") and self.world > 1:
            import torch.distributed._symmetric_memory as symm

            # destination 0 is local, the rest are the peers' copies of C, rotated so that ranks do not all
            # push to the same peer at the same moment
            order = [(self.rank + i) % self.world for i in range(self.world)]
            self.bufs = []
            for _ in range(depth):
                c = symm.empty((M, N), dtype=torch.bfloat16, device=device)
                h = symm.rendezvous(c, dist.group.WORLD if group is None else group)
                self.bufs.append((c, h, [c] + [h.get_buffer(r, (M, N), torch.bfloat16) for r in order[1:]]))
            self.c_full, self.symm, self.dests = self.bufs[0]
            self.c_shard = self.c_full[:, self.lo:self.hi]
            self.gathered = None
        else:
            self.c_shard = torch.empty((M, self.hi - self.lo), dtype=torch.bfloat16, device=device)
            self.gathered = torch.empty((self.world, M, self.hi - self.lo), dtype=torch.bfloat16, device=device) \
                if self.world > 1 else None
            self.c_full = torch.empty((M, N), dtype=torch.bfloat16, device=device) if self.world > 1 else self.c_shard

    def local_gemm(self, A, scale_A, B_shard, scale_B_shard) -> torch.Tensor:
        """This rank's [M, N/g] block of C (no exchange)."""
        if self.mode in ("fused", "copy") and self.world > 1:
            from .gemm import dispatch_multi

            # (into the buffer of the latest call: no peer is written, so no ordering is needed)
            dispatch_multi(A, B_shard, self.dests[:1], self.lo, scale_A, scale_B_shard, self.fmt)
        else:
            dispatch_micro(A, B_shard, self.c_shard, scale_A, scale_B_shard, self.fmt)
        return self.c_shard

    def gather(self) -> torch.Tensor:
        if self.world == 1:
            return self.c_shard
        dist.all_gather_into_tensor(self.gathered.view(-1), self.c_shard.view(-1), group=self.group)
        return assemble_columns(self.gathered, self.c_full)

    def __call__(self, A, scale_A, B_shard, scale_B_shard) -> torch.Tensor:
        if self.mode in ("fused", "copy") and self.world > 1:
            from .gemm import dispatch_copy_gather, dispatch_multi

            self.c_full, self.symm, self.dests = self.bufs[self.calls % self.depth]
            self.c_shard = self.c_full[:, self.lo:self.hi]
            if self.depth == 1 and self.calls > 0:
                self.symm.barrier()      # every rank's readers of the previous C are done before anyone overwrites it
            self.calls += 1
            if self.mode == "copy":
                dispatch_copy_gather(A, B_shard, self.dests, self.lo, scale_A, scale_B_shard, self.copy_scratch,
                                     self.copy_streams, self.strip_tiles, self.fmt)
            else:
                dispatch_multi(A, B_shard, self.dests, self.lo, scale_A, scale_B_shard, self.fmt)
            self.symm.barrier()          # every rank's pushes have landed before anyone reads C
            return self.c_full
        self.local_gemm(A, scale_A, B_shard, scale_B_shard)
        return self.gather()


class RowParallelGemm:
    """The reference's own multi-GPU split (distributed-kernels/bf16_gemm/example.py:70,112): A is sharded by rows,
    B is replicated, rank r owns rows [r*M/g, (r+1)*M/g) of C and there is no exchange.  With `gather=True` the row
    blocks are additionally pushed to every peer by the GEMM epilogue (symmetric memory), so that each rank ends
    with all of C; row blocks are contiguous, so no re-layout is involved either way."""

    def __init__(self, M: int, N: int, K: int, group=None, device=None, fmt: int = E2M3, gather: bool = False,
                 depth: int = 2):
        if depth not in (1, 2):
            raise ValueError("depth must be 1 or 2")
        self.depth, self.calls = depth, 0
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.M, self.N, self.K, self.fmt = M, N, K, fmt
        self.lo, self.hi = shard_bounds(M, self.world, self.rank)
        self.push = gather and self.world > 1
        self.symm = None
        if self.push:
            import torch.distributed._symmetric_memory as symm

            order = [(self.rank + i) % self.world for i in range(self.world)]
            self.bufs = []
            for _ in range(depth):        # same ordering contract between steps as ColumnParallelGemm
                c = symm.empty((M, N), dtype=torch.bfloat16, device=device)
                h = symm.rendezvous(c, dist.group.WORLD if group is None else group)
                views = [c] + [h.get_buffer(r, (M, N), torch.bfloat16) for r in order[1:]]
                self.bufs.append((c, h, [b[self.lo:self.hi] for b in views]))
            self.c_full, self.symm, self.dests = self.bufs[0]
            self.c_rows = self.dests[0]
        else:
            self.c_rows = torch.empty((self.hi - self.lo, N), dtype=torch.bfloat16, device=device)
            self.c_full = None

    def __call__(self, A_rows, scale_A_rows, B, scale_B) -> torch.Tensor:
        """A_rows: this rank's [M/g, .] block of A.  Returns the rank's rows of C, or all of C with gather=True."""
        if self.push:
            from .gemm import dispatch_multi

            self.c_full, self.symm, self.dests = self.bufs[self.calls % self.depth]
            self.c_rows = self.dests[0]
            if self.depth == 1 and self.calls > 0:
                self.symm.barrier()
            self.calls += 1
            dispatch_multi(A_rows, B, self.dests, 0, scale_A_rows, scale_B, self.fmt)
            self.symm.barrier()
            return self.c_full
        dispatch_micro(A_rows, B, self.c_rows, scale_A_rows, scale_B, self.fmt)
        return self.c_rows
