"""Host logic of the column-parallel wrapper on CPU: partition arithmetic, gather layout, and a
world_size-2 and -4 gloo runs in which the per-rank GEMM is replaced by the oracle (no GPU)."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from hipkittensp_b200 import sharded
from oracle import mxfp6_ref as R


def test_shard_bounds_cover_and_reject():
    for N, g in ((57344, 2), (57344, 4), (57344, 8), (1024, 1)):
        spans = [sharded.shard_bounds(N, g, r) for r in range(g)]
        assert spans[0][0] == 0 and spans[-1][1] == N
        for a, b in zip(spans, spans[1:]):
            assert a[1] == b[0]
        assert len({hi - lo for lo, hi in spans}) == 1
    with pytest.raises(ValueError):
        sharded.shard_bounds(1000, 3, 0)


def test_assemble_columns_layout():
    g, M, per = 4, 5, 3
    full = torch.arange(M * g * per, dtype=torch.float32).view(M, g * per)
    gathered = torch.stack([full[:, r * per:(r + 1) * per].contiguous() for r in range(g)])
    out = torch.empty(M, g * per)
    assert torch.equal(sharded.assemble_columns(gathered, out), full)


def test_shard_rows_matches_bounds():
    t = torch.arange(64).view(16, 4)
    parts = [sharded.shard_rows(t, 4, r) for r in range(4)]
    assert torch.equal(torch.cat(parts), t)
    assert all(p.is_contiguous() for p in parts)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, M, N, K, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        A, B = R.make_inputs("normal", M, N, K, seed=0)
        pa, sa = R.quantize(A, R.E2M3)
        pb, sb = R.quantize(B, R.E2M3)
        op = sharded.ColumnParallelGemm(M, N, K, device="cpu")
        b_sh = sharded.shard_rows(torch.from_numpy(pb), world, rank)
        sb_sh = sharded.shard_rows(torch.from_numpy(sb), world, rank)

        def fake_local(a, s_a, b, s_b):            # the oracle stands in for the GPU kernel
            op.c_shard.copy_(R.gemm_cpu_path(a, s_a, b, s_b))
            return op.c_shard

        op.local_gemm = fake_local
        C = op(torch.from_numpy(pa), torch.from_numpy(sa), b_sh, sb_sh)
        want = R.gemm_cpu_path(torch.from_numpy(pa), torch.from_numpy(sa), torch.from_numpy(pb), torch.from_numpy(sb))
        ret[rank] = bool(torch.equal(C.float(), want.float()))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_gloo_ranks_gather_equals_single(world):
    with mp.Manager() as mgr:
        ret = mgr.dict()
        mp.spawn(_worker, args=(world, _free_port(), 64, 256, 256, ret), nprocs=world, join=True)
        assert dict(ret) == {r: True for r in range(world)}


def test_row_parallel_single_process_bounds():
    # without a process group the wrapper owns all rows; only the partition arithmetic is exercised here
    rp = sharded.RowParallelGemm(64, 32, 128, device="cpu")
    assert (rp.lo, rp.hi) == (0, 64) and tuple(rp.c_rows.shape) == (64, 32) and rp.c_full is None
