"""Column-parallel GEMM on 2+ GPUs: every rank's gathered C equals the single-GPU result bit for bit (same
kernel, same tile arithmetic), for both exchanges.  Runs as child processes, one per GPU."""
import os
import socket
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

WORKER = r'''
import os, sys, torch, torch.distributed as dist
sys.path.insert(0, os.environ["MXFP6_ROOT"])
import hipkittensp_b200 as hk
from hipkittensp_b200.sharded import ColumnParallelGemm, shard_rows
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(rank); dev = torch.device("cuda", rank)
dist.init_process_group("nccl", device_id=dev)
M, N, K = 512, 2048, 1024
g = torch.Generator(device=dev).manual_seed(5)
A = torch.randn(M, K, device=dev, generator=g); B = torch.randn(N, K, device=dev, generator=g)
pa, sa = hk.quantize(A); pb, sb = hk.quantize(B)
want = hk.gemm(pa, sa, pb, sb)                      # single-GPU result of the whole problem
ok = True
for mode in ("nccl", "fused"):
    op = ColumnParallelGemm(M, N, K, device=dev, gather=mode)
    for rep in range(2):
        C = op(pa, sa, shard_rows(pb, world, rank), shard_rows(sb, world, rank))
        torch.cuda.synchronize()
        ok = ok and bool(torch.equal(C.view(torch.int16), want.view(torch.int16)))
from hipkittensp_b200.sharded import RowParallelGemm
for g in (False, True):
    rp = RowParallelGemm(M, N, K, device=dev, gather=g)
    out = rp(shard_rows(pa, world, rank), shard_rows(sa, world, rank), pb, sb)
    torch.cuda.synchronize()
    exp = want if g else want[rp.lo:rp.hi]
    ok = ok and bool(torch.equal(out.view(torch.int16), exp.contiguous().view(torch.int16)))
assert hk.device_status() == 0
flag = torch.tensor([1 if ok else 0], device=dev)
dist.all_reduce(flag, op=dist.ReduceOp.MIN)
if rank == 0:
    print("SHARDED_OK" if int(flag) == 1 else "SHARDED_MISMATCH", flush=True)
dist.barrier(); dist.destroy_process_group()
'''


def test_column_parallel_matches_single_gpu():
    n = torch.cuda.device_count()
    if n < 2:
        pytest.skip("needs at least 2 GPUs")
    world = 2
    s = socket.socket(); s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]; s.close()
    env = dict(os.environ, MXFP6_ROOT=ROOT, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", str(port), "-c", WORKER]
    # torchrun has no -c: write the worker next to the test's temp dir instead
    import tempfile
    with tempfile.NamedTemporaryFile("w", suffix=".py", delete=False) as f:
        f.write(WORKER)
        path = f.name
    cmd = cmd[:-2] + [path]
    try:
        out = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    finally:
        os.unlink(path)
    assert "SHARDED_OK" in out.stdout, out.stdout[-2000:] + out.stderr[-2000:]
