"""Column-parallel GEMM on 2+ GPUs: every rank's gathered C equals the single-GPU result bit for bit (same
kernel, same tile arithmetic), for both exchanges.  Every step has its own A, a reader of C is queued behind
each step without a host synchronisation, and the ranks take turns falling behind, so a step that overwrote a
C still being read on a slower rank would show as a mismatch.  Runs as child processes, one per GPU."""
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
from hipkittensp_b200.sharded import ColumnParallelGemm, RowParallelGemm, shard_rows
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(rank); dev = torch.device("cuda", rank)
dist.init_process_group("nccl", device_id=dev)
STEPS = 6
ok = True
def digest(C):
    # a reader of C queued on the stream right behind the step (no host synchronisation in between)
    return (C.view(torch.int16).to(torch.int64) * torch.arange(1, C.numel() + 1, device=dev).view_as(C)).sum()
def column_parallel_case(M, N, K, modes):
    global ok
    g = torch.Generator(device=dev).manual_seed(5)
    B = torch.randn(N, K, device=dev, generator=g)
    pb, sb = hk.quantize(B)
    # a different A for every step, and the single-GPU result of each whole problem
    ops, want = [], []
    for i in range(STEPS):
        pa, sa = hk.quantize(torch.randn(M, K, device=dev, generator=g))
        ops.append((pa, sa)); want.append(hk.gemm(pa, sa, pb, sb))
    want_digest = [digest(w) for w in want]
    pbs, sbs = shard_rows(pb, world, rank), shard_rows(sb, world, rank)
    for mode, depth, kw in modes:
        op = ColumnParallelGemm(M, N, K, device=dev, gather=mode, depth=depth, **kw)
        ok = ok and op.mode == mode
        got = []
        for i in range(STEPS):
            C = op(ops[i][0], ops[i][1], pbs, sbs)
            got.append(digest(C))                 # the next step follows without waiting for this reader on the host
            if rank == i % world:
                torch.cuda._sleep(2000000)        # one rank falls behind: its peers run ahead into the next step
        torch.cuda.synchronize()
        ok = ok and all(int(a) == int(b) for a, b in zip(got, want_digest))
        ok = ok and bool(torch.equal(C.view(torch.int16), want[-1].view(torch.int16)))
    return ops, want, pb, sb
M, N, K = 512, 2048, 1024
ops, want, pb, sb = column_parallel_case(M, N, K, (("nccl", 2, {}), ("fused", 2, {}), ("fused", 1, {})))
# a shard large enough for the CTA-pair kernel (2 row groups, ragged column strips, sliced last wave): the exchange by
# copy engines behind per-block flags, with one and with two copy streams per peer
column_parallel_case(4352, 2 * 2304, 512, (("copy", 2, dict(strip_tiles=4)), ("copy", 1, dict(strip_tiles=2, streams_per_peer=1)),
                                           ("fused", 2, {})))
for gth, depth in ((False, 2), (True, 2), (True, 1)):
    rp = RowParallelGemm(M, N, K, device=dev, gather=gth, depth=depth)
    got = []
    for i in range(STEPS):
        out = rp(shard_rows(ops[i][0], world, rank), shard_rows(ops[i][1], world, rank), pb, sb)
        exp = want[i] if gth else want[i][rp.lo:rp.hi]
        got.append((digest(out.contiguous()), digest(exp.contiguous())))
        if rank == i % world:
            torch.cuda._sleep(2000000)
    torch.cuda.synchronize()
    ok = ok and all(int(a) == int(b) for a, b in got)
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
