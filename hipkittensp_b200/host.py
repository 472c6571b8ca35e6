"""GEMM for callers whose operands and result live in (pinned) host memory.

`HostGemm` keeps two sets of device staging buffers and three CUDA streams (host->device, compute,
device->host): the copy-in of call i+1 and the copy-out of call i-1 overlap the kernel of call i, and the
two PCIe directions run at the same time.  Every call moves its own operands in and its own result out; calls
return as soon as the work is queued, `synchronize()` waits for all of it.  torch supplies the streams,
events and pinned-memory copies; the GEMM itself is the C ABI (`dispatch_micro`).
"""
from __future__ import annotations

import torch

from ._lib import E2M3, E4M3, E5M2
from .gemm import dispatch_micro


class HostGemm:
    def __init__(self, M: int, N: int, K: int, device="cuda:0", fmt: int = E2M3, depth: int = 2, gemm=None):
        self.M, self.N, self.K, self.fmt, self.depth = M, N, K, fmt, depth
        self.device = torch.device(device)
        u8 = dict(dtype=torch.uint8, device=self.device)
        row_bytes = K if fmt in (E4M3, E5M2) else K * 3 // 4      # one byte per fp8 element, 3 bytes per 4 fp6 elements
        self.slots = []
        for _ in range(depth):
            self.slots.append(dict(
                a=torch.empty((M, row_bytes), **u8), sa=torch.empty((M, K // 32), **u8),
                b=torch.empty((N, row_bytes), **u8), sb=torch.empty((N, K // 32), **u8),
                c=torch.empty((M, N), dtype=torch.bfloat16, device=self.device),
                loaded=torch.cuda.Event(), computed=torch.cuda.Event(), drained=torch.cuda.Event()))
        self.s_in = torch.cuda.Stream(self.device)
        self.s_mm = torch.cuda.Stream(self.device)
        self.s_out = torch.cuda.Stream(self.device)
        self.n = 0
        # gemm(slot) runs the kernel(s) of one call on the current stream and returns the tensor to copy out
        self._gemm = gemm or (lambda s: (dispatch_micro(s["a"], s["b"], s["c"], s["sa"], s["sb"], self.fmt), s["c"])[1])

    def __call__(self, a_host, sa_host, b_host, sb_host, out_host):
        """Queue one GEMM: operands from host tensors (pinned for true asynchrony), result into out_host."""
        s = self.slots[self.n % self.depth]
        first_use = self.n < self.depth
        with torch.cuda.stream(self.s_in):
            if not first_use:
                self.s_in.wait_event(s["computed"])      # the kernel that last read these buffers is done
            s["a"].copy_(a_host, non_blocking=True)
            s["sa"].copy_(sa_host, non_blocking=True)
            s["b"].copy_(b_host, non_blocking=True)
            s["sb"].copy_(sb_host, non_blocking=True)
            s["loaded"].record()
        with torch.cuda.stream(self.s_mm):
            self.s_mm.wait_event(s["loaded"])
            if not first_use:
                self.s_mm.wait_event(s["drained"])       # the previous result in this slot has left the device
            out_dev = self._gemm(s)
            s["computed"].record()
        with torch.cuda.stream(self.s_out):
            self.s_out.wait_event(s["computed"])
            out_host.copy_(out_dev, non_blocking=True)
            s["drained"].record()
        self.n += 1

    def synchronize(self):
        self.s_out.synchronize()
        self.s_mm.synchronize()
        self.s_in.synchronize()
