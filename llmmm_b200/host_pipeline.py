"""FP8 blockwise GEMM on host-resident operands, the way the reference's example
program runs it (examples/005.fp8.mm.cu:2700-2860: cudaMemcpy in, launch,
cudaMemcpy out), but with the three phases of successive calls overlapped.

A call copies A_q, A_s, B_q, B_s from (pinned) host memory to the device,
launches the GEMM through the C ABI and copies C_q, C_s back.  Each phase has its
own stream and the device buffers exist `depth` times, so the host->device copy
of call i+1 (one copy engine), the kernel of call i and the device->host copy of
call i-1 (the other copy engine) run at the same time; a stream of calls then
costs max(copy in, kernel, copy out) per call instead of their sum.  All kernels
run on one stream, in order, so they can share one registered scratch buffer.
"""
from __future__ import annotations

import torch

from . import capi


class Fp8GemmHostPipeline:
    """`submit()` enqueues one GEMM on host operands and returns at once;
    `drain()` waits until every result has landed in its host buffers."""

    def __init__(self, M: int, N: int, K: int, depth: int = 2, device=None):
        if M < 1 or N % 128 or K % 128:
            raise RuntimeError(f"M or N or K are not aligned. (need M>=1, N%128==0, K%128==0; got {M} {N} {K})")
        self.M, self.N, self.K, self.depth = M, N, K, depth
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        capi.lib()  # fails loudly if the CUDA library is missing
        with torch.cuda.device(self.device):
            capi.ensure_workspace(M, N, K, self.device)
            dev = self.device
            self.slots = []
            for _ in range(depth):
                self.slots.append({
                    "A_q": torch.empty(M, K, dtype=torch.uint8, device=dev),
                    "A_s": torch.empty(K // 128, M, dtype=torch.float32, device=dev),
                    "B_q": torch.empty(N, K, dtype=torch.uint8, device=dev),
                    "B_s": torch.empty(N // 128, K // 128, dtype=torch.float32, device=dev),
                    "C_q": torch.empty(M, N, dtype=torch.uint8, device=dev),
                    "C_s": torch.empty(N // 128, M, dtype=torch.float32, device=dev),
                    "loaded": torch.cuda.Event(), "computed": torch.cuda.Event(), "stored": torch.cuda.Event(),
                    "used": False,
                })
            self.s_in, self.s_mm, self.s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev), torch.cuda.Stream(dev)
        self.calls = 0
        self.h2d_bytes = M * K + 4 * (K // 128) * M + N * K + 4 * (N // 128) * (K // 128)
        self.d2h_bytes = M * N + 4 * (N // 128) * M

    def submit(self, A_q, A_s, B_q, B_s, C_q, C_s) -> None:
        """Host tensors (pinned for the copies to be asynchronous); layouts as in the C ABI.  The output
        tensors must not be read before `drain()` (or a later `submit` that reuses them) returns."""
        M, N, K = self.M, self.N, self.K
        slot = self.slots[self.calls % self.depth]
        self.calls += 1
        with torch.cuda.device(self.device):
            with torch.cuda.stream(self.s_in):
                if slot["used"]:
                    self.s_in.wait_event(slot["computed"])  # the kernel that read these buffers last
                slot["A_q"].copy_(A_q, non_blocking=True)
                slot["A_s"].copy_(A_s, non_blocking=True)
                slot["B_q"].copy_(B_q, non_blocking=True)
                slot["B_s"].copy_(B_s, non_blocking=True)
                slot["loaded"].record(self.s_in)
            self.s_mm.wait_event(slot["loaded"])
            if slot["used"]:
                self.s_mm.wait_event(slot["stored"])  # the copy-out that read this slot's C last
            capi.fp8_blockwise_mm(slot["A_q"], slot["A_s"], slot["B_q"], slot["B_s"], slot["C_q"], slot["C_s"],
                                  M, N, K, stream=self.s_mm)
            slot["computed"].record(self.s_mm)
            with torch.cuda.stream(self.s_out):
                self.s_out.wait_event(slot["computed"])
                C_q.copy_(slot["C_q"], non_blocking=True)
                C_s.copy_(slot["C_s"], non_blocking=True)
                slot["stored"].record(self.s_out)
            slot["used"] = True

    def drain(self) -> None:
        with torch.cuda.device(self.device):
            self.s_in.synchronize()
            self.s_mm.synchronize()
            self.s_out.synchronize()
            capi.check_status(self.s_mm)
