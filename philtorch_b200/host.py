"""Host-buffer entry points: inputs and outputs live in (pinned) host memory.

The reference runs this path on CPU tensors; a caller that keeps its signals in host memory can
call these functions instead and get the GPU kernels with the transfers overlapped: rows are
independent, so the batch is cut into row blocks and block k+1 is uploaded while block k is
computed and block k-1 is downloaded (three CUDA streams, PCIe in both directions at once).
"""
from __future__ import annotations

from typing import Optional

import torch
from torch import Tensor

from . import ops  # noqa: F401

_ops = torch.ops.philtorch_b200


def _pinned_like(t: Tensor) -> Tensor:
    return torch.empty(t.shape, dtype=t.dtype, pin_memory=True)


class HostPipeline:
    """Reusable staging for first-order per-sample-coefficient forward+backward on host buffers.

    ``run(a, zi, x, gy, out)`` computes y, grad_a, grad_zi, grad_x of
    ``lpv.linear_recurrence`` for host tensors ``a, x, gy`` of shape (B, T) and ``zi`` (B,),
    writing into the host tensors of ``out`` (dict with keys y, grad_a, grad_zi, grad_x).
    All host tensors should be pinned; device staging buffers are allocated once.

    ``rows_per_block``: the first block's upload and the last block's download overlap nothing, so
    small blocks waste less of the link (B=256, T=2^20, fp32 on a Gen5 x16 link whose two directions
    together sustain 66 ms for these 2 x 3.2 GB: 8 rows per block 69.5 ms, 32 rows 72.1 ms, 64 rows
    78.0 ms); below 8 the host-side launch work per block starts to show.
    """

    def __init__(self, B: int, T: int, dtype=torch.float32, device="cuda", rows_per_block: int = 8):
        self.B, self.T = B, T
        self.device = torch.device(device)
        self.rows = max(1, min(rows_per_block, B))
        self.nblk = (B + self.rows - 1) // self.rows
        self.nbuf = min(3, self.nblk)
        mk = lambda *s: torch.empty(*s, dtype=dtype, device=self.device)
        self.bufs = [dict(a=mk(self.rows, T), x=mk(self.rows, T), gy=mk(self.rows, T), zi=mk(self.rows))
                     for _ in range(self.nbuf)]
        self.s_in = torch.cuda.Stream(self.device)
        self.s_cmp = torch.cuda.Stream(self.device)
        self.s_out = torch.cuda.Stream(self.device)
        self.h2d_bytes = 0
        self.d2h_bytes = 0

    def run(self, a: Tensor, zi: Tensor, x: Tensor, gy: Tensor, out: dict) -> None:
        B, rows = self.B, self.rows
        esz = a.element_size()
        self.h2d_bytes = (a.numel() + x.numel() + gy.numel() + zi.numel()) * esz
        self.d2h_bytes = (3 * x.numel() + zi.numel()) * esz
        cur = torch.cuda.current_stream(self.device)
        for s in (self.s_in, self.s_cmp, self.s_out):
            s.wait_stream(cur)
        free_ev: list[Optional[torch.cuda.Event]] = [None] * self.nbuf   # staging buffer reusable
        keep = []
        for k in range(self.nblk):
            r0, r1 = k * rows, min(B, (k + 1) * rows)
            n = r1 - r0
            buf = self.bufs[k % self.nbuf]
            with torch.cuda.stream(self.s_in):
                if free_ev[k % self.nbuf] is not None:
                    self.s_in.wait_event(free_ev[k % self.nbuf])
                buf["a"][:n].copy_(a[r0:r1], non_blocking=True)
                buf["x"][:n].copy_(x[r0:r1], non_blocking=True)
                buf["gy"][:n].copy_(gy[r0:r1], non_blocking=True)
                buf["zi"][:n].copy_(zi[r0:r1], non_blocking=True)
                up = torch.cuda.Event()
                up.record(self.s_in)
            with torch.cuda.stream(self.s_cmp):
                self.s_cmp.wait_event(up)
                ab, zb, xb, gb = buf["a"][:n], buf["zi"][:n], buf["x"][:n], buf["gy"][:n]
                y = _ops.lpv_recur(ab, zb, xb)
                ga, gzi, gx = _ops.lpv_recur_bwd(ab, zb, y, gb, None, True, True)
                done = torch.cuda.Event()
                done.record(self.s_cmp)
                free_ev[k % self.nbuf] = done
            with torch.cuda.stream(self.s_out):
                self.s_out.wait_event(done)
                out["y"][r0:r1].copy_(y, non_blocking=True)
                out["grad_a"][r0:r1].copy_(ga, non_blocking=True)
                out["grad_x"][r0:r1].copy_(gx, non_blocking=True)
                out["grad_zi"][r0:r1].copy_(gzi, non_blocking=True)
                for t in (y, ga, gx, gzi):
                    t.record_stream(self.s_out)
            keep.append((y, ga, gx, gzi))
        cur.wait_stream(self.s_out)
        cur.wait_stream(self.s_cmp)


def linear_recurrence_fwd_bwd_host(a: Tensor, zi: Tensor, x: Tensor, gy: Tensor, device="cuda",
                                   rows_per_block: int = 8) -> dict:
    """One-shot convenience wrapper around :class:`HostPipeline` (allocates pinned outputs)."""
    B, T = x.shape
    pipe = HostPipeline(B, T, x.dtype, device, rows_per_block)
    out = dict(y=_pinned_like(x), grad_a=_pinned_like(x), grad_x=_pinned_like(x), grad_zi=_pinned_like(zi))
    pipe.run(a, zi, x, gy, out)
    torch.cuda.synchronize(pipe.device)
    return out
