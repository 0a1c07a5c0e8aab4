"""Layer calls over batches that live in pinned host memory.

``HostStreamer`` keeps a small ring of device buffers and three CUDA streams: batch k+1 is copied to the
device and batch k-1 is copied back while batch k runs, so a stream of host batches costs about
max(compute, copy) per batch instead of their sum.  Every batch is still copied in and out in full; the
layer call itself is the ordinary module ``forward``.
"""
from __future__ import annotations

import torch


class HostStreamer:
    def __init__(self, layer, tokens: int, hidden: int, device, depth: int = 2, dtype=torch.bfloat16):
        self.layer, self.depth = layer, depth
        self.device = torch.device(device)
        self.h2d, self.compute, self.d2h = (torch.cuda.Stream(self.device) for _ in range(3))
        self.x_dev = [torch.empty(1, tokens, hidden, dtype=dtype, device=self.device) for _ in range(depth)]
        self.y_dev = [torch.empty(1, tokens, hidden, dtype=dtype, device=self.device) for _ in range(depth)]
        mk = lambda: [torch.cuda.Event() for _ in range(depth)]   # noqa: E731
        self.x_ready, self.x_free, self.y_ready, self.y_free = mk(), mk(), mk(), mk()
        self.k = 0
        cur = torch.cuda.current_stream(self.device)
        for s in (self.h2d, self.compute, self.d2h):
            s.wait_stream(cur)

    @torch.no_grad()
    def submit(self, x_host: torch.Tensor, y_host: torch.Tensor) -> None:
        """Queue one batch: x_host (tokens, hidden) pinned -> layer -> y_host (tokens, hidden) pinned."""
        i, first = self.k % self.depth, self.k < self.depth
        with torch.cuda.stream(self.h2d):
            if not first:
                self.h2d.wait_event(self.x_free[i])
            self.x_dev[i][0].copy_(x_host, non_blocking=True)
            self.x_ready[i].record(self.h2d)
        with torch.cuda.stream(self.compute):
            self.compute.wait_event(self.x_ready[i])
            if not first:
                self.compute.wait_event(self.y_free[i])
            self.y_dev[i].copy_(self.layer(self.x_dev[i]))
            self.x_free[i].record(self.compute)
            self.y_ready[i].record(self.compute)
        with torch.cuda.stream(self.d2h):
            self.d2h.wait_event(self.y_ready[i])
            y_host.copy_(self.y_dev[i][0], non_blocking=True)
            self.y_free[i].record(self.d2h)
        self.k += 1

    def join(self) -> None:
        """Make the current stream wait for everything queued so far."""
        cur = torch.cuda.current_stream(self.device)
        for s in (self.h2d, self.compute, self.d2h):
            cur.wait_stream(s)
