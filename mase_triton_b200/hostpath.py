"""Host-buffer front end: run a quantisation op on tensors that live in (pinned) host memory.

The tensor is cut into row chunks; chunk i+1 is copied to the device while chunk i is computed
and chunk i-1 is copied back, on three CUDA streams, so PCIe traffic in both directions overlaps
the kernels.  Only two device staging buffers per direction are held, whatever the tensor size.
"""

from __future__ import annotations

from typing import Callable

import torch
from torch import Tensor


class HostPipeline:
    """``run(x_host, out_host)`` applies ``op(x_dev, out_dev)`` (which must write its result into
    ``out_dev``) chunk by chunk.  ``x_host`` and ``out_host`` should be pinned for the copies to be
    asynchronous."""

    def __init__(self, op: Callable[[Tensor, Tensor], None], device: torch.device | str = "cuda", chunk_rows: int = 1024):
        self.op = op
        self.device = torch.device(device)
        self.chunk_rows = chunk_rows
        self.s_in = torch.cuda.Stream(self.device)
        self.s_run = torch.cuda.Stream(self.device)
        self.s_out = torch.cuda.Stream(self.device)
        self._stage = None
        self.launches = 0

    def _staging(self, rows: int, cols: int, in_dtype, out_dtype):
        key = (rows, cols, in_dtype, out_dtype)
        if self._stage is None or self._stage[0] != key:
            mk = lambda dt: [torch.empty((rows, cols), dtype=dt, device=self.device) for _ in range(2)]  # noqa: E731
            self._stage = (key, mk(in_dtype), mk(out_dtype))
        return self._stage[1], self._stage[2]

    def run(self, x_host: Tensor, out_host: Tensor) -> None:
        assert x_host.ndim == 2 and x_host.shape == out_host.shape
        rows, cols = x_host.shape
        cr = min(self.chunk_rows, rows)
        d_in, d_out = self._staging(cr, cols, x_host.dtype, out_host.dtype)
        n_chunks = (rows + cr - 1) // cr
        in_ready = [torch.cuda.Event() for _ in range(2)]
        run_done = [torch.cuda.Event() for _ in range(2)]
        out_done = [torch.cuda.Event() for _ in range(2)]
        cur = torch.cuda.current_stream(self.device)
        for s in (self.s_in, self.s_run, self.s_out):
            s.wait_stream(cur)
        for c in range(n_chunks):
            b = c & 1
            r0, r1 = c * cr, min(rows, (c + 1) * cr)
            n = r1 - r0
            with torch.cuda.stream(self.s_in):
                if c >= 2:
                    self.s_in.wait_event(run_done[b])        # staging buffer b is free again
                d_in[b][:n].copy_(x_host[r0:r1], non_blocking=True)
                in_ready[b].record(self.s_in)
            with torch.cuda.stream(self.s_run):
                self.s_run.wait_event(in_ready[b])
                if c >= 2:
                    self.s_run.wait_event(out_done[b])
                self.op(d_in[b][:n], d_out[b][:n])
                run_done[b].record(self.s_run)
                self.launches += 1
            with torch.cuda.stream(self.s_out):
                self.s_out.wait_event(run_done[b])
                out_host[r0:r1].copy_(d_out[b][:n], non_blocking=True)
                out_done[b].record(self.s_out)
        for s in (self.s_in, self.s_run, self.s_out):
            cur.wait_stream(s)
