"""Running INT8 layers on activations that live in host memory.

A layer call on host data is three transfers in a row -- input to the device, kernels, output
back -- and the two copy directions use different DMA engines.  ``HostPipeline`` keeps one
stream per engine (host->device, compute, device->host) and chains them with events, so the
upload of request i+1 and the download of request i-1 run under the kernels of request i.
Host tensors must be pinned for the copies to be asynchronous.
"""
from __future__ import annotations

from typing import Callable, Sequence

import torch


class HostPipeline:
    def __init__(self, device):
        self.device = torch.device(device)
        self.s_in = torch.cuda.Stream(device=self.device)
        self.s_run = torch.cuda.Stream(device=self.device)
        self.s_out = torch.cuda.Stream(device=self.device)

    def run(self, fns: Sequence[Callable[[torch.Tensor], torch.Tensor]],
            host_in: Sequence[torch.Tensor], host_out: Sequence[torch.Tensor]) -> None:
        """``host_out[i].copy_(fns[i](host_in[i] on the device))`` for every i, pipelined.
        Returns once everything is enqueued; call ``synchronize()`` (or wait on the streams)
        before reading ``host_out``."""
        cur = torch.cuda.current_stream(self.device)
        for s in (self.s_in, self.s_run, self.s_out):
            s.wait_stream(cur)
        for fn, hx, hy in zip(fns, host_in, host_out):
            with torch.cuda.stream(self.s_in):
                xd = hx.to(self.device, non_blocking=True)
                up = torch.cuda.Event()
                up.record(self.s_in)
            with torch.cuda.stream(self.s_run):
                self.s_run.wait_event(up)
                xd.record_stream(self.s_run)
                y = fn(xd)
                done = torch.cuda.Event()
                done.record(self.s_run)
            with torch.cuda.stream(self.s_out):
                self.s_out.wait_event(done)
                y.record_stream(self.s_out)
                hy.copy_(y, non_blocking=True)
        for s in (self.s_in, self.s_run, self.s_out):
            cur.wait_stream(s)

    def synchronize(self) -> None:
        for s in (self.s_in, self.s_run, self.s_out):
            s.synchronize()
