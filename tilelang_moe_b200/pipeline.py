"""Host-side pipeline around a device step: inputs live in pinned host memory, results go back to pinned host
memory, and consecutive steps overlap their copies with each other's compute.

Three streams and two sets of device buffers: while step i computes, step i+1's inputs are uploaded on the copy-in
stream and step i-1's output is downloaded on the copy-out stream (the GPU has separate DMA engines for the two
directions).  Every step still uploads its own inputs and downloads its own result; only the waiting is hidden.
"""
from __future__ import annotations

from typing import Callable, List, Sequence

import torch


class HostPipeline:
    def __init__(self, device: torch.device, host_inputs: Sequence[torch.Tensor], out_shape, out_dtype: torch.dtype,
                 compute: Callable[..., None], depth: int = 2):
        """host_inputs: pinned host tensors uploaded every step.  compute(*device_inputs, out) must enqueue the
        step on the current stream and leave its result in ``out``."""
        for h in host_inputs:
            if not h.is_pinned():
                raise ValueError("host inputs must be pinned")
        self.device, self.host_inputs, self.compute, self.depth = device, list(host_inputs), compute, depth
        self.in_dev: List[List[torch.Tensor]] = [[torch.empty(h.shape, dtype=h.dtype, device=device) for h in host_inputs]
                                                 for _ in range(depth)]
        self.out_dev = [torch.empty(out_shape, dtype=out_dtype, device=device) for _ in range(depth)]
        self.out_host = [torch.empty(out_shape, dtype=out_dtype).pin_memory() for _ in range(depth)]
        self.s_in = torch.cuda.Stream(device=device)
        self.s_out = torch.cuda.Stream(device=device)
        self.h2d_bytes = sum(h.numel() * h.element_size() for h in host_inputs)
        self.d2h_bytes = self.out_host[0].numel() * self.out_host[0].element_size()

    def run(self, steps: int) -> torch.Tensor:
        """Enqueue `steps` pipelined steps; on return the current stream has waited for the last download.
        Returns the pinned host tensor holding the last step's result."""
        cur = torch.cuda.current_stream(self.device)
        self.s_in.wait_stream(cur)
        self.s_out.wait_stream(cur)
        ev_c = [None] * self.depth     # compute of the step that last used buffer b
        ev_out = [None] * self.depth   # download of that step's output
        for i in range(steps):
            b = i % self.depth
            with torch.cuda.stream(self.s_in):
                if ev_c[b] is not None:
                    self.s_in.wait_event(ev_c[b])            # the step that read these input buffers is done
                for d, h in zip(self.in_dev[b], self.host_inputs):
                    d.copy_(h, non_blocking=True)
                ev_in = torch.cuda.Event()
                ev_in.record(self.s_in)
            cur.wait_event(ev_in)
            if ev_out[b] is not None:
                cur.wait_event(ev_out[b])                    # this output buffer has been drained
            self.compute(*self.in_dev[b], self.out_dev[b])
            ev_c[b] = torch.cuda.Event()
            ev_c[b].record(cur)
            with torch.cuda.stream(self.s_out):
                self.s_out.wait_event(ev_c[b])
                self.out_host[b].copy_(self.out_dev[b], non_blocking=True)
                ev_out[b] = torch.cuda.Event()
                ev_out[b].record(self.s_out)
        for e in ev_out:
            if e is not None:
                cur.wait_event(e)
        return self.out_host[(steps - 1) % self.depth]
