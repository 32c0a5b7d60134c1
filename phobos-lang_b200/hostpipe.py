"""Leaf calls on operands that live in host memory.

The reference's launchers take device pointers; a caller that holds its tensors in (pinned) host memory
pays an upload per operand and a download of the result around every call.  HostPipeline runs a sequence
of same-shaped calls so that the uploads of call i+1 and the download of call i-1 overlap the kernel of
call i: three CUDA streams (upload, compute, download), `depth` device buffer sets, events between them.
Every call still moves all of its operands and its result; only the waiting is shared.
"""
from __future__ import annotations


class HostPipeline:
    def __init__(self, torch, device, operand_specs, kernel, result_index: int, depth: int = 2):
        """operand_specs: [(shape, dtype), ...] of the device buffers of one call, in kernel argument order.
        kernel(*device_tensors, stream=...) enqueues the leaf.  result_index: which buffer holds the result."""
        self.torch, self.kernel, self.result_index, self.depth = torch, kernel, result_index, depth
        self.up, self.run, self.down = (torch.cuda.Stream(device=device) for _ in range(3))
        self.bufs = [[torch.empty(shape, dtype=dtype, device=device) for shape, dtype in operand_specs] for _ in range(depth)]
        self.uploaded = [torch.cuda.Event() for _ in range(depth)]
        self.computed = [torch.cuda.Event() for _ in range(depth)]
        self.released = [None] * depth      # download of the previous user of the slot
        self.n = 0

    def submit(self, host_operands, host_result) -> None:
        """host_operands: pinned host tensors, None for a buffer that is output only."""
        torch = self.torch
        slot = self.n % self.depth
        self.n += 1
        bufs = self.bufs[slot]
        with torch.cuda.stream(self.up):
            if self.released[slot] is not None:
                self.up.wait_event(self.released[slot])     # the slot's previous result has left the device
            for dst, src in zip(bufs, host_operands):
                if src is not None:
                    dst.copy_(src, non_blocking=True)
            self.uploaded[slot].record(self.up)
        with torch.cuda.stream(self.run):
            self.run.wait_event(self.uploaded[slot])
            self.kernel(*bufs, stream=self.run)
            self.computed[slot].record(self.run)
        with torch.cuda.stream(self.down):
            self.down.wait_event(self.computed[slot])
            host_result.copy_(bufs[self.result_index], non_blocking=True)
            ev = torch.cuda.Event()
            ev.record(self.down)
            self.released[slot] = ev

    def join(self, stream=None) -> None:
        """Makes `stream` (default: the current stream) wait for everything submitted so far."""
        torch = self.torch
        stream = stream or torch.cuda.current_stream()
        for s in (self.up, self.run, self.down):
            ev = torch.cuda.Event()
            ev.record(s)
            stream.wait_event(ev)
