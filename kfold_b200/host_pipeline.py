"""Host-resident inputs and outputs around a device function, with the copies of neighbouring items overlapped.

K-Fold's drivers hold the features of a complex in host memory and read the results back to the host
(src/kfold/cli/predict.py builds its batches on the CPU and `.to(device)`s them).  When several items are processed one
after another -- complexes of a batch job, or the blocks of a benchmark loop -- the host-to-device copy of item i+1 and
the device-to-host copy of item i-1 can run under the compute of item i: PCIe is full duplex and the copy engines are
separate from the SMs.  `HostPipeline` does exactly that with three CUDA streams; every item is still copied in from
pinned host memory and its result copied out, nothing is cached between items.
"""
from __future__ import annotations

import torch

__all__ = ["HostPipeline"]


class HostPipeline:
    """``fn(*device_inputs) -> tensor or tuple of tensors`` over pinned host inputs.

    `run(inputs, outputs)`: `inputs` is a sequence of tuples of pinned host tensors, `outputs` a sequence of tuples of
    pinned host tensors that receive the results (same count and shapes as `fn` returns).  Returns when every copy has
    been *enqueued*; the calling stream waits for the last device-to-host copy, so a synchronisation (or an event) on it
    covers the whole run.  At most `depth` items are in flight (their inputs live on the device at the same time).
    """

    def __init__(self, fn, device, depth: int = 2):
        if depth < 1:
            raise ValueError("depth must be at least 1")
        self.fn, self.device, self.depth = fn, torch.device(device), depth
        self._h2d = torch.cuda.Stream(self.device)
        self._d2h = torch.cuda.Stream(self.device)

    def run(self, inputs, outputs) -> None:
        if len(inputs) != len(outputs):
            raise ValueError("one tuple of output buffers per tuple of inputs")
        for item in list(inputs) + list(outputs):
            for t in item:
                if not t.is_pinned():
                    raise ValueError("HostPipeline needs pinned host tensors (the copies would not be asynchronous)")
        compute = torch.cuda.current_stream(self.device)
        start = torch.cuda.Event()
        start.record(compute)
        self._h2d.wait_event(start)          # nothing of this run starts before earlier work on the calling stream
        self._d2h.wait_event(start)
        consumed = []                        # per item: event after the compute that read its inputs
        last_out = None
        for i, (ins, outs) in enumerate(zip(inputs, outputs)):
            with torch.cuda.stream(self._h2d):
                if i >= self.depth:
                    self._h2d.wait_event(consumed[i - self.depth])      # bound the device memory held by queued inputs
                dev_in = tuple(t.to(self.device, non_blocking=True) for t in ins)
                ready = torch.cuda.Event()
                ready.record(self._h2d)
            compute.wait_event(ready)
            for t in dev_in:
                t.record_stream(compute)
            res = self.fn(*dev_in)
            res = (res,) if isinstance(res, torch.Tensor) else tuple(res)
            if len(res) != len(outs):
                raise ValueError(f"fn returned {len(res)} tensors, {len(outs)} output buffers given")
            done = torch.cuda.Event()
            done.record(compute)
            consumed.append(done)
            with torch.cuda.stream(self._d2h):
                self._d2h.wait_event(done)
                for r, o in zip(res, outs):
                    r.record_stream(self._d2h)
                    o.copy_(r.reshape(o.shape), non_blocking=True)
                last_out = torch.cuda.Event()
                last_out.record(self._d2h)
        if last_out is not None:
            compute.wait_event(last_out)
