"""Double-buffered host <-> device pipeline around a perception step.

When particle systems live in host memory (a data loader, a CPU simulation that consumes the
gradients), the host->device copy of the next batch and the device->host copy of the previous
results can run on the copy engines while the current batch is in the kernels.  This helper runs
``step(inputs_on_device) -> outputs_on_device`` over a sequence of pinned host batches with the
three stages on three CUDA streams and ``depth`` device buffers in flight.
"""
from __future__ import annotations

from typing import Callable, Iterable, List, Sequence

import torch


class HostStepPipeline:
    """Overlaps H2D copies, ``step`` and D2H copies of consecutive batches.

    ``example_inputs`` / ``example_outputs`` are sequences of tensors that fix shapes and dtypes
    (host or device, only metadata is used).  ``run`` takes an iterable of batches, each a sequence
    of pinned host tensors, and a callback ``consume(index, outputs_host)`` that is called once a
    batch's results are complete in pinned host memory (the tensors are reused ``depth`` batches
    later, so copy what must be kept).
    """

    def __init__(self, step: Callable[[Sequence[torch.Tensor]], Sequence[torch.Tensor]],
                 example_inputs: Sequence[torch.Tensor], example_outputs: Sequence[torch.Tensor],
                 device=None, depth: int = 2):
        if depth < 1:
            raise ValueError("depth must be at least 1")
        self.step = step
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self.depth = depth
        self.h2d = torch.cuda.Stream(self.device)
        self.d2h = torch.cuda.Stream(self.device)
        self.in_dev = [[torch.empty(t.shape, dtype=t.dtype, device=self.device) for t in example_inputs]
                       for _ in range(depth)]
        self.out_host = [[torch.empty(t.shape, dtype=t.dtype).pin_memory() for t in example_outputs]
                         for _ in range(depth)]
        self.loaded = [torch.cuda.Event() for _ in range(depth)]     # inputs of the slot are on the device
        self.computed = [torch.cuda.Event() for _ in range(depth)]   # step of the slot has been enqueued/finished
        self.stored = [torch.cuda.Event() for _ in range(depth)]     # outputs of the slot are in host memory

    def run(self, batches: Iterable[Sequence[torch.Tensor]], consume: Callable[[int, List[torch.Tensor]], None] = None):
        compute = torch.cuda.current_stream(self.device)
        pending = []  # (index, slot) whose outputs are still in flight
        count = 0
        for n, batch in enumerate(batches):
            count += 1
            slot = n % self.depth
            if n >= self.depth:
                # the slot is reused: its previous outputs must have reached the host ...
                idx, sl = pending.pop(0)
                self.stored[sl].synchronize()
                if consume is not None:
                    consume(idx, self.out_host[sl])
                # ... and its previous step must be done with the input buffers
                self.h2d.wait_event(self.computed[slot])
            with torch.cuda.stream(self.h2d):
                for dst, src in zip(self.in_dev[slot], batch):
                    dst.copy_(src, non_blocking=True)
                self.loaded[slot].record(self.h2d)
            compute.wait_event(self.loaded[slot])
            outs = self.step(self.in_dev[slot])
            self.computed[slot].record(compute)
            self.d2h.wait_event(self.computed[slot])
            with torch.cuda.stream(self.d2h):
                for dst, src in zip(self.out_host[slot], outs):
                    src.record_stream(self.d2h)
                    dst.copy_(src, non_blocking=True)
                self.stored[slot].record(self.d2h)
            pending.append((n, slot))
        for idx, sl in pending:
            self.stored[sl].synchronize()
            if consume is not None:
                consume(idx, self.out_host[sl])
        return count
