"""Host-to-device staging of training batches on a side stream.

The reference's loader thread copies every batch from pinned memory on its
own CUDA stream and the training loop picks it up with `record_stream`
(data_loader/dataset.py:290-327,366-371 of the reference project).
`DevicePrefetcher` is the same idea without a thread: while step i runs on
the compute stream, batch i+1 travels on the copy stream into the other half
of a double buffer.
"""

from __future__ import annotations

from collections.abc import Iterable, Iterator

import torch


class DevicePrefetcher:
    """Wraps an iterable of tuples of pinned CPU tensors; yields tuples of CUDA
    tensors whose copy was issued one iteration earlier."""

    def __init__(self, batches: Iterable[tuple[torch.Tensor, ...]], device: torch.device, depth: int = 2,
                 copy_stream: torch.cuda.Stream | None = None):
        self.batches = batches
        self.device = device
        self.depth = max(2, depth)
        self.copy_stream = copy_stream if copy_stream is not None else torch.cuda.Stream(device)

    def _issue(self, host_batch, slot):
        compute = torch.cuda.current_stream(self.device)
        # the slot's previous tensors may still be read by kernels of an earlier step
        self.copy_stream.wait_stream(compute)
        with torch.cuda.stream(self.copy_stream):
            dev = tuple(t.to(self.device, non_blocking=True) for t in host_batch)
            ready = torch.cuda.Event()
            ready.record(self.copy_stream)
        return dev, ready

    def __iter__(self) -> Iterator[tuple[torch.Tensor, ...]]:
        it = iter(self.batches)
        pending = []
        try:
            for _ in range(self.depth - 1):
                pending.append(self._issue(next(it), len(pending)))
        except StopIteration:
            pass
        while pending:
            dev, ready = pending.pop(0)
            try:
                pending.append(self._issue(next(it), 0))
            except StopIteration:
                pass
            compute = torch.cuda.current_stream(self.device)
            compute.wait_event(ready)
            for t in dev:
                t.record_stream(compute)  # allocated on the copy stream, consumed on the compute stream
            yield dev
