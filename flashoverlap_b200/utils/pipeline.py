"""Double-buffered host-to-device input feeder and device-to-host result reader.

A serving loop that receives every step's activations from the host pays the
PCIe copy on the critical path unless the copy of step i+1 runs while step i
computes.  ``HostFeeder`` keeps two device buffers and a copy stream: ``take()``
returns the device tensor holding the batch submitted last and ``submit()``
starts the copy of the next one.  ``ResultReader`` does the same in the other
direction: the result of step i travels to pinned host memory while step i+1
computes."""
from __future__ import annotations

from typing import Optional

import torch


class HostFeeder:
    def __init__(self, shape, dtype, device=None):
        self.device = device if device is not None else torch.device("cuda", torch.cuda.current_device())
        self.bufs = [torch.empty(shape, dtype=dtype, device=self.device) for _ in range(2)]
        self.ready = [torch.cuda.Event(), torch.cuda.Event()]
        self.consumed = [torch.cuda.Event(), torch.cuda.Event()]
        self.copy_stream = torch.cuda.Stream(device=self.device)
        self.slot = 0
        self.primed = False

    def submit(self, host_tensor: torch.Tensor) -> None:
        """Start copying ``host_tensor`` (pinned memory) into the free buffer."""
        s = self.slot
        with torch.cuda.stream(self.copy_stream):
            if self.primed:
                self.copy_stream.wait_event(self.consumed[s])  # the compute stream is done with this buffer
            self.bufs[s].copy_(host_tensor, non_blocking=True)
            self.ready[s].record(self.copy_stream)
        self.pending = s
        self.slot ^= 1

    def take(self) -> torch.Tensor:
        """Device tensor of the last submitted batch; the current stream waits for its copy."""
        s = self.pending
        torch.cuda.current_stream().wait_event(self.ready[s])
        return self.bufs[s]

    def release(self, slot_tensor: torch.Tensor) -> None:
        """Tell the feeder that the work reading ``slot_tensor`` has been enqueued."""
        s = 0 if slot_tensor.data_ptr() == self.bufs[0].data_ptr() else 1
        self.consumed[s].record(torch.cuda.current_stream())
        self.primed = True


class ResultReader:
    """Copies every step's result into one of two pinned host buffers on a
    copy stream of its own.

    The fused all-reduce returns a tensor that aliases one of two alternating
    symmetric result buffers, so the copy of step i must have finished before
    step i+2 overwrites that buffer: call ``before_step()`` before launching a
    step, ``fetch(result)`` after it, and ``wait_all()`` before reading the
    host buffers."""

    def __init__(self, shape, dtype, device=None):
        self.device = device if device is not None else torch.device("cuda", torch.cuda.current_device())
        self.host = [torch.empty(shape, dtype=dtype).pin_memory() for _ in range(2)]
        self.done = [torch.cuda.Event(), torch.cuda.Event()]
        self.produced = torch.cuda.Event()
        self.copy_stream = torch.cuda.Stream(device=self.device)
        self.slot = 0
        self.used = [False, False]

    def before_step(self) -> None:
        """The step about to be launched may overwrite the device buffer that the
        copy issued two steps ago reads: make the current stream wait for it."""
        if self.used[self.slot]:
            torch.cuda.current_stream().wait_event(self.done[self.slot])

    def fetch(self, result: torch.Tensor) -> torch.Tensor:
        """Start copying ``result`` to the host once the work enqueued so far on
        the current stream is done.  Returns the host buffer it will land in."""
        s = self.slot
        if self.used[s]:
            self.done[s].synchronize()  # the host buffer still holds the result of two steps ago
        self.produced.record(torch.cuda.current_stream())
        with torch.cuda.stream(self.copy_stream):
            self.copy_stream.wait_event(self.produced)
            self.host[s].copy_(result, non_blocking=True)
            self.done[s].record(self.copy_stream)
        self.used[s] = True
        self.slot ^= 1
        return self.host[s]

    def wait_all(self) -> None:
        for s in range(2):
            if self.used[s]:
                self.done[s].synchronize()
