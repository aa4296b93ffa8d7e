"""Double-buffered host-to-device input feeder.

A serving loop that receives every step's activations from the host pays the
PCIe copy on the critical path unless the copy of step i+1 runs while step i
computes.  ``HostFeeder`` keeps two device buffers and a copy stream: ``next()``
returns the device tensor holding the batch submitted one call earlier and
starts the copy of the batch passed now."""
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
