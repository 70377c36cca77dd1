"""Host-buffer entry: run an operator of ``ops`` on operands that live in pinned host
memory, with the host->device copies, the kernel and the device->host copy of the
result on three streams and two buffer slots, so that consecutive calls overlap
(copy-in of step i+1, kernel of step i, copy-out of step i-1).

PyTorch provides the device buffers, streams and events; the arithmetic is the
C-ABI kernel that ``launch`` calls.
"""
from __future__ import annotations

import torch


class HostPipeline:
    """``launch(dev_inputs, dev_outputs)`` enqueues the operator on the current stream.

    ``inputs`` / ``outputs`` are example tensors (shape and dtype are taken from them;
    their device is the device to run on)."""

    def __init__(self, launch, inputs, outputs, slots: int = 2, broadcast=None):
        """``broadcast`` = (input indices, torch.distributed module) for operands that are identical on every rank: rank 0
        uploads them from its host buffer and an NCCL broadcast over NVLink delivers them to the other ranks, whose
        ``host_inputs`` entries for these indices are ``None`` (one PCIe upload per job instead of one per rank)."""
        self.launch = launch
        self.bcast_idx = set(broadcast[0]) if broadcast else set()
        self.dist = broadcast[1] if broadcast else None
        self.device = inputs[0].device
        self.slots = slots
        self.dev_in = [[torch.empty_like(t) for t in inputs] for _ in range(slots)]
        self.dev_out = [[torch.empty_like(t) for t in outputs] for _ in range(slots)]
        self.s_in = torch.cuda.Stream(self.device)
        self.s_run = torch.cuda.Stream(self.device)
        self.s_out = torch.cuda.Stream(self.device)
        self.ev_in = [torch.cuda.Event() for _ in range(slots)]
        self.ev_run = [torch.cuda.Event() for _ in range(slots)]
        self.ev_out = [torch.cuda.Event() for _ in range(slots)]
        self.count = 0

    def submit(self, host_inputs, host_outputs) -> None:
        """Enqueue one step: pinned host operands in, pinned host results out (asynchronous)."""
        k = self.count % self.slots
        first_use = self.count < self.slots
        self.count += 1
        with torch.cuda.stream(self.s_in):
            if not first_use:
                self.s_in.wait_event(self.ev_run[k])       # the kernel that read this slot's inputs is done
            for i, (d, h) in enumerate(zip(self.dev_in[k], host_inputs)):
                if h is not None:
                    d.copy_(h, non_blocking=True)
                if i in self.bcast_idx:
                    self.dist.broadcast(d, src=0)      # enqueued behind the upload on this stream
            self.ev_in[k].record(self.s_in)
        with torch.cuda.stream(self.s_run):
            self.s_run.wait_event(self.ev_in[k])
            if not first_use:
                self.s_run.wait_event(self.ev_out[k])      # this slot's previous result has left the device
            self.launch(self.dev_in[k], self.dev_out[k])
            self.ev_run[k].record(self.s_run)
        with torch.cuda.stream(self.s_out):
            self.s_out.wait_event(self.ev_run[k])
            for h, d in zip(host_outputs, self.dev_out[k]):
                h.copy_(d, non_blocking=True)
            self.ev_out[k].record(self.s_out)

    def drain(self) -> None:
        """Wait until every submitted step has delivered its result to host memory."""
        self.s_out.synchronize()
        self.s_run.synchronize()
        self.s_in.synchronize()

    def record_done(self, event: torch.cuda.Event) -> None:
        """Record `event` after everything submitted so far, on the output stream."""
        self.s_out.wait_stream(self.s_run)
        self.s_out.wait_stream(self.s_in)
        event.record(self.s_out)
