"""Double-buffered staging of host inputs for a sequence of attention steps.

A training step of the non-absorbed path reads 2.4 GB of inputs (C3: B=2, S=8192, H=128) and
runs for about 23 ms on a B200, while copying those inputs from pinned host memory takes about
twice as long.  A caller that copies, computes and copies again on one stream therefore spends
two thirds of its time on the bus with the tensor cores idle.  `HostPipeline` keeps two sets of
device buffers and a copy stream, so that the copy of step i+1 runs while step i computes:

    pipe = HostPipeline(example_inputs, device)
    pipe.stage(host_inputs[0])
    for i in range(steps):
        if i + 1 < steps:
            pipe.stage(host_inputs[i + 1])
        x = pipe.acquire()                 # the compute stream now waits for step i's copy
        out, lse = mla.prefill_forward(x["q_nope"], ...)
        ...
        pipe.release()                     # step i's buffers may be overwritten after this point

Only CUDA events order the two streams; nothing here synchronises the host.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch


class HostPipeline:
    def __init__(self, example: Dict[str, torch.Tensor], device: torch.device, depth: int = 2):
        if depth < 2:
            raise ValueError("a pipeline needs at least two buffer sets")
        self.device = device
        self.copy_stream = torch.cuda.Stream(device)
        self.buffers: List[Dict[str, torch.Tensor]] = [
            {k: torch.empty(v.shape, dtype=v.dtype, device=device) for k, v in example.items()} for _ in range(depth)
        ]
        self.ready: List[Optional[torch.cuda.Event]] = [None] * depth      # copy finished
        self.free: List[Optional[torch.cuda.Event]] = [None] * depth       # compute that read the set was enqueued and finished
        self.staged = 0
        self.acquired = 0
        self.released = 0
        # copies must not start before work already enqueued on the caller's stream (e.g. a timing event)
        self.copy_stream.wait_stream(torch.cuda.current_stream(device))

    @property
    def bytes_per_step(self) -> int:
        return sum(v.numel() * v.element_size() for v in self.buffers[0].values())

    def stage(self, host: Dict[str, torch.Tensor]) -> None:
        """Enqueues the copy of one step's inputs (pinned host tensors) on the copy stream."""
        if self.staged - self.released >= len(self.buffers):
            raise RuntimeError("every buffer set is in use: release() a step before staging another")
        slot = self.staged % len(self.buffers)
        if self.free[slot] is not None:
            self.copy_stream.wait_event(self.free[slot])
        with torch.cuda.stream(self.copy_stream):
            for key, target in self.buffers[slot].items():
                source = host[key]
                if not source.is_pinned():
                    raise ValueError(f"host tensor '{key}' is not in pinned memory")
                target.copy_(source, non_blocking=True)
            event = torch.cuda.Event()
            event.record(self.copy_stream)
        self.ready[slot] = event
        self.staged += 1

    def acquire(self) -> Dict[str, torch.Tensor]:
        """Makes the current stream wait for the oldest staged step and returns its device tensors."""
        if self.acquired >= self.staged:
            raise RuntimeError("acquire() without a staged step")
        if self.acquired != self.released:
            raise RuntimeError("release() the previous step first")
        slot = self.acquired % len(self.buffers)
        torch.cuda.current_stream(self.device).wait_event(self.ready[slot])
        self.acquired += 1
        return self.buffers[slot]

    def release(self) -> None:
        """Marks the acquired step's buffers reusable once the work enqueued so far has run."""
        if self.released >= self.acquired:
            raise RuntimeError("release() without acquire()")
        slot = self.released % len(self.buffers)
        event = torch.cuda.Event()
        event.record(torch.cuda.current_stream(self.device))
        self.free[slot] = event
        self.released += 1
