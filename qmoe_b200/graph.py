"""CUDA-graph replay of one layer step.

A MoE layer step here is a fixed sequence of ~20 small launches around two large ones (plus two
NCCL all-to-alls in the expert-parallel layer) with no host synchronisation and no data-dependent
shapes, so it can be captured once and replayed: the launch overhead that dominates at 8 GPUs
(≈ 0.3 ms of a 1 ms step) disappears.  The reference has nothing comparable: its layer loop needs the
host after every expert (sub1.py:315-317).
"""
from __future__ import annotations

from typing import Callable

import torch


class GraphedStep:
    """Capture ``fn(static_input) -> tensor`` once; ``__call__(x)`` copies ``x`` into the static
    input, replays the graph and returns the static output (overwritten by the next call)."""

    def __init__(self, fn: Callable[[torch.Tensor], torch.Tensor], example: torch.Tensor, warmup: int = 3):
        self.static_in = example.clone()
        side = torch.cuda.Stream(device=example.device)
        side.wait_stream(torch.cuda.current_stream(example.device))
        with torch.cuda.stream(side):
            for _ in range(max(warmup, 1)):   # first calls build per-device tables and size the pools
                fn(self.static_in)
        torch.cuda.current_stream(example.device).wait_stream(side)
        torch.cuda.synchronize(example.device)
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            self.static_out = fn(self.static_in)

    def close(self) -> None:
        """Destroy the captured graph.  Call this before ``destroy_process_group()``: NCCL keeps a
        communicator alive while a graph that captured one of its collectives exists, and tearing
        the process group down first blocks forever."""
        if self.graph is not None:
            self.graph.reset()
            self.graph = None
            self.static_out = None

    def replay(self) -> torch.Tensor:
        self.graph.replay()
        return self.static_out

    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        self.static_in.copy_(x, non_blocking=True)
        self.graph.replay()
        return self.static_out


class PipelinedStep:
    """Host-to-host pipeline around a :class:`GraphedStep`: the host-to-device copy of the next
    input and the device-to-host copy of the previous result run on their own streams while the
    graph of the current step executes, with two device buffers on either side.

    ``submit(host_in, host_out)`` enqueues one step and returns at once; ``host_out`` (pinned) is
    complete after ``drain()`` followed by a synchronisation of the current stream, or after the
    event ``submit`` returns.  Results are those of ``gstep(host_in)`` in submission order."""

    def __init__(self, gstep: GraphedStep):
        self.g = gstep
        dev = gstep.static_in.device
        self.dev = dev
        self.s_in = torch.cuda.Stream(device=dev)
        self.s_out = torch.cuda.Stream(device=dev)
        self.bufs_in = [torch.empty_like(gstep.static_in) for _ in range(2)]
        self.bufs_out = [torch.empty_like(gstep.static_out) for _ in range(2)]
        self.ev_in_ready = [torch.cuda.Event() for _ in range(2)]
        self.ev_done = [torch.cuda.Event() for _ in range(2)]
        self.ev_out_free = [torch.cuda.Event() for _ in range(2)]
        self.count = 0

    def submit(self, host_in: torch.Tensor, host_out: torch.Tensor) -> torch.cuda.Event:
        b = self.count % 2
        again = self.count >= 2                       # buffer b was used two steps ago
        cur = torch.cuda.current_stream(self.dev)
        with torch.cuda.stream(self.s_in):
            if again:
                self.s_in.wait_event(self.ev_done[b])     # that step's compute has read bufs_in[b]
            self.bufs_in[b].copy_(host_in, non_blocking=True)
            self.ev_in_ready[b].record(self.s_in)
        cur.wait_event(self.ev_in_ready[b])
        if again:
            cur.wait_event(self.ev_out_free[b])           # its result has left bufs_out[b]
        self.g.static_in.copy_(self.bufs_in[b], non_blocking=True)
        self.g.graph.replay()
        self.bufs_out[b].copy_(self.g.static_out, non_blocking=True)
        self.ev_done[b].record(cur)
        with torch.cuda.stream(self.s_out):
            self.s_out.wait_event(self.ev_done[b])
            host_out.copy_(self.bufs_out[b], non_blocking=True)
            self.ev_out_free[b].record(self.s_out)
        self.count += 1
        return self.ev_out_free[b]

    def drain(self) -> None:
        """Make the current stream wait for every result copy submitted so far."""
        cur = torch.cuda.current_stream(self.dev)
        for b in range(min(self.count, 2)):
            cur.wait_event(self.ev_out_free[b])
