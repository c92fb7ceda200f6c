"""Exchange buffers of the expert-parallel layer in peer-mapped GPU memory.

Every rank allocates one block of symmetric memory (``torch.distributed._symmetric_memory``: the
same allocation on every rank, mapped into every peer's address space over NVLink) that holds

  flags   int32[2, G]            one word per (barrier of the step, peer)
  recv    bf16[G * cap, d + 8]   rows this rank's experts receive, block r written by rank r
  ret     bf16[G * cap, d]       results coming back to this rank, block r written by rank r

and three small device tables of addresses valid on this GPU: where this rank's block starts in
every peer's ``recv`` and ``ret`` and where every rank's flags are.  The kernels of
``csrc/moe_ep.cu`` store rows straight into the peers' buffers; no collective library is in the data
path.  The reference moves whole activations between GPUs instead (sub1.py:307-309,320).

Ranks that share a GPU cannot use this (their kernels would wait for each other's launches), and a
build of torch without symmetric memory cannot either: :func:`PeerBuffers.create` raises and the
caller stays on NCCL.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from . import _lib

_ALIGN = 1024


def _round_up(n: int, a: int = _ALIGN) -> int:
    return (n + a - 1) // a * a


class PeerBuffers:
    def __init__(self, group, device: torch.device, pair_capacity: int, d_model: int):
        import torch.distributed._symmetric_memory as symm

        self.group = group if group is not None else dist.group.WORLD
        G = dist.get_world_size(self.group)
        rank = dist.get_rank(self.group)
        self.world, self.rank, self.cap, self.d_model, self.device = G, rank, int(pair_capacity), int(d_model), device
        # one GPU per rank, or the barrier kernels of two ranks could wait for each other on one GPU
        mine = str(torch.cuda.get_device_properties(device).uuid)
        seen = [None] * G
        dist.all_gather_object(seen, mine, group=self.group)
        if len(set(seen)) != G:
            raise RuntimeError("peer exchange needs one GPU per rank")
        rows = G * self.cap
        off_recv = _round_up(2 * G * 4)
        off_ret = off_recv + _round_up(rows * (d_model + 8) * 2)
        total = off_ret + _round_up(rows * d_model * 2)

        def agreed(step, fn):
            """Run a step that can fail on one rank alone; every rank learns whether all succeeded
            before anyone enters the next collective call."""
            err, out = None, None
            try:
                out = fn()
            except Exception as exc:  # noqa: BLE001
                err = exc
            ok = torch.tensor([0 if err is not None else 1], dtype=torch.int32, device=device)
            dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=self.group)
            if int(ok.item()) == 0:
                raise RuntimeError(f"peer exchange set-up failed at '{step}' on some rank"
                                   + (f": {err}" if err is not None else ""))
            return out

        self.buffer = agreed("allocate", lambda: symm.empty(total, dtype=torch.uint8, device=device))
        self.handle = agreed("rendezvous", lambda: symm.rendezvous(self.buffer, self.group.group_name))

        def addresses():
            got = [int(p) for p in self.handle.buffer_ptrs]
            if len(got) != G or any(p == 0 for p in got):
                raise RuntimeError("symmetric memory gave no peer addresses")
            return got

        ptrs = agreed("peer addresses", addresses)
        self.buffer.zero_()
        self.flags = self.buffer[: 2 * G * 4].view(torch.int32)
        self.recv = self.buffer[off_recv: off_recv + rows * (d_model + 8) * 2].view(torch.bfloat16).view(rows, d_model + 8)
        self.ret = self.buffer[off_ret: off_ret + rows * d_model * 2].view(torch.bfloat16).view(rows, d_model)
        table = lambda vals: torch.tensor(vals, dtype=torch.int64).to(device)  # noqa: E731
        self.dest_blocks = table([p + off_recv + rank * self.cap * (d_model + 8) * 2 for p in ptrs])
        self.out_blocks = table([p + off_ret + rank * self.cap * d_model * 2 for p in ptrs])
        self.flag_blocks = table(ptrs)
        self.status = torch.zeros(1, dtype=torch.int32, device=device)
        self.limit_ms = 20000
        torch.cuda.synchronize(device)
        dist.barrier(group=self.group)  # nobody raises a flag before every block is zeroed

    @classmethod
    def create(cls, group, device, pair_capacity, d_model) -> "PeerBuffers":
        return cls(group, device, pair_capacity, d_model)

    def barrier(self, channel: int) -> None:
        """Launch the barrier kernel of ``channel`` (0 or 1) on the current stream."""
        dev = self.device
        _lib.check(_lib.load().qmoe_moe_peer_barrier(
            self.flag_blocks.data_ptr(), self.rank, self.world, int(channel), int(self.limit_ms),
            self.status.data_ptr(), dev.index, torch.cuda.current_stream(dev).cuda_stream))

    def timeouts(self) -> int:
        """Barrier waits that ran out of time (a device-to-host read)."""
        return int(self.status.item())
