"""Expert-parallel top-1 MoE layer: one process per GPU, experts sharded, tokens data-parallel.

The reference places whole layers on GPUs and hops activations between them (sub1.py:296-297,
307-309,320,322-331); it has no collective.  Here rank ``r`` of ``G`` holds experts
``[r * E/G, (r+1) * E/G)`` of the layer and ``T/G`` of the tokens, and one step is

  route -> dispatch all-to-all -> local grouped expert FFN -> combine all-to-all -> scale.

Both exchanges use fixed-size slots: every (source, destination) pair owns ``pair_capacity`` rows.
That keeps all sizes known on the host: no count exchange, no device-to-host synchronisation, and
the step can be replayed from a CUDA graph.  Each row carries its local expert id in a 16-byte
trailer, so one collective moves payload and metadata together.  Received rows land in this GPU's
own memory before any kernel reads them, and they are not copied again: the grouped FFN reads them
through a row list and writes its results back to the same rows of the return buffer.

``pair_capacity`` defaults to twice the mean number of rows a pair exchanges under uniform routing
plus 16 (about nine standard deviations at 8 ranks), capped by the local token count, which is the
worst case.  A token that does not fit is not exchanged: it passes through the layer scaled by its
router probability, exactly like a token dropped by the router's own capacity rule, and is counted
in ``overflow_count()``.  ``pair_capacity=n_local`` (or ``exact=True``, which re-runs an overflowing
step at the worst case after a host check) never drops one.

Two ways to move the rows (``exchange``): ``"nccl"``, two ``all_to_all_single`` calls, and
``"peer"``, where the packing kernel stores every row straight into its destination's receive
buffer and the grouped FFN stores every result row straight into the source's return buffer, both
in peer-mapped memory over NVLink (:mod:`qmoe_b200.peer`), with one small barrier kernel after each
side.  ``"auto"`` (the default; environment variable ``QMOE_EP_EXCHANGE`` overrides it) takes
``"peer"`` on GPUs when every rank has its own GPU and symmetric memory can be set up, else NCCL.
Both give the same bits.

The device work goes through an ``ops`` namespace, by default the CUDA entry points of
:mod:`qmoe_b200.sub1`; the CPU test-suite substitutes a torch re-statement to check the index
arithmetic and the exchanges among gloo ranks.
"""
from __future__ import annotations

import os
import warnings
from typing import Optional

import torch
import torch.distributed as dist

TRAILER = 8  # bf16 elements appended to every exchanged row (16 bytes; the first 4 hold the expert id)


def _default_ops():
    from . import sub1
    return sub1


def default_pair_capacity(n_local: int, world: int) -> int:
    """Rows every (source, destination) pair can exchange per step."""
    if world <= 1:
        return n_local
    mean = (n_local + world - 1) // world
    return min(n_local, (2 * mean + 16 + 7) // 8 * 8)


class ExpertParallelMLP:
    """``store`` holds this rank's experts; ``n_experts`` is the global count."""

    def __init__(self, router_weight: Optional[torch.Tensor], store, n_experts: int,
                 group: Optional[dist.ProcessGroup] = None, expert_capacity: int = 1024,
                 pair_capacity: Optional[int] = None, ops=None, exact: bool = False, exchange: str = "auto"):
        self.ops = ops if ops is not None else _default_ops()
        self.store = store
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        if n_experts % self.world != 0:
            raise ValueError("the number of experts must be a multiple of the number of ranks")
        self.n_experts = int(n_experts)
        self.local_experts = self.n_experts // self.world
        if store.n_experts != self.local_experts:
            raise ValueError(f"store holds {store.n_experts} experts, expected {self.local_experts}")
        self.expert_capacity = int(expert_capacity)
        self.pair_capacity = pair_capacity
        self.exact = bool(exact)
        self.overflow = torch.zeros(1, dtype=torch.int32, device=store.device)
        exchange = os.environ.get("QMOE_EP_EXCHANGE", exchange)
        if exchange not in ("auto", "peer", "nccl"):
            raise ValueError("exchange must be 'auto', 'peer' or 'nccl'")
        if self.world <= 1 or (exchange == "auto" and (ops is not None or store.device.type != "cuda")):
            exchange = "nccl"
        self.exchange = exchange
        self._peer = {}  # (pair capacity, d_model) -> PeerBuffers
        self.router = None
        if router_weight is not None:
            from .sub1 import RouterClassifier
            self.router = RouterClassifier(router_weight, store.device)

    def router_logits(self, hidden2d: torch.Tensor) -> torch.Tensor:
        return self.router(hidden2d)

    def overflow_count(self, reset: bool = False) -> int:
        """Tokens that did not fit their pair's exchange capacity since the last reset (a device-to-host
        read: call it where the caller synchronises anyway)."""
        n = int(self.overflow.item())
        if reset:
            self.overflow.zero_()
        return n

    def _peer_buffers(self, cap: int, d: int):
        """Peer-mapped exchange buffers for this capacity (a collective call on first use), or None
        after falling back to NCCL."""
        key = (cap, d)
        if key not in self._peer:
            from .peer import PeerBuffers
            try:
                self._peer[key] = PeerBuffers.create(self.group, self.store.device, cap, d)
            except Exception as exc:  # no symmetric memory in this build, ranks sharing a GPU, ...
                # (PeerBuffers makes every rank fail together, so all ranks take this branch)
                if self.exchange == "peer":
                    raise
                warnings.warn(f"expert-parallel exchange falls back to NCCL: {exc}")
                self.exchange = "nccl"
                return None
            self.exchange = "peer"
        return self._peer[key]

    def peer_timeouts(self) -> int:
        """Barrier waits of the peer exchange that ran out of time (device-to-host reads)."""
        return sum(p.timeouts() for p in self._peer.values())

    def forward(self, hidden: torch.Tensor, router_logits: Optional[torch.Tensor] = None, seq_len: int = 0,
                pair_capacity: Optional[int] = None):
        """``hidden`` bf16 [n_local, d_model] (every rank passes the same n_local)."""
        ops, G, d = self.ops, self.world, hidden.shape[1]
        n = hidden.shape[0]
        cap = int(pair_capacity or self.pair_capacity or default_pair_capacity(n, G))
        seq_len = seq_len or n
        if router_logits is None:
            router_logits = self.router_logits(hidden)
        choice, prob = ops.route_top1(router_logits.reshape(n, self.n_experts).float().contiguous())
        if self.exact and cap < n:
            before = self.overflow_count()
        peer = self._peer_buffers(cap, d) if self.exchange != "nccl" else None
        # capacity rule on the global expert id, destination rank, rows packed into exchange slots
        if peer is not None:
            expert, slot = ops.ep_dispatch_peer(choice, hidden, self.n_experts, G, seq_len, self.expert_capacity,
                                                cap, self.overflow, peer.dest_blocks)
        else:
            expert, slot, send = ops.ep_dispatch(choice, hidden, self.n_experts, G, seq_len, self.expert_capacity,
                                                 cap, self.overflow)
        if self.exact and cap < n:
            # every rank must take the same branch: the largest overflow decides
            over = torch.tensor([self.overflow_count() - before], dtype=torch.int32, device=hidden.device)
            if G > 1:
                dist.all_reduce(over, op=dist.ReduceOp.MAX, group=self.group)
            if int(over.item()) > 0:
                self.overflow.fill_(before)
                return self.forward(hidden, router_logits, seq_len, pair_capacity=n)

        if peer is not None:
            # the rows are in the peers' memory already: wait until everybody's are in ours, group them by
            # local expert and let the FFN store every result where its source rank will read it
            peer.barrier(0)
            offsets_r, _, row_of_slot, out_ptrs = ops.plan_rows_peer(self.local_experts, peer.recv, d,
                                                                     peer.out_blocks, cap, 2 * d)
            ops.grouped_ffn_scatter(self.store, offsets_r, peer.recv, row_of_slot, out_ptrs, G * cap)
            peer.barrier(1)
            out = ops.combine(peer.ret, hidden, slot, prob)
            return out, (router_logits, torch.clamp(expert, min=0).to(torch.int64))
        if G > 1:
            recv = torch.empty_like(send)
            dist.all_to_all_single(recv, send, group=self.group)
        else:
            recv = send
        # received rows grouped by local expert, in place: row lists instead of sorted copies
        offsets_r, _, row_of_slot = ops.plan_rows(self.local_experts, rows=recv, d_model=d)
        ret = torch.empty((G * cap, d), dtype=torch.bfloat16, device=hidden.device)
        ops.grouped_ffn_rows(self.store, offsets_r, recv, row_of_slot, ret, row_of_slot, G * cap)
        if G > 1:
            back = torch.empty_like(ret)
            dist.all_to_all_single(back, ret, group=self.group)
        else:
            back = ret
        out = ops.combine(back, hidden, slot, prob)
        return out, (router_logits, torch.clamp(expert, min=0).to(torch.int64))

    __call__ = forward
