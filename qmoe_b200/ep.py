"""Expert-parallel top-1 MoE layer: one process per GPU, experts sharded, tokens data-parallel.

The reference places whole layers on GPUs and hops activations between them (sub1.py:296-297,
307-309,320,322-331); it has no collective.  Here rank ``r`` of ``G`` holds experts
``[r * E/G, (r+1) * E/G)`` of the layer and ``T/G`` of the tokens, and one step is

  route -> dispatch all-to-all -> local grouped expert FFN -> combine all-to-all -> scale.

Both exchanges use fixed-size slots: every (source, destination) pair owns ``pair_capacity`` rows
(by default the local token count, the worst case, so no token is ever dropped by the exchange).
That keeps all sizes known on the host: no count exchange, no device-to-host synchronisation, and
the step can be replayed from a CUDA graph.  Each row carries its local expert id in a 16-byte
trailer, so one collective moves payload and metadata together.  Received rows land in this GPU's
own memory before any kernel reads them.

The device work (ranking, permutation, grouped FFN, combine) goes through an ``ops`` namespace, by
default the CUDA entry points of :mod:`qmoe_b200.sub1`; the CPU test-suite substitutes a torch
re-statement to check the index arithmetic and the exchanges among gloo ranks.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist

TRAILER = 8  # bf16 elements appended to every exchanged row (16 bytes; the first 4 hold the expert id)


def _default_ops():
    from . import sub1
    return sub1


class ExpertParallelMLP:
    """``store`` holds this rank's experts; ``n_experts`` is the global count."""

    def __init__(self, router_weight: Optional[torch.Tensor], store, n_experts: int,
                 group: Optional[dist.ProcessGroup] = None, expert_capacity: int = 1024,
                 pair_capacity: Optional[int] = None, ops=None):
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
        self.router = None
        if router_weight is not None:
            from .sub1 import RouterClassifier
            self.router = RouterClassifier(router_weight, store.device)

    def router_logits(self, hidden2d: torch.Tensor) -> torch.Tensor:
        return self.router(hidden2d)

    def forward(self, hidden: torch.Tensor, router_logits: Optional[torch.Tensor] = None, seq_len: int = 0):
        """``hidden`` bf16 [n_local, d_model] (every rank passes the same n_local)."""
        ops, G, d = self.ops, self.world, hidden.shape[1]
        n = hidden.shape[0]
        dev = hidden.device
        cap = int(self.pair_capacity or n)
        seq_len = seq_len or n
        if router_logits is None:
            router_logits = self.router_logits(hidden)
        choice, prob = ops.route_top1(router_logits.reshape(n, self.n_experts).float().contiguous())
        # capacity rule on the global expert id, then bucket by destination rank
        expert, _, _, _ = ops.rank_buckets(choice, self.n_experts, seq_len, self.expert_capacity)
        dest = torch.where(expert >= 0, torch.div(expert, self.local_experts, rounding_mode="floor"),
                           expert).to(torch.int32)
        bucket, rank, _, _ = ops.rank_buckets(dest, G, n, cap)

        # send buffer: G * cap rows (+1 scratch row that absorbs the metadata of dropped tokens)
        row = d + TRAILER
        send = torch.empty((G * cap + 1, row), dtype=torch.bfloat16, device=dev)
        meta = send.view(torch.int32)[:, d // 2]
        meta.fill_(-1)
        fixed = torch.arange(G + 1, dtype=torch.int32, device=dev) * cap
        slot = ops.permute_rows(bucket, rank, fixed, hidden, send[:, :d])
        local_id = (expert - dest * self.local_experts).to(torch.int32)
        meta.index_copy_(0, torch.where(slot >= 0, slot, G * cap).to(torch.int64), local_id)

        recv = torch.empty((G * cap, row), dtype=torch.bfloat16, device=dev)
        if G > 1:
            dist.all_to_all_single(recv, send[:G * cap], group=self.group)
        else:
            recv.copy_(send[:G * cap])

        meta_r = recv.view(torch.int32)[:, d // 2].contiguous()
        bucket_r, rank_r, _, offsets_r = ops.rank_buckets(meta_r, self.local_experts, G * cap, G * cap)
        xs = torch.empty((G * cap, d), dtype=torch.bfloat16, device=dev)
        slot_r = ops.permute_rows(bucket_r, rank_r, offsets_r, recv[:, :d], xs)
        ys = ops.grouped_ffn(self.store, offsets_r, xs, G * cap)
        ret = torch.empty((G * cap, d), dtype=torch.bfloat16, device=dev)
        ops.unpermute_rows(ys, slot_r, ret)

        back = torch.empty_like(ret)
        if G > 1:
            dist.all_to_all_single(back, ret, group=self.group)
        else:
            back = ret
        out = ops.combine(back, hidden, slot, prob)
        return out, (router_logits, torch.clamp(expert, min=0).to(torch.int64))

    __call__ = forward
