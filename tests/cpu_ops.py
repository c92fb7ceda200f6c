"""Torch-CPU re-statement of the device ops the expert-parallel layer calls (route, rank, permute,
grouped FFN via the oracle, unpermute, combine).  A TEST DOUBLE: it lets world_size-2 gloo ranks
exercise the exchange logic and index arithmetic of qmoe_b200.ep without a GPU."""
import torch

from util import reference_router


class CpuStore:
    def __init__(self, experts):
        self.experts = experts
        self.n_experts = len(experts)
        self.d_model, self.d_ff = experts[0].d_model, experts[0].d_ff
        self.device = torch.device("cpu")


def route_top1(logits):
    mask, probs = reference_router(logits.unsqueeze(0), capacity=10 ** 9)
    return mask[0].argmax(-1).to(torch.int32), probs.reshape(-1)


def rank_buckets(choice, n_buckets, seq_len, capacity):
    n = choice.numel()
    bucket = torch.full((n,), -1, dtype=torch.int32)
    rank = torch.zeros(n, dtype=torch.int32)
    counts = torch.zeros(n_buckets, dtype=torch.int32)
    seen_seq = {}
    for t in range(n):
        c = int(choice[t])
        if c < 0 or c >= n_buckets:
            continue
        key = (t // seq_len, c)
        before = seen_seq.get(key, 0)
        seen_seq[key] = before + 1
        if before < capacity:
            bucket[t] = c
            rank[t] = counts[c]
            counts[c] += 1
    offsets = torch.zeros(n_buckets + 1, dtype=torch.int32)
    offsets[1:] = torch.cumsum(counts, 0)
    return bucket, rank, counts, offsets


def permute_rows(bucket, rank, offsets, hidden, xs):
    slot = torch.where(bucket >= 0, offsets[bucket.clamp(min=0).long()] + rank, torch.full_like(rank, -1))
    for t in range(hidden.shape[0]):
        if slot[t] >= 0:
            xs[int(slot[t])] = hidden[t]
    return slot.to(torch.int32)


def unpermute_rows(ys, slot, out):
    for t in range(out.shape[0]):
        out[t] = ys[int(slot[t])] if slot[t] >= 0 else 0


def ep_dispatch(choice, hidden, n_experts, n_ranks, seq_len, expert_capacity, pair_capacity, overflow):
    n, d = hidden.shape
    local = n_experts // n_ranks
    expert, _, _, _ = rank_buckets(choice, n_experts, seq_len, expert_capacity)
    send = torch.zeros((n_ranks * pair_capacity, d + 8), dtype=torch.bfloat16)
    meta = send.view(torch.int32)[:, d // 2]
    meta.fill_(-1)
    slot = torch.full((n,), -1, dtype=torch.int32)
    used = [0] * n_ranks
    for t in range(n):
        e = int(expert[t])
        if e < 0:
            continue
        dst = e // local
        if used[dst] >= pair_capacity:
            overflow += 1
            continue
        s = dst * pair_capacity + used[dst]
        used[dst] += 1
        slot[t] = s
        send[s, :d] = hidden[t]
        meta[s] = e - dst * local
    return expert, slot, send


def plan_rows(n_buckets, bucket=None, rows=None, d_model=0):
    if rows is not None:
        bucket = rows.view(torch.int32)[:, d_model // 2].clone()
    m = bucket.numel()
    b = torch.where((bucket >= 0) & (bucket < n_buckets), bucket, torch.full_like(bucket, -1))
    counts = torch.zeros(n_buckets, dtype=torch.int32)
    offsets = torch.zeros(n_buckets + 1, dtype=torch.int32)
    for i in range(m):
        if b[i] >= 0:
            counts[int(b[i])] += 1
    offsets[1:] = torch.cumsum(counts, 0)
    slot_of_row = torch.full((m,), -1, dtype=torch.int32)
    row_of_slot = torch.zeros(m, dtype=torch.int32)
    seen = [0] * n_buckets
    for i in range(m):
        if b[i] >= 0:
            s = int(offsets[int(b[i])]) + seen[int(b[i])]
            seen[int(b[i])] += 1
            slot_of_row[i] = s
            row_of_slot[s] = i
    return offsets, slot_of_row, row_of_slot


def grouped_ffn_rows(store, offsets, xs, x_rows, ys, y_rows, max_slots):
    d = store.d_model
    for e in range(store.n_experts):
        a, b = int(offsets[e]), int(offsets[e + 1])
        if b > a:
            src = [int(x_rows[s]) if x_rows is not None else s for s in range(a, b)]
            dst = [int(y_rows[s]) if y_rows is not None else s for s in range(a, b)]
            y = store.experts[e].oracle_ffn(xs[src, :d].contiguous())
            for k, r in enumerate(dst):
                ys[r] = y[k]
    return ys


def grouped_ffn(store, offsets, xs, max_slots):
    ys = torch.zeros((max_slots, store.d_model), dtype=torch.bfloat16)
    for e in range(store.n_experts):
        a, b = int(offsets[e]), int(offsets[e + 1])
        if b > a:
            ys[a:b] = store.experts[e].oracle_ffn(xs[a:b].contiguous())
    return ys


def combine(ys, hidden, slot, prob):
    out = torch.empty_like(hidden)
    for t in range(hidden.shape[0]):
        src = ys[int(slot[t])] if slot[t] >= 0 else hidden[t]
        out[t] = (prob[t].float() * src.float()).bfloat16()
    return out
