"""A Switch-shaped decoder stack around the compressed MoE layer, for end-to-end generation timing.

The reference times generation through HuggingFace's Switch Transformers (sub1.py:365-385) with
published compressed checkpoints; neither is available offline, so this module is a self-contained
stand-in with the same structure where it matters for the hot path: every block is
RMS-norm -> multi-head self-attention with a KV cache -> RMS-norm -> top-1 MoE FFN over compressed
experts, with residual connections, seeded random dense weights (bf16, N(0, 0.02)) and seeded
ternary experts.  Dense parts use torch (cuBLAS / SDPA); the MoE FFN is this package's grouped path.

Expert parallelism for generation: the token stream is replicated (batch 1), every rank holds
``n_experts / world`` experts of every layer, computes the FFN of the tokens routed to its own
experts, and an all-reduce sums the disjoint contributions -- for one token per step that is one
small all-reduce per layer instead of two all-to-alls.
"""
from __future__ import annotations

import math
from typing import List, Optional

import torch
import torch.distributed as dist
import torch.nn.functional as F

from . import sub1, synth


class ReplicatedTokenMoE:
    """Top-1 MoE over the local experts of every rank, for tokens that all ranks hold.

    Same arithmetic as :class:`qmoe_b200.sub1.FasterMLP` (sub1.py:306-321); a token whose expert
    lives on another rank contributes zeros here and receives its result through the all-reduce."""

    def __init__(self, router_weight: torch.Tensor, store, n_experts: int, rank: int = 0, world: int = 1,
                 group=None, expert_capacity: int = 1024):
        self.store, self.n_experts, self.rank, self.world, self.group = store, n_experts, rank, world, group
        self.local = n_experts // world
        self.capacity = expert_capacity
        self.router = sub1.RouterClassifier(router_weight, store.device)
        self.trace: Optional[torch.Tensor] = None   # int32[n_experts]: tokens routed to every expert in decode steps
        self.force: Optional[torch.Tensor] = None   # int64[1] on the device: expert that decode steps are sent to

    def decode_step(self, x: torch.Tensor, ln_weight: torch.Tensor) -> torch.Tensor:
        """``x + moe(rms_norm(x))`` for one token; the norm rides on the router's matrix-vector
        product when the router weights are exact in bf16."""
        if self.router.w16 is not None and x.shape[0] == 1:
            logits, hidden = sub1.gemv(x, self.router.w16, ln_weight=ln_weight, f32_out=True, want_normed=True)
            return self(hidden, residual=x, logits=logits)
        return self(sub1.rms_norm(x, ln_weight), residual=x)

    def __call__(self, hidden: torch.Tensor, residual: Optional[torch.Tensor] = None,
                 logits: Optional[torch.Tensor] = None) -> torch.Tensor:
        """MoE output for ``hidden``; with ``residual`` (single-rank only) ``residual + output``."""
        n, d = hidden.shape
        if logits is None:
            logits = self.router(hidden).contiguous()
        if self.force is not None and n == 1:
            # measurement aid: the step's expert is given (a large logit), whatever the router computed
            logits = logits.index_fill(1, self.force, 1e4)
        if n <= 32:
            # a decode step: routing, ranking and permutation in one launch (every rank does the same
            # routing on the same replicated token)
            prob, offsets, slot, xs = sub1.route_small(logits, hidden, self.n_experts, self.capacity)
            if self.trace is not None and n == 1:                # decode steps only, not a short prefill
                self.trace += offsets[1:] - offsets[:-1]
            if self.world == 1:
                ys = sub1.grouped_ffn(self.store, offsets, xs, n)
            else:
                # This rank's experts are a window of the offsets; rows of other ranks' experts stay zero
                # and arrive through the all-reduce (one rank holds the row, the sum is exact).
                lo = self.rank * self.local
                ys = torch.zeros_like(xs)
                sub1.grouped_ffn_rows(self.store, offsets[lo:lo + self.local + 1], xs, None, ys, None, n)
                dist.all_reduce(ys, group=self.group)
            if residual is not None:
                return sub1.combine_add(ys, hidden, slot, prob, residual)
            return sub1.combine(ys, hidden, slot, prob)
        choice, prob = sub1.route_top1(logits)
        if self.world == 1:
            # all experts are local: the single-GPU layer (route, rank, permute, FFN, combine)
            bucket, rank, _, offsets = sub1.rank_buckets(choice, self.n_experts, n, self.capacity)
            xs = torch.empty_like(hidden)
            slot = sub1.permute_rows(bucket, rank, offsets, hidden, xs)
            ys = sub1.grouped_ffn(self.store, offsets, xs, n)
            if residual is not None:
                return sub1.combine_add(ys, hidden, slot, prob, residual)
            return sub1.combine(ys, hidden, slot, prob)
        expert, _, _, _ = sub1.rank_buckets(choice, self.n_experts, n, self.capacity)
        lo = self.rank * self.local
        mine = (expert >= lo) & (expert < lo + self.local)
        local_choice = torch.where(mine, expert - lo, torch.full_like(expert, -1))
        bucket, rank, _, offsets = sub1.rank_buckets(local_choice, self.local, n, n)
        xs = torch.empty_like(hidden)
        slot = sub1.permute_rows(bucket, rank, offsets, hidden, xs)
        ys = sub1.grouped_ffn(self.store, offsets, xs, n)
        part = torch.empty_like(hidden)
        sub1.unpermute_rows(ys, slot, part)                      # zeros for tokens of other ranks
        dist.all_reduce(part, group=self.group)
        # tokens dropped by the capacity rule pass through (sub1.py:312,318)
        ident = torch.arange(n, dtype=torch.int32, device=hidden.device)
        out = sub1.combine(part, hidden, torch.where(expert >= 0, ident, torch.full_like(ident, -1)), prob)
        return out if residual is None else residual + out


def _rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    v = x.float()
    return (v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + eps)).to(x.dtype) * w


class SwitchDecoderLM:
    """``n_layers`` blocks of (self-attention, MoE FFN); greedy generation with a static KV cache."""

    def __init__(self, d_model: int, d_ff: int, n_experts: int, n_layers: int, n_heads: int, vocab: int,
                 max_len: int, device, seed: int = 0, rank: int = 0, world: int = 1, group=None,
                 drop_reference_layout: bool = True):
        self.d, self.h, self.hd, self.L, self.vocab, self.max_len = d_model, n_heads, d_model // n_heads, n_layers, vocab, max_len
        self.dev = torch.device(device)
        g = torch.Generator().manual_seed(seed * 9973 + 1)

        def dense(*shape):
            return (torch.randn(*shape, generator=g) * 0.02).bfloat16().to(self.dev)

        d_attn = self.h * self.hd
        self.embed = dense(vocab, d_model)
        self.lm_head = dense(vocab, d_model)
        self.final_norm = torch.ones(d_model, dtype=torch.bfloat16, device=self.dev)
        self.blocks: List[dict] = []
        local = n_experts // world
        for layer in range(n_layers):
            ids = [layer * n_experts + e for e in range(rank * local, (rank + 1) * local)]   # distinct seeds per layer
            store = synth.build_store(d_model, d_ff, ids, seed, self.dev)
            if drop_reference_layout and store.il_codes is not None:
                store.drop_reference_layout()       # 15 layers of both layouts would not fit one GPU
            router = (torch.randn(n_experts, d_model, generator=g) / math.sqrt(d_model)).bfloat16().float()
            self.blocks.append({
                "ln1": torch.ones(d_model, dtype=torch.bfloat16, device=self.dev),
                "ln2": torch.ones(d_model, dtype=torch.bfloat16, device=self.dev),
                "wqkv": dense(3 * d_attn, d_model), "wo": dense(d_model, d_attn),
                "moe": ReplicatedTokenMoE(router, store, n_experts, rank, world, group),
            })
        if drop_reference_layout:
            torch.cuda.empty_cache()                # hand the freed streams back before graphs are captured
        self._graph = None
        self._step_ids = self._step_pos = None
        self.fused_decode = True                    # single-token steps take _forward_one
        self.k_cache = torch.zeros(n_layers, self.h, max_len, self.hd, dtype=torch.bfloat16, device=self.dev)
        self.v_cache = torch.zeros_like(self.k_cache)

    @property
    def compressed_bytes(self) -> int:
        return sum(b["moe"].store.compressed_bytes for b in self.blocks)

    def forward(self, ids: torch.Tensor, pos: torch.Tensor) -> torch.Tensor:
        """``ids`` int64[n] at cache positions ``pos`` int64[n] (contiguous, ascending); returns the
        logits fp32[n, vocab].  Attention sees cache positions <= the query's own position; the mask
        is built from ``pos`` on the device, so the same code serves prefill, eager decoding and
        CUDA-graph replay of a decode step."""
        n = ids.shape[0]
        if n == 1 and self.fused_decode:
            return self._forward_one(ids, pos)
        x = self.embed[ids]
        all_pos = torch.arange(self.max_len, device=self.dev)
        mask = all_pos[None, :] <= pos[:, None]                                    # [n, max_len]
        for i, b in enumerate(self.blocks):
            hn = _rms_norm(x, b["ln1"])
            qkv = (hn @ b["wqkv"].t()).view(n, 3, self.h, self.hd)
            self.k_cache[i].index_copy_(1, pos, qkv[:, 1].transpose(0, 1))
            self.v_cache[i].index_copy_(1, pos, qkv[:, 2].transpose(0, 1))
            q = qkv[:, 0].transpose(0, 1)                                            # [h, n, hd]
            att = F.scaled_dot_product_attention(q.unsqueeze(0), self.k_cache[i].unsqueeze(0),
                                                 self.v_cache[i].unsqueeze(0), attn_mask=mask[None, None])
            x = x + att[0].transpose(0, 1).reshape(n, -1) @ b["wo"].t()
            x = x + b["moe"](_rms_norm(x, b["ln2"]).contiguous())
        return (_rms_norm(x, self.final_norm) @ self.lm_head.t()).float()

    def _forward_one(self, ids: torch.Tensor, pos: torch.Tensor) -> torch.Tensor:
        """The same block arithmetic for a single token with one launch per group of operations:
        matrix-vector products with the RMS norm fused in front or the residual behind, one
        attention kernel that also stores the token's key and value, one routing kernel, and the
        MoE combine with the residual addition folded in."""
        x = self.embed[ids]
        for i, b in enumerate(self.blocks):
            qkv = sub1.gemv(x, b["wqkv"], ln_weight=b["ln1"])
            att = sub1.decode_attention(qkv, self.k_cache[i], self.v_cache[i], pos)
            x = sub1.gemv(att, b["wo"], residual=x)
            x = b["moe"].decode_step(x, b["ln2"])
        return sub1.gemv(x, self.lm_head, ln_weight=self.final_norm, f32_out=True)

    @torch.no_grad()
    def trace_experts(self, on: bool) -> None:
        """Start (zeroed) or stop counting, per block, the tokens every expert receives in decode
        steps.  Adds two small launches per block: for untimed, eager passes."""
        for b in self.blocks:
            moe = b["moe"]
            moe.trace = torch.zeros(moe.n_experts, dtype=torch.int32, device=self.dev) if on else None

    def set_forced_routing(self, schedule: Optional[torch.Tensor]) -> None:
        """``schedule`` int64[steps, n_layers]: decode step ``k`` of :meth:`generate` sends its token
        to expert ``schedule[k, i]`` in block ``i`` (its router probability becomes 1).  Random
        weights route almost every token of a sequence to the same few experts per block, which then
        stay in L2; a trained model does not.  ``None`` gives the routing back to the routers.  A
        captured decode graph is dropped either way."""
        self.close()
        if schedule is None:
            self._route_sched = None
            for b in self.blocks:
                b["moe"].force = None
            return
        assert schedule.dtype == torch.int64 and schedule.shape[1] == len(self.blocks)
        self._route_sched = schedule.to(self.dev).contiguous()
        self._route_now = torch.zeros(len(self.blocks), dtype=torch.int64, device=self.dev)
        for i, b in enumerate(self.blocks):
            b["moe"].force = self._route_now[i:i + 1]

    def expert_trace(self) -> torch.Tensor:
        """int32[n_layers, n_experts] of the counts since ``trace_experts(True)`` (a host copy)."""
        return torch.stack([b["moe"].trace for b in self.blocks]).cpu()

    def generate(self, prompt: torch.Tensor, n_new: int, use_graph: bool = True,
                 forced: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Prefill the prompt, then ``n_new`` single-token steps.  Greedy by default: every step's
        input is the previous step's argmax.  With ``forced`` (int64[n_new - 1]) step ``k`` is fed
        ``forced[k]`` instead (teacher forcing: the returned argmax tokens are still computed), so that
        a model with random weights, whose greedy output soon repeats one token, still visits different
        experts from step to step as a trained model does."""
        import time
        p = prompt.shape[0]
        assert p + n_new <= self.max_len
        torch.cuda.synchronize(self.dev)
        t_start = time.perf_counter()
        logits = self.forward(prompt.to(self.dev), torch.arange(p, device=self.dev))
        tok = logits[-1].argmax().reshape(1)
        torch.cuda.synchronize(self.dev)
        t_prefill = time.perf_counter()
        out = [tok]
        if self._step_pos is None:
            self._step_ids = tok.clone()
            self._step_pos = torch.zeros(1, dtype=torch.int64, device=self.dev)
        step_ids, step_pos = self._step_ids, self._step_pos
        step_ids.copy_(tok)
        step_pos.fill_(p)
        graph = None
        if use_graph and n_new > 4:
            # The decode step reads its position from a device tensor, so one captured graph serves
            # every later call; it is captured on first use and kept until close().
            if self._graph is None:
                from .graph import GraphedStep
                try:
                    self._graph = GraphedStep(lambda t: self.forward(t, step_pos)[-1].argmax().reshape(1), step_ids)
                    step_pos.fill_(p)                 # capture and its warm-up runs did not advance it
                except Exception as exc:  # keep generating eagerly, but say so
                    import warnings
                    warnings.warn(f"CUDA-graph capture of the decode step failed, decoding eagerly: {exc!r}")
            graph = self._graph
        self.last_generate_used_graph = graph is not None
        torch.cuda.synchronize(self.dev)
        t_capture = time.perf_counter()
        if forced is not None:
            forced = forced.to(self.dev).reshape(-1, 1)
            assert forced.shape[0] >= n_new - 1
        sched = getattr(self, "_route_sched", None)
        assert sched is None or sched.shape[0] >= n_new - 1
        for k in range(n_new - 1):
            step_ids.copy_(tok if forced is None else forced[k])
            if sched is not None:
                self._route_now.copy_(sched[k])
            if graph is not None:
                graph.static_in.copy_(step_ids)
                tok = graph.replay().clone()
            else:
                tok = self.forward(step_ids, step_pos)[-1].argmax().reshape(1)
            out.append(tok)
            step_pos += 1
        torch.cuda.synchronize(self.dev)
        t_end = time.perf_counter()
        self.last_timing = {"prefill_s": t_prefill - t_start, "graph_capture_s": t_capture - t_prefill,
                            "decode_s": t_end - t_capture, "decode_steps": n_new - 1}
        return torch.cat(out)

    def close(self) -> None:
        """Destroy the captured decode graph (before tearing down a process group it captured)."""
        if self._graph is not None:
            self._graph.close()
            self._graph = None
