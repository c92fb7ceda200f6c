"""Seeded synthetic stand-ins for the Switch checkpoints (which need a network to fetch).

Shapes and value distributions follow the benchmark configurations: ternary symbols i.i.d. with
P(0) = 0.90 and P(1) = P(2) = 0.05, per-row scale s ~ U(0.01, 0.1) stored as the reference's bf16
(min, max) = (-s, +s) pair (sub1.py:147-149), bf16 activations ~ N(0, 1), router logits ~ N(0, 1).

Symbols come from a counter-based hash so that any rank can regenerate any expert without
communication: symbol ``i`` of matrix ``m`` is ``ternary(seed, (m << 32) + i)``.  The numpy twin
(:func:`ternary_numpy`) produces the same symbols on the CPU; the tests use it to feed the oracle.
"""
from __future__ import annotations

from typing import List, Optional, Tuple

import numpy as np
import torch

from . import _lib, sub1_cuda
from ._lib import MatrixDesc

SHAPES = {
    # name: (d_model, d_ff, n_experts)
    "switch-base-128": (768, 3072, 128),
    "switch-large-128": (1024, 4096, 128),
    "switch-c-2048": (2080, 6144, 2048),
}

_M64 = (1 << 64) - 1


def _splitmix64(x: np.ndarray) -> np.ndarray:
    x = (x + np.uint64(0x9E3779B97F4A7C15)) & np.uint64(_M64)
    x = ((x ^ (x >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)) & np.uint64(_M64)
    x = ((x ^ (x >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)) & np.uint64(_M64)
    return x ^ (x >> np.uint64(31))


def ternary_numpy(count: int, seed: int, first_index: int, p_zero: float) -> np.ndarray:
    """CPU twin of ``qmoe_synth_ternary``: uint8[count]."""
    assert first_index % 4 == 0
    t0 = int(float(np.float32(p_zero)) * 65536.0 + 0.5)
    t1 = t0 + (65536 - min(t0, 65536)) // 2
    idx = np.arange(first_index, first_index + count, dtype=np.uint64)
    with np.errstate(over="ignore"):
        base = np.uint64((seed * 0xD1342543DE82EF95) & _M64)
        h = _splitmix64(base + (idx >> np.uint64(2)))
    u = ((h >> ((idx & np.uint64(3)) * np.uint64(16))) & np.uint64(0xFFFF)).astype(np.int64)
    return np.where(u < t0, 0, np.where(u < t1, 1, 2)).astype(np.uint8)


def ternary_cuda(count: int, seed: int, first_index: int, p_zero: float, device) -> torch.Tensor:
    dev = torch.device(device)
    sym = torch.empty(count, dtype=torch.uint8, device=dev)
    _lib.check(_lib.load().qmoe_synth_ternary(sym.data_ptr(), count, seed & _M64, first_index, float(p_zero),
                                              dev.index, int(torch.cuda.current_stream(dev).cuda_stream)))
    return sym


def matrix_first_index(matrix_id: int) -> int:
    return matrix_id << 32


def row_scales(height: int, seed: int, matrix_id: int) -> torch.Tensor:
    """bf16[2 * height] interleaved (-s, +s), s ~ U(0.01, 0.1), from a CPU generator keyed by
    (seed, matrix) so that every rank and the CPU oracle see the same values."""
    g = torch.Generator().manual_seed((seed * 1000003 + matrix_id) & 0x7FFFFFFFFFFFFFFF)
    s = (torch.rand(height, generator=g) * 0.09 + 0.01).bfloat16()
    return torch.column_stack((-s, s)).flatten()


def build_store(d_model: int, d_ff: int, expert_ids: List[int], seed: int, device, p_zero: float = 0.90,
                batch: int = 32):
    """Generate and pack the wi / wo matrices of the given (global) expert ids on ``device``.
    Matrix ids are ``2 * expert`` (wi) and ``2 * expert + 1`` (wo).  Returns an ExpertStore whose local
    expert ``i`` is ``expert_ids[i]``."""
    from .sub1 import ExpertStore, TRIE
    dev = torch.device(device)
    trie = TRIE(dev)
    n = len(expert_ids)
    results = {}
    for kind, (h, w) in (("wi", (d_ff, d_model)), ("wo", (d_model, d_ff))):
        chunks = []
        for b0 in range(0, n, batch):
            ids = expert_ids[b0:b0 + batch]
            sym = torch.empty((len(ids), h, w), dtype=torch.uint8, device=dev)
            for j, e in enumerate(ids):
                m = 2 * e + (0 if kind == "wi" else 1)
                _lib.check(_lib.load().qmoe_synth_ternary(
                    sym[j].data_ptr(), h * w, seed & _M64, matrix_first_index(m), float(p_zero), dev.index,
                    int(torch.cuda.current_stream(dev).cuda_stream)))
            chunks.append(sub1_cuda.sub1pack_u8(trie, sym))
            del sym
        results[kind] = chunks
    # Interleave wi / wo per expert into flat arrays.
    total_codes = sum(int(c[0].numel()) for k in results for c in results[k])
    codes = torch.zeros(total_codes + 8, dtype=torch.int16, device=dev)
    row_off = torch.empty(n * (d_ff + 1 + d_model + 1), dtype=torch.int32, device=dev)
    minmax = torch.empty(2 * n * (d_ff + d_model), dtype=torch.bfloat16, device=dev)
    descs: List[Optional[MatrixDesc]] = [None] * (2 * n)
    code_pos = 0
    for kind, (h, w), which in (("wi", (d_ff, d_model), 0), ("wo", (d_model, d_ff), 1)):
        i = 0
        for c_codes, c_row_off, c_base, c_n in results[kind]:
            codes[code_pos:code_pos + c_codes.numel()] = c_codes
            base_host = c_base.tolist()
            n_host = c_n.tolist()
            for j in range(len(base_host)):
                e_local = i + j
                m_local = 2 * e_local + which
                ro_base = e_local * (d_ff + 1 + d_model + 1) + (0 if which == 0 else d_ff + 1)
                mm_base = e_local * (d_ff + d_model) + (0 if which == 0 else d_ff)
                row_off[ro_base:ro_base + h + 1] = c_row_off[j]
                mid = 2 * expert_ids[e_local] + which
                minmax[2 * mm_base:2 * (mm_base + h)] = row_scales(h, seed, mid).to(dev)
                descs[m_local] = MatrixDesc(code_pos + base_host[j], n_host[j], ro_base, mm_base, h, w)
            code_pos += c_codes.numel()
            i += len(base_host)
    return ExpertStore(codes, row_off, minmax, descs, d_model, d_ff)


def matrix_cpu(height: int, width: int, seed: int, matrix_id: int, p_zero: float = 0.90
               ) -> Tuple[np.ndarray, torch.Tensor]:
    """(symbols uint8[H, W], ter_minmax bf16[2H]) of one synthetic matrix, on the CPU."""
    sym = ternary_numpy(height * width, seed, matrix_first_index(matrix_id), p_zero).reshape(height, width)
    return sym, row_scales(height, seed, matrix_id)


def tokens(n: int, d_model: int, seed: int) -> torch.Tensor:
    g = torch.Generator().manual_seed(seed * 7919 + 17)
    return torch.randn(n, d_model, generator=g).bfloat16()


def router_logits(n: int, n_experts: int, seed: int, hot_experts: int = 0, hot_fraction: float = 0.0
                  ) -> torch.Tensor:
    """fp32 logits ~ N(0, 1).  With ``hot_experts`` > 0, ``hot_fraction`` of the tokens (the first
    ones) get a large logit on one of the first ``hot_experts`` experts (the skewed-router case)."""
    g = torch.Generator().manual_seed(seed * 104729 + 29)
    logits = torch.randn(n, n_experts, generator=g)
    if hot_experts > 0 and hot_fraction > 0:
        k = int(n * hot_fraction)
        idx = torch.arange(k) % hot_experts
        logits[torch.arange(k), idx] += 20.0
    return logits
