"""Host side of the compressed-expert path, mirroring the reference's ``sub1.py`` interface.

* :func:`setup` -- the fixed dictionary ``dec`` / ``trie`` (sub1.py:29-102), built by the native
  library in a few tens of milliseconds instead of at import time;
* :class:`Sub1Linear` -- same buffers (``w_comp``, ``row_off``, ``ter_minmax``, ``weight``), same
  ``forward`` / ``make`` contract as sub1.py:114-166, but one batched launch per call instead of one
  launch per token;
* :class:`ExpertStore` -- every expert matrix of a sparse layer in three flat device arrays, the
  layout the grouped kernels stream from;
* :class:`FasterMLP` -- the top-1 MoE layer of sub1.py:299-321 on one GPU: route, group, grouped
  FFN over all active experts, combine, without host synchronisation.
"""
from __future__ import annotations

import ctypes
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch
import torch.nn as nn

from . import _lib, sub1_cuda
from ._lib import MatrixDesc

# ---------------------------------------------------------------------------------------------
# Dictionary (sub1.py:29-111): built lazily, uploaded per device on first use.
# ---------------------------------------------------------------------------------------------
_DICT: Optional[Tuple[torch.Tensor, torch.Tensor]] = None
_DEC: Dict[int, torch.Tensor] = {}
_TRIE: Dict[int, torch.Tensor] = {}


def setup() -> Tuple[torch.Tensor, torch.Tensor]:
    """(dec int32[131072], trie int32[65537, 9]) on the CPU, bit-identical to the reference's
    ``setup()`` (sub1.py:29-102)."""
    global _DICT
    if _DICT is None:
        dec = np.zeros(2 * _lib.DICT_COUNT, dtype=np.int32)
        trie = np.zeros((_lib.DICT_COUNT + 1, 9), dtype=np.int32)
        _lib.check(_lib.load().qmoe_sub1_build_dictionary(dec.ctypes.data, trie.ctypes.data))
        _DICT = (torch.from_numpy(dec), torch.from_numpy(trie))
    return _DICT


def _dev_index(device) -> int:
    device = torch.device(device)
    if device.type != "cuda":
        raise RuntimeError("the sub1 kernels run on CUDA devices only")
    return torch.cuda.current_device() if device.index is None else device.index


def DEC(device) -> torch.Tensor:
    """The decoder table on ``device`` (the reference keeps one copy per GPU, sub1.py:110)."""
    i = _dev_index(device)
    if i not in _DEC:
        _DEC[i] = setup()[0].to(torch.device("cuda", i))
    return _DEC[i]


def TRIE(device) -> torch.Tensor:
    """The encoder trie on ``device`` (sub1.py:111)."""
    i = _dev_index(device)
    if i not in _TRIE:
        _TRIE[i] = setup()[1].to(torch.device("cuda", i)).contiguous()
    return _TRIE[i]


# ---------------------------------------------------------------------------------------------
# Sub1Linear (sub1.py:114-166)
# ---------------------------------------------------------------------------------------------
class Sub1Linear(nn.Module):
    """One compressed ``[height, width]`` matrix.  Buffers and state-dict keys are the reference's
    (sub1.py:118-130), so ``expNN.pt`` checkpoints load unchanged."""

    def __init__(self, height: int, comp_size: int):
        super().__init__()
        self.register_buffer("w_comp", torch.zeros(comp_size, dtype=torch.int16))
        self.register_buffer("row_off", torch.zeros(height + 1, dtype=torch.int32))
        self.register_buffer("ter_minmax", torch.zeros(2 * height, dtype=torch.bfloat16))
        # HuggingFace Switch checks `wi.weight.dtype`; the reference keeps an empty tensor for it.
        self.register_buffer("weight", torch.zeros(0, dtype=torch.bfloat16))

    @property
    def height(self) -> int:
        return self.row_off.shape[0] - 1

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        """``x[t, width] -> y[t, height]`` bf16; equals the reference's zero-then-accumulate loop
        (sub1.py:132-143) because ``0 + v`` is exact in bf16."""
        lead = x.shape[:-1]
        x2 = x.reshape(-1, x.shape[-1])
        if x2.dtype != torch.bfloat16:
            x2 = x2.bfloat16()
        if x2.stride(-1) != 1:
            x2 = x2.contiguous()
        y = torch.empty((x2.shape[0], self.height), dtype=torch.bfloat16, device=x2.device)
        if x2.shape[0]:
            sub1_cuda.sub1matmul(DEC(self.w_comp.device), self.w_comp, self.row_off, self.ter_minmax, x2, y, 0)
        return y.reshape(*lead, self.height)

    def forward_per_token(self, x: torch.Tensor) -> torch.Tensor:
        """The reference's literal protocol: zero ``y`` and call ``sub1matvec`` once per token."""
        y = torch.zeros((x.shape[0], self.height), dtype=torch.bfloat16, device=x.device)
        dec = DEC(self.w_comp.device)
        for i in range(y.shape[0]):
            sub1_cuda.sub1matvec(dec, self.w_comp, self.row_off, self.ter_minmax, x[i], y[i])
        return y

    @staticmethod
    def make(w: torch.Tensor) -> "Sub1Linear":
        """Compress a matrix whose rows hold at most three distinct values {min, 0, max}
        (sub1.py:145-166): symbols 1 / 2 mark the row minimum / maximum."""
        w = w.bfloat16()
        ter_minmax = torch.column_stack((w.min(1)[0], w.max(1)[0])).flatten()
        row_off = torch.zeros(w.shape[0] + 1, dtype=torch.int32, device=w.device)
        w_tern = torch.zeros(w.shape, dtype=torch.int32, device=w.device)
        w_tern[w == ter_minmax[0::2].reshape((-1, 1))] = 1
        w_tern[w == ter_minmax[1::2].reshape((-1, 1))] = 2
        w_comp = sub1_cuda.sub1pack(TRIE(w.device), w_tern, row_off)
        linear = Sub1Linear(w.shape[0], w_comp.shape[0])
        linear.w_comp = w_comp
        linear.row_off = row_off
        linear.ter_minmax = ter_minmax
        linear.weight = linear.weight.to(w.device)
        return linear


# ---------------------------------------------------------------------------------------------
# Expert store: all matrices of a sparse layer in flat arrays
# ---------------------------------------------------------------------------------------------
class ExpertStore:
    """Matrices ``2e`` (wi, ``[d_ff, d_model]``) and ``2e + 1`` (wo, ``[d_model, d_ff]``) of the
    local experts ``e`` of one sparse layer.

    ``codes`` int16: every matrix's stream, each starting on a 16-byte boundary;
    ``row_off`` int32: the matrices' ``height + 1`` offsets (relative to their own stream);
    ``minmax`` bf16: interleaved (min, max) per row;
    ``descs``: device array of ``qmoe_matrix_desc``."""

    def __init__(self, codes: torch.Tensor, row_off: torch.Tensor, minmax: torch.Tensor,
                 descs: Sequence[MatrixDesc], d_model: int, d_ff: int, interleave: bool = True,
                 dec: Optional[torch.Tensor] = None):
        assert codes.dtype == torch.int16 and row_off.dtype == torch.int32 and minmax.dtype == torch.bfloat16
        assert len(descs) % 2 == 0
        self.codes, self.row_off, self.minmax = codes, row_off, minmax
        self.d_model, self.d_ff = int(d_model), int(d_ff)
        self.n_experts = len(descs) // 2
        self.host_descs = list(descs)
        self._desc_array = (MatrixDesc * len(descs))(*descs)
        raw = np.frombuffer(bytes(self._desc_array), dtype=np.uint8).copy()
        self.descs = torch.from_numpy(raw).to(codes.device)
        self.device = codes.device
        self.dec = dec                                   # decoder table of these streams (None: the standard one)
        if dec is not None and dec.is_cuda:
            sub1_cuda.track_dec(dec)                     # the library's cache follows the tensor's life
        self.il_codes: Optional[torch.Tensor] = None     # lane-interleaved copy of the streams
        self.blk_base: Optional[torch.Tensor] = None     # int64, first 16-byte entry of every 32-row block
        self.il_rows: Optional[torch.Tensor] = None      # int32, row of its matrix kept at every position of the copy
        if interleave and codes.is_cuda and d_model % 32 == 0 and d_ff % 32 == 0:
            self.interleave()

    def _rows_by_length(self) -> torch.Tensor:
        """int32[total rows]: for every position of the interleaved store the row of its matrix that
        is kept there -- inside every 1024 positions of a matrix (what one CTA of the grouped kernel
        takes) the rows in decreasing order of their code count, stable."""
        dev = self.device
        total = sum(d.height for d in self.host_descs)
        rows = torch.empty(total, dtype=torch.int32, device=dev)
        by_height = {}
        for m, d in enumerate(self.host_descs):
            by_height.setdefault(d.height, []).append(m)
        for h, ms in by_height.items():
            for m0 in range(0, len(ms), 512):                     # bounded temporaries for large layers
                part = ms[m0:m0 + 512]
                ro_base = torch.tensor([self.host_descs[m].rowoff_base for m in part], dtype=torch.int64, device=dev)
                mm_base = torch.tensor([self.host_descs[m].minmax_base for m in part], dtype=torch.int64, device=dev)
                ro = self.row_off[ro_base[:, None] + torch.arange(h + 1, device=dev)[None, :]]
                length = ro[:, 1:] - ro[:, :-1]
                perm = torch.empty_like(length)
                for s0 in range(0, h, 1024):
                    seg = length[:, s0:s0 + 1024]
                    perm[:, s0:s0 + seg.shape[1]] = torch.argsort(seg, dim=1, descending=True, stable=True) + s0
                rows[(mm_base[:, None] + torch.arange(h, device=dev)[None, :]).reshape(-1)] = perm.reshape(-1).to(torch.int32)
        return rows

    def interleave(self, renumber: bool = True, sort_rows: bool = True) -> None:
        """Build the lane-interleaved copy of the code streams that the grouped kernel reads with
        coalesced loads (layout in include/qmoe_sub1.h), with code values renumbered by decreasing
        frequency so that the part of the table kept in shared memory serves as many lookups as
        possible, and with rows of similar length side by side (``sort_rows``) so that the 32 lanes of
        a warp finish together.  One-time cost when a store is created."""
        L = _lib.load()
        dev = self.device
        self.il_rows = self._rows_by_length() if sort_rows else None
        rows_ptr = None if self.il_rows is None else self.il_rows.data_ptr()
        dec = self.dec if self.dec is not None else DEC(dev)
        remap_ptr = None
        if renumber:
            hist = torch.zeros(_lib.DICT_COUNT, dtype=torch.int64, device=dev)
            last = self.host_descs[min(63, len(self.host_descs) - 1)]      # 64 matrices are sample enough
            n = min(last.code_base + last.n_codes, self.codes.numel())
            _lib.check(L.qmoe_sub1_code_histogram(self.codes.data_ptr(), n, hist.data_ptr(), dev.index, _s(dev)))
            order = torch.argsort(hist, descending=True, stable=True)
            remap = torch.empty(_lib.DICT_COUNT, dtype=torch.int32, device=dev)
            remap[order] = torch.arange(_lib.DICT_COUNT, dtype=torch.int32, device=dev)
            self.remap = remap
            remap_ptr = remap.data_ptr()
        self.il_table = torch.empty(_lib.DICT_COUNT, dtype=torch.int32, device=dev)
        self.il_dec = torch.empty(2 * _lib.DICT_COUNT, dtype=torch.int32, device=dev)
        _lib.check(L.qmoe_sub1_remap_tables(dec.data_ptr(), remap_ptr, self.il_table.data_ptr(),
                                            self.il_dec.data_ptr(), dev.index, _s(dev)))
        rows = sum(d.height for d in self.host_descs)
        units = torch.empty(rows // 32, dtype=torch.int32, device=dev)
        if rows_ptr is None:
            _lib.check(L.qmoe_moe_interleave_count(self.row_off.data_ptr(), self.descs.data_ptr(),
                                                   ctypes.addressof(self._desc_array), len(self.host_descs),
                                                   units.data_ptr(), dev.index, _s(dev)))
        else:
            _lib.check(L.qmoe_moe_interleave_count_rows(self.row_off.data_ptr(), self.descs.data_ptr(),
                                                        ctypes.addressof(self._desc_array), len(self.host_descs),
                                                        rows_ptr, units.data_ptr(), dev.index, _s(dev)))
        base = torch.zeros(rows // 32 + 1, dtype=torch.int64, device=dev)
        base[1:] = torch.cumsum(units, 0, dtype=torch.int64)
        total = int(base[-1].item())
        il = torch.empty((max(total, 1), 4), dtype=torch.int32, device=dev)
        if rows_ptr is None:
            _lib.check(L.qmoe_moe_interleave_emit(self.codes.data_ptr(), self.row_off.data_ptr(),
                                                  self.descs.data_ptr(), len(self.host_descs), base.data_ptr(),
                                                  remap_ptr, il.data_ptr(), dev.index, _s(dev)))
        else:
            _lib.check(L.qmoe_moe_interleave_emit_rows(self.codes.data_ptr(), self.row_off.data_ptr(),
                                                       self.descs.data_ptr(), len(self.host_descs), rows_ptr,
                                                       base.data_ptr(), remap_ptr, il.data_ptr(), dev.index, _s(dev)))
        self.il_codes, self.blk_base = il, base
        self.il_struct = _lib.InterleavedStore(il.data_ptr(), base.data_ptr(), self.il_table.data_ptr(),
                                               self.il_dec.data_ptr(), rows_ptr)

    def aliased(self, n_experts: int) -> "ExpertStore":
        """A store of ``n_experts`` experts whose expert ``e`` IS this store's expert
        ``e % self.n_experts``: the same arrays and the same interleaved copy under a longer descriptor
        table, nothing copied.  For measurements that need a full layer's routing pattern over weights
        small enough to stay in L2."""
        descs = [self.host_descs[2 * (e % self.n_experts) + k] for e in range(n_experts) for k in (0, 1)]
        other = ExpertStore(self.codes, self.row_off, self.minmax, descs, self.d_model, self.d_ff,
                            interleave=False, dec=self.dec)
        if self.il_codes is not None:
            for name in ("il_codes", "blk_base", "il_table", "il_dec", "il_struct", "il_rows"):
                setattr(other, name, getattr(self, name))
            if hasattr(self, "remap"):
                other.remap = self.remap
        return other

    @property
    def resident_bytes(self) -> int:
        """Device bytes held, including the interleaved copy."""
        total = self.row_off.numel() * 4 + self.minmax.numel() * 2
        if self.codes is not None:
            total += self.codes.numel() * 2
        if self.il_codes is not None:
            total += self.il_codes.numel() * 4 + self.blk_base.numel() * 8 + 3 * 4 * _lib.DICT_COUNT
            if getattr(self, "il_rows", None) is not None:
                total += self.il_rows.numel() * 4
        return total

    def drop_reference_layout(self) -> None:
        """Free the row-by-row streams and keep only the interleaved copy (about half the device
        memory).  Afterwards :meth:`matrix` is unavailable and experts with many tokens stay on the
        per-row kernel (the tensor-core tile path reads the row-by-row streams)."""
        if self.il_codes is None:
            raise RuntimeError("store has no interleaved copy to fall back on")
        self._code_elems = self.codes.numel()
        self.codes = None

    @property
    def compressed_bytes(self) -> int:
        n = self.codes.numel() if self.codes is not None else self._code_elems
        return n * 2 + self.row_off.numel() * 4 + self.minmax.numel() * 2

    def matrix_bytes(self, m: int) -> int:
        """Algorithmic bytes of one matrix: codes + row offsets + (min, max) pairs."""
        d = self.host_descs[m]
        return 2 * d.n_codes + 4 * (d.height + 1) + 4 * d.height

    def matrix(self, m: int) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
        """(w_comp, row_off, ter_minmax) views of matrix ``m`` in the reference's per-matrix layout."""
        d = self.host_descs[m]
        if self.codes is None:
            raise RuntimeError("the row-by-row streams of this store were dropped")
        return (self.codes[d.code_base:d.code_base + d.n_codes],
                self.row_off[d.rowoff_base:d.rowoff_base + d.height + 1],
                self.minmax[2 * d.minmax_base:2 * (d.minmax_base + d.height)])

    @staticmethod
    def from_linears(experts: Sequence[Tuple[Sub1Linear, Sub1Linear]], d_model: int, d_ff: int) -> "ExpertStore":
        """Concatenate (wi, wo) pairs of :class:`Sub1Linear` into a store."""
        parts = []
        for wi, wo in experts:
            parts.append((wi.w_comp, wi.row_off, wi.ter_minmax, d_ff, d_model))
            parts.append((wo.w_comp, wo.row_off, wo.ter_minmax, d_model, d_ff))
        return ExpertStore.from_matrices(parts, d_model, d_ff)

    @staticmethod
    def from_matrices(parts: Sequence[Tuple[torch.Tensor, torch.Tensor, torch.Tensor, int, int]],
                      d_model: int, d_ff: int) -> "ExpertStore":
        dev = parts[0][0].device
        descs: List[MatrixDesc] = []
        code_base = rowoff_base = minmax_base = 0
        for w_comp, row_off, minmax, h, w in parts:
            assert row_off.numel() == h + 1 and minmax.numel() == 2 * h
            descs.append(MatrixDesc(code_base, w_comp.numel(), rowoff_base, minmax_base, h, w))
            code_base += (w_comp.numel() + 7) // 8 * 8
            rowoff_base += h + 1
            minmax_base += h
        codes = torch.zeros(max(code_base, 8), dtype=torch.int16, device=dev)
        row_offs = torch.empty(rowoff_base, dtype=torch.int32, device=dev)
        minmaxs = torch.empty(2 * minmax_base, dtype=torch.bfloat16, device=dev)
        for d, (w_comp, row_off, minmax, h, w) in zip(descs, parts):
            codes[d.code_base:d.code_base + d.n_codes] = w_comp.view(torch.int16)
            row_offs[d.rowoff_base:d.rowoff_base + h + 1] = row_off
            minmaxs[2 * d.minmax_base:2 * (d.minmax_base + h)] = minmax
        return ExpertStore(codes, row_offs, minmaxs, descs, d_model, d_ff)


# ---------------------------------------------------------------------------------------------
# Device-side MoE plumbing shared by the single-GPU and the expert-parallel layer
# ---------------------------------------------------------------------------------------------
def _s(dev: torch.device) -> int:
    return int(torch.cuda.current_stream(dev).cuda_stream)


_MM_OUT_DTYPE_OK: Optional[bool] = None


class RouterClassifier:
    """The router's bias-free classifier, evaluated in fp32 as the Switch router does (its
    ``hidden_states.to(float32)`` + fp32 classifier).  When every weight is exactly representable in
    bf16 (checkpoints store the classifier in bf16) the product of bf16 inputs with fp32
    accumulation gives the same logits up to summation order, so the bf16 tensor-core GEMM with an
    fp32 result is used; otherwise a plain fp32 matmul."""

    def __init__(self, weight: torch.Tensor, device):
        self.w32 = weight.to(device, torch.float32).contiguous()
        w16 = self.w32.bfloat16()
        self.w16 = w16.contiguous() if bool((w16.float() == self.w32).all()) else None

    def __call__(self, hidden_bf16: torch.Tensor) -> torch.Tensor:
        global _MM_OUT_DTYPE_OK
        if self.w16 is not None and hidden_bf16.dtype == torch.bfloat16 and _MM_OUT_DTYPE_OK is not False:
            try:
                out = torch.mm(hidden_bf16, self.w16.t(), out_dtype=torch.float32)
                _MM_OUT_DTYPE_OK = True
                return out
            except (TypeError, RuntimeError):
                _MM_OUT_DTYPE_OK = False
        return hidden_bf16.float() @ self.w32.t()


def route_top1(logits: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """(choice int32[n], prob bf16[n]) from fp32 logits ``[n, E]``."""
    assert logits.is_cuda and logits.dtype == torch.float32 and logits.dim() == 2 and logits.is_contiguous()
    n, e = logits.shape
    dev = logits.device
    choice = torch.empty(n, dtype=torch.int32, device=dev)
    prob = torch.empty(n, dtype=torch.bfloat16, device=dev)
    _lib.check(_lib.load().qmoe_moe_route(logits.data_ptr(), choice.data_ptr(), prob.data_ptr(), n, e,
                                          dev.index, _s(dev)))
    return choice, prob


def rank_buckets(choice: torch.Tensor, n_buckets: int, seq_len: int, capacity: int):
    """(bucket, rank, counts, offsets): capacity rule, stable ranks, bucket sizes and their
    exclusive prefix sums (``offsets`` has ``n_buckets + 1`` entries)."""
    assert choice.is_cuda and choice.dtype == torch.int32 and choice.is_contiguous()
    n = choice.numel()
    dev = choice.device
    bucket = torch.empty(n, dtype=torch.int32, device=dev)
    rank = torch.empty(n, dtype=torch.int32, device=dev)
    counts = torch.empty(n_buckets, dtype=torch.int32, device=dev)
    offsets = torch.empty(n_buckets + 1, dtype=torch.int32, device=dev)
    L = _lib.load()
    _lib.check(L.qmoe_moe_rank(choice.data_ptr(), bucket.data_ptr(), rank.data_ptr(), counts.data_ptr(), n,
                               n_buckets, max(int(seq_len), 1), int(capacity), dev.index, _s(dev)))
    _lib.check(L.qmoe_moe_scan(counts.data_ptr(), offsets.data_ptr(), n_buckets, dev.index, _s(dev)))
    return bucket, rank, counts, offsets


def permute_rows(bucket, rank, offsets, hidden: torch.Tensor, xs: torch.Tensor) -> torch.Tensor:
    """``xs[offsets[bucket] + rank] = hidden[token]``; returns slot int32[n] (-1 = dropped)."""
    n, d = hidden.shape
    dev = hidden.device
    slot = torch.empty(n, dtype=torch.int32, device=dev)
    _lib.check(_lib.load().qmoe_moe_permute(bucket.data_ptr(), rank.data_ptr(), offsets.data_ptr(),
                                            slot.data_ptr(), hidden.data_ptr(), xs.data_ptr(), n, d,
                                            hidden.stride(0), xs.stride(0), dev.index, _s(dev)))
    return slot


def unpermute_rows(ys: torch.Tensor, slot: torch.Tensor, out: torch.Tensor) -> None:
    n, d = out.shape
    dev = out.device
    _lib.check(_lib.load().qmoe_moe_unpermute(ys.data_ptr(), slot.data_ptr(), out.data_ptr(), n, d,
                                              ys.stride(0), out.stride(0), dev.index, _s(dev)))


def capacity_rule(choice: torch.Tensor, n_experts: int, seq_len: int, capacity: int) -> torch.Tensor:
    """``expert[t]`` = ``choice[t]`` if the router's capacity rule keeps token ``t`` (fewer than
    ``capacity`` earlier tokens of its sequence chose the same expert), else -1.  One launch."""
    n = choice.numel()
    dev = choice.device
    expert = torch.empty(n, dtype=torch.int32, device=dev)
    _lib.check(_lib.load().qmoe_moe_keep(choice.data_ptr(), expert.data_ptr(), n, int(n_experts),
                                         max(int(seq_len), 1), int(capacity), dev.index, _s(dev)))
    return expert


def plan_rows(n_buckets: int, bucket: Optional[torch.Tensor] = None, rows: Optional[torch.Tensor] = None,
              d_model: int = 0):
    """Group rows by bucket, stable in row order, in one launch.  The bucket of row ``i`` is
    ``bucket[i]`` or, with ``rows`` (bf16 ``[m, d_model + 8]`` as exchanged by the expert-parallel
    layer), the int32 in the row's trailer; values outside ``[0, n_buckets)`` mean "no row".
    Returns (offsets int32[n_buckets + 1], slot_of_row int32[m], row_of_slot int32[m])."""
    src = rows if rows is not None else bucket
    m = src.shape[0]
    dev = src.device
    offsets = torch.empty(n_buckets + 1, dtype=torch.int32, device=dev)
    slot_of_row = torch.empty(m, dtype=torch.int32, device=dev)
    row_of_slot = torch.zeros(m, dtype=torch.int32, device=dev)
    if rows is not None:
        assert rows.dtype == torch.bfloat16 and rows.stride(1) == 1 and rows.shape[1] >= d_model + 2
        args = (rows.data_ptr(), rows.stride(0), int(d_model), None)
    else:
        assert bucket.dtype == torch.int32 and bucket.is_contiguous()
        args = (None, 0, 0, bucket.data_ptr())
    _lib.check(_lib.load().qmoe_moe_plan(*args, m, int(n_buckets), offsets.data_ptr(), slot_of_row.data_ptr(),
                                         row_of_slot.data_ptr(), dev.index, _s(dev)))
    return offsets, slot_of_row, row_of_slot


def ep_dispatch(choice: torch.Tensor, hidden: torch.Tensor, n_experts: int, n_ranks: int, seq_len: int,
                expert_capacity: int, pair_capacity: int, overflow: torch.Tensor):
    """Capacity rule, destination ranks and the packing of the kept rows into ``n_ranks *
    pair_capacity`` exchange slots of ``d_model + 8`` bf16 (row + 16-byte trailer with the expert's
    index on its rank), in two launches.  Returns (expert int32[n] or -1, slot int32[n] or -1, send).
    Tokens that do not fit their pair's capacity get slot -1 and are counted in ``overflow``
    (int32[1], zeroed by the caller once)."""
    n, d = hidden.shape
    dev = hidden.device
    expert = torch.empty(n, dtype=torch.int32, device=dev)
    dest = torch.empty(n, dtype=torch.int32, device=dev)
    slot = torch.empty(n, dtype=torch.int32, device=dev)
    send = torch.empty((n_ranks * pair_capacity, d + 8), dtype=torch.bfloat16, device=dev)
    assert hidden.dtype == torch.bfloat16 and hidden.stride(1) == 1 and choice.dtype == torch.int32
    _lib.check(_lib.load().qmoe_moe_ep_dispatch(
        choice.data_ptr(), hidden.data_ptr(), hidden.stride(0), expert.data_ptr(), dest.data_ptr(), slot.data_ptr(),
        send.data_ptr(), overflow.data_ptr(), n, int(n_experts), int(n_ranks), max(int(seq_len), 1),
        int(expert_capacity), int(pair_capacity), d, dev.index, _s(dev)))
    return expert, slot, send


def ep_dispatch_peer(choice: torch.Tensor, hidden: torch.Tensor, n_experts: int, n_ranks: int, seq_len: int,
                     expert_capacity: int, pair_capacity: int, overflow: torch.Tensor, dest_blocks: torch.Tensor):
    """:func:`ep_dispatch` that stores the kept rows straight into the destinations' receive buffers
    (``dest_blocks`` int64[n_ranks]: where this rank's block starts in every rank's buffer, as
    addresses valid on this GPU).  Returns (expert, slot)."""
    n, d = hidden.shape
    dev = hidden.device
    expert = torch.empty(n, dtype=torch.int32, device=dev)
    dest = torch.empty(n, dtype=torch.int32, device=dev)
    slot = torch.empty(n, dtype=torch.int32, device=dev)
    assert hidden.dtype == torch.bfloat16 and hidden.stride(1) == 1 and choice.dtype == torch.int32
    assert dest_blocks.dtype == torch.int64 and dest_blocks.numel() == n_ranks and dest_blocks.is_cuda
    _lib.check(_lib.load().qmoe_moe_ep_dispatch_peer(
        choice.data_ptr(), hidden.data_ptr(), hidden.stride(0), expert.data_ptr(), dest.data_ptr(), slot.data_ptr(),
        dest_blocks.data_ptr(), overflow.data_ptr(), n, int(n_experts), int(n_ranks), max(int(seq_len), 1),
        int(expert_capacity), int(pair_capacity), d, dev.index, _s(dev)))
    return expert, slot


def plan_rows_peer(n_buckets: int, rows: torch.Tensor, d_model: int, out_blocks: torch.Tensor, rows_per_block: int,
                   out_row_bytes: int):
    """:func:`plan_rows` over received rows that also returns, per slot, the address of its result
    row in the source rank's return buffer (int64[m])."""
    m = rows.shape[0]
    dev = rows.device
    offsets = torch.empty(n_buckets + 1, dtype=torch.int32, device=dev)
    slot_of_row = torch.empty(m, dtype=torch.int32, device=dev)
    row_of_slot = torch.zeros(m, dtype=torch.int32, device=dev)
    out_ptrs = torch.zeros(m, dtype=torch.int64, device=dev)
    assert rows.dtype == torch.bfloat16 and rows.stride(1) == 1 and rows.shape[1] >= d_model + 2
    assert out_blocks.dtype == torch.int64 and out_blocks.is_cuda
    _lib.check(_lib.load().qmoe_moe_plan_peer(
        rows.data_ptr(), rows.stride(0), int(d_model), m, int(n_buckets), offsets.data_ptr(), slot_of_row.data_ptr(),
        row_of_slot.data_ptr(), out_blocks.data_ptr(), int(rows_per_block), int(out_row_bytes), out_ptrs.data_ptr(),
        dev.index, _s(dev)))
    return offsets, slot_of_row, row_of_slot, out_ptrs


def grouped_ffn_scatter(store: ExpertStore, offsets: torch.Tensor, xs: torch.Tensor, x_rows: Optional[torch.Tensor],
                        y_row_ptrs: torch.Tensor, max_slots: int, work: Optional[torch.Tensor] = None) -> None:
    """:func:`grouped_ffn_rows` whose result of slot ``s`` is stored at the address ``y_row_ptrs[s]``
    (``d_model`` bf16; the row may lie in a peer GPU's memory)."""
    dev = store.device
    L = _lib.load()
    if max_slots == 0:
        return
    hs = torch.empty((max_slots, store.d_ff), dtype=torch.bfloat16, device=dev)
    nbytes = int(L.qmoe_moe_work_bytes(store.n_experts, max_slots, store.d_model, store.d_ff))
    if work is None or work.numel() < nbytes:
        work = torch.empty(nbytes, dtype=torch.uint8, device=dev)
    assert xs.dtype == torch.bfloat16 and xs.stride(1) == 1 and y_row_ptrs.dtype == torch.int64
    dec = store.dec if store.dec is not None else DEC(dev)
    _lib.check(L.qmoe_moe_grouped_ffn_scatter(
        dec.data_ptr(), None if store.codes is None else store.codes.data_ptr(), store.row_off.data_ptr(),
        store.minmax.data_ptr(), store.descs.data_ptr(),
        ctypes.addressof(store.il_struct) if store.il_codes is not None else None, offsets.data_ptr(),
        xs.data_ptr(), xs.stride(0), None if x_rows is None else x_rows.data_ptr(), hs.data_ptr(),
        y_row_ptrs.data_ptr(), work.data_ptr(), store.n_experts, max_slots, store.d_model, store.d_ff, dev.index,
        _s(dev)))


def grouped_ffn_rows(store: ExpertStore, offsets: torch.Tensor, xs: torch.Tensor, x_rows: Optional[torch.Tensor],
                     ys: torch.Tensor, y_rows: Optional[torch.Tensor], max_slots: int,
                     work: Optional[torch.Tensor] = None) -> torch.Tensor:
    """:func:`grouped_ffn` through row lists: slot ``s`` reads row ``x_rows[s]`` of ``xs`` (any row
    stride) and writes row ``y_rows[s]`` of ``ys``; ``None`` means ``s`` itself.  No sorted copy of
    the activations is made."""
    dev = store.device
    L = _lib.load()
    if max_slots == 0:
        return ys
    hs = torch.empty((max_slots, store.d_ff), dtype=torch.bfloat16, device=dev)
    nbytes = int(L.qmoe_moe_work_bytes(store.n_experts, max_slots, store.d_model, store.d_ff))
    if work is None or work.numel() < nbytes:
        work = torch.empty(nbytes, dtype=torch.uint8, device=dev)
    assert xs.dtype == torch.bfloat16 and ys.dtype == torch.bfloat16 and xs.stride(1) == 1 and ys.stride(1) == 1
    dec = store.dec if store.dec is not None else DEC(dev)
    _lib.check(L.qmoe_moe_grouped_ffn_rows(
        dec.data_ptr(), None if store.codes is None else store.codes.data_ptr(), store.row_off.data_ptr(),
        store.minmax.data_ptr(), store.descs.data_ptr(),
        ctypes.addressof(store.il_struct) if store.il_codes is not None else None, offsets.data_ptr(),
        xs.data_ptr(), xs.stride(0), None if x_rows is None else x_rows.data_ptr(), hs.data_ptr(), ys.data_ptr(),
        ys.stride(0), None if y_rows is None else y_rows.data_ptr(), work.data_ptr(), store.n_experts, max_slots,
        store.d_model, store.d_ff, dev.index, _s(dev)))
    return ys


def grouped_ffn(store: ExpertStore, offsets: torch.Tensor, xs: torch.Tensor, max_slots: int,
                work: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``wo(ReLU(wi(x)))`` for tokens sorted by local expert (``offsets`` int32[E+1]); returns
    ``ys`` bf16[max_slots, d_model].  Rows past ``offsets[E]`` are left untouched."""
    dev = store.device
    L = _lib.load()
    hs = torch.empty((max_slots, store.d_ff), dtype=torch.bfloat16, device=dev)
    ys = torch.empty((max_slots, store.d_model), dtype=torch.bfloat16, device=dev)
    if max_slots == 0:
        return ys
    nbytes = int(L.qmoe_moe_work_bytes(store.n_experts, max_slots, store.d_model, store.d_ff))
    if work is None or work.numel() < nbytes:
        work = torch.empty(nbytes, dtype=torch.uint8, device=dev)
    assert xs.is_contiguous() and xs.shape[1] == store.d_model
    dec = store.dec if store.dec is not None else DEC(dev)
    if store.il_codes is not None:
        _lib.check(L.qmoe_moe_grouped_ffn_interleaved(
            dec.data_ptr(), None if store.codes is None else store.codes.data_ptr(),
            store.row_off.data_ptr(), store.minmax.data_ptr(),
            store.descs.data_ptr(), ctypes.addressof(store.il_struct), offsets.data_ptr(),
            xs.data_ptr(), hs.data_ptr(), ys.data_ptr(), work.data_ptr(), store.n_experts, max_slots,
            store.d_model, store.d_ff, dev.index, _s(dev)))
        return ys
    _lib.check(L.qmoe_moe_grouped_ffn(dec.data_ptr(), store.codes.data_ptr(), store.row_off.data_ptr(),
                                      store.minmax.data_ptr(), store.descs.data_ptr(), offsets.data_ptr(),
                                      xs.data_ptr(), hs.data_ptr(), ys.data_ptr(), work.data_ptr(),
                                      store.n_experts, max_slots, store.d_model, store.d_ff, dev.index, _s(dev)))
    return ys


def work_plan(work: torch.Tensor, max_slots: int, d_ff: int) -> Dict[str, int]:
    """What the last :func:`grouped_ffn` call that used ``work`` planned (synchronises): numbers of
    row-per-thread and row-per-warp work items of wi and wo, rows per row-per-thread item, the tile
    items, the tokens decoded together, and the wo items that also cover their matrix's remainder
    rows (a height that is not a multiple of 1024) one row per warp."""
    out = (ctypes.c_int32 * 10)()
    dev = work.device
    _lib.check(_lib.load().qmoe_moe_work_summary(work.data_ptr(), int(max_slots), int(d_ff), out, dev.index, _s(dev)))
    return {"wi_items": out[0], "wo_items": out[1], "wi_warp_items": out[2], "wo_warp_items": out[3],
            "wi_rows_per_item": out[4], "wo_rows_per_item": out[5], "tile_wi_items": out[6],
            "tile_wo_items": out[7], "group_tokens": out[8], "wo_items_with_remainder": out[9]}


def tile_timeouts(device, reset: bool = False) -> int:
    """Number of tensor-core tile CTAs on ``device`` whose bounded wait gave up since the last reset
    (0 in normal operation).  Synchronises the device: call it where the caller synchronises anyway.
    A non-zero value means that grouped-FFN outputs produced since the last reset hold zeros for the
    rows those CTAs did not finish."""
    count = ctypes.c_int(0)
    _lib.check(_lib.load().qmoe_moe_tile_timeouts(_dev_index(device), 1 if reset else 0, ctypes.byref(count)))
    return int(count.value)


def check_tile_status(device) -> None:
    """Raise if a tile kernel on ``device`` reported a timeout (and clear the status)."""
    n = tile_timeouts(device, reset=True)
    if n:
        raise _lib.QmoeError(_lib.ERR_TIMEOUT, f"{n} tensor-core tile CTA(s) gave up waiting; outputs are incomplete")


def combine(ys: torch.Tensor, hidden: torch.Tensor, slot: torch.Tensor, prob: torch.Tensor) -> torch.Tensor:
    """``out[t] = prob[t] * (ys[slot[t]] if slot[t] >= 0 else hidden[t])`` (sub1.py:312,317-318)."""
    n, d = hidden.shape
    dev = hidden.device
    out = torch.empty_like(hidden)
    assert hidden.is_contiguous() and (ys.numel() == 0 or ys.is_contiguous())
    _lib.check(_lib.load().qmoe_moe_combine(ys.data_ptr(), hidden.data_ptr(), slot.data_ptr(), prob.data_ptr(),
                                            out.data_ptr(), n, d, dev.index, _s(dev)))
    return out


def route_small(logits: torch.Tensor, hidden: torch.Tensor, n_experts: int, capacity: int):
    """Routing, capacity rule, ranks, bucket offsets and the row permutation for at most 32 tokens
    of one sequence in one launch; returns (prob bf16[n], offsets int32[E + 1], slot int32[n], xs)."""
    n, d = hidden.shape
    dev = hidden.device
    assert logits.dtype == torch.float32 and logits.is_contiguous() and hidden.is_contiguous() and n <= 32
    prob = torch.empty(n, dtype=torch.bfloat16, device=dev)
    offsets = torch.empty(n_experts + 1, dtype=torch.int32, device=dev)
    slot = torch.empty(n, dtype=torch.int32, device=dev)
    xs = torch.empty_like(hidden)
    _lib.check(_lib.load().qmoe_moe_route_small(logits.data_ptr(), hidden.data_ptr(), n, n_experts, d,
                                                int(capacity), prob.data_ptr(), offsets.data_ptr(), slot.data_ptr(),
                                                xs.data_ptr(), dev.index, _s(dev)))
    return prob, offsets, slot, xs


def combine_add(ys: torch.Tensor, hidden: torch.Tensor, slot: torch.Tensor, prob: torch.Tensor,
                residual: torch.Tensor) -> torch.Tensor:
    """``residual + combine(ys, hidden, slot, prob)`` in one launch (bf16 addition)."""
    n, d = hidden.shape
    dev = hidden.device
    out = torch.empty_like(hidden)
    assert hidden.is_contiguous() and residual.is_contiguous() and (ys.numel() == 0 or ys.is_contiguous())
    _lib.check(_lib.load().qmoe_moe_combine_add(ys.data_ptr(), hidden.data_ptr(), slot.data_ptr(), prob.data_ptr(),
                                                residual.data_ptr(), out.data_ptr(), n, d, dev.index, _s(dev)))
    return out


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    """T5-style RMS norm of bf16 rows in one launch."""
    assert x.is_cuda and x.dtype == torch.bfloat16 and x.is_contiguous() and weight.dtype == torch.bfloat16
    out = torch.empty_like(x)
    d = x.shape[-1]
    _lib.check(_lib.load().qmoe_rms_norm(x.data_ptr(), weight.data_ptr(), out.data_ptr(), x.numel() // d, d,
                                         float(eps), x.device.index, _s(x.device)))
    return out


def gemv(x: torch.Tensor, w: torch.Tensor, ln_weight: Optional[torch.Tensor] = None,
         residual: Optional[torch.Tensor] = None, f32_out: bool = False, want_normed: bool = False):
    """``w @ x`` for one token (``x`` bf16 [1, k], ``w`` bf16 [n, k]) in one launch, optionally with
    the RMS norm of ``x`` in front (``ln_weight``) or a residual behind.  Returns ``y`` [1, n], or
    ``(y, normed_x)`` with ``want_normed``."""
    n, k = w.shape
    dev = x.device
    assert x.numel() == k and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and w.is_contiguous()
    y = torch.empty((1, n), dtype=torch.float32 if f32_out else torch.bfloat16, device=dev)
    normed = torch.empty((1, k), dtype=torch.bfloat16, device=dev) if want_normed else None
    _lib.check(_lib.load().qmoe_gemv(
        x.data_ptr(), None if ln_weight is None else ln_weight.data_ptr(), w.data_ptr(),
        None if residual is None else residual.data_ptr(), y.data_ptr(),
        None if normed is None else normed.data_ptr(), n, k, 1e-6, 1 if f32_out else 0, dev.index, _s(dev)))
    return (y, normed) if want_normed else y


def decode_attention(qkv: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, pos: torch.Tensor,
                     scale: float = 0.0, bias: Optional[torch.Tensor] = None,
                     status: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Causal self-attention of one new token (``qkv`` bf16 [3, heads, head_dim]) against caches
    bf16 [heads, max_len, head_dim]; the token's key / value are stored at ``pos`` (device int64[1]).
    ``scale`` multiplies the scores (0: 1 / sqrt(head_dim); T5 / Switch attention uses 1); ``bias``
    fp32 [heads, max_len] is added to them (a relative-position bias); with ``status`` (int32[1]) a
    position outside the cache is refused and counted instead of clamped."""
    heads, max_len, hd = k_cache.shape
    assert qkv.is_contiguous() and k_cache.is_contiguous() and v_cache.is_contiguous() and pos.dtype == torch.int64
    out = torch.empty((1, heads * hd), dtype=torch.bfloat16, device=qkv.device)
    if scale == 0.0 and bias is None and status is None:
        _lib.check(_lib.load().qmoe_decode_attention(qkv.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(),
                                                     pos.data_ptr(), out.data_ptr(), heads, hd, max_len,
                                                     qkv.device.index, _s(qkv.device)))
        return out
    assert bias is None or (bias.dtype == torch.float32 and bias.is_contiguous() and bias.shape == (heads, max_len))
    assert status is None or status.dtype == torch.int32
    _lib.check(_lib.load().qmoe_decode_attention_ex(
        qkv.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), pos.data_ptr(), out.data_ptr(), heads, hd, max_len,
        float(scale), None if bias is None else bias.data_ptr(), None if status is None else status.data_ptr(),
        qkv.device.index, _s(qkv.device)))
    return out


# ---------------------------------------------------------------------------------------------
# FasterMLP (sub1.py:299-321): the single-GPU top-1 MoE layer
# ---------------------------------------------------------------------------------------------
class FasterMLP(nn.Module):
    """Top-1 MoE layer over compressed experts.

    ``router_weight``: the router classifier ``[n_experts, d_model]`` (no bias, as in HF Switch);
    ``store``: the layer's :class:`ExpertStore`; ``expert_capacity``: tokens of one sequence an
    expert accepts before the router drops them (dropped tokens pass through scaled by their router
    probability, sub1.py:312,318).  Unlike the reference there is no loop over active experts and
    no host synchronisation: one grouped launch per linear covers every expert that got tokens, and
    the tokens are not copied into expert order (the kernels read them through a row list)."""

    def __init__(self, router_weight: Optional[torch.Tensor], store: ExpertStore, expert_capacity: int = 1024):
        super().__init__()
        self.store = store
        self.expert_capacity = int(expert_capacity)
        self.router = None if router_weight is None else RouterClassifier(router_weight, store.device)

    def router_logits(self, hidden2d: torch.Tensor) -> torch.Tensor:
        return self.router(hidden2d)

    def forward(self, hidden_states: torch.Tensor, router_logits: Optional[torch.Tensor] = None):
        shape = hidden_states.shape
        seq_len = shape[-2] if hidden_states.dim() >= 3 else shape[0]
        hidden = hidden_states.reshape(-1, shape[-1]).to(self.store.device)
        if hidden.dtype != torch.bfloat16 or not hidden.is_contiguous():
            hidden = hidden.bfloat16().contiguous()
        n = hidden.shape[0]
        if router_logits is None:
            router_logits = self.router_logits(hidden)
        logits2d = router_logits.reshape(n, -1).float().contiguous()
        choice, prob = route_top1(logits2d)
        expert = capacity_rule(choice, self.store.n_experts, seq_len, self.expert_capacity)
        # tokens grouped by expert without copying them: the grouped FFN reads row row_of_slot[s]
        offsets, slot, row_of_slot = plan_rows(self.store.n_experts, bucket=expert)
        ys = torch.empty_like(hidden)
        grouped_ffn_rows(self.store, offsets, hidden, row_of_slot, ys, None, n)
        out = combine(ys, hidden, slot, prob)
        expert_index = torch.clamp(expert, min=0).to(torch.int64)
        lead = shape[:-1]
        return (out.reshape(shape).to(hidden_states.device),
                (router_logits.reshape(*lead, -1), expert_index.reshape(lead)))
