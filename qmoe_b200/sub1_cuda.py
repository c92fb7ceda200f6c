"""Drop-in replacement of the reference's ``sub1_cuda`` extension module.

``sub1matvec`` and ``sub1pack`` keep the reference's signatures, dtypes and in-place effects
(sub1_cuda.cpp:35-59); behind them are the sm_100a kernels of ``libqmoe_sub1.so``, reached through
its C ABI with raw device pointers and torch's current stream.  ``sub1matmul`` / ``sub1decode`` /
``sub1pack_u8`` are additive entry points.  There is no CPU path: CPU tensors are rejected.

To let unmodified reference code ``import sub1_cuda``, call :func:`install` first (it registers this
module under that name in ``sys.modules``).
"""
from __future__ import annotations

import sys
from typing import Optional, Tuple

import torch

from . import _lib
from ._lib import FLAG_ACCUMULATE, FLAG_RELU, QmoeError  # noqa: F401  (re-exported)


def install() -> None:
    """Register this module as ``sub1_cuda`` so that ``import sub1_cuda`` resolves to it."""
    sys.modules["sub1_cuda"] = sys.modules[__name__]


def _stream(device: torch.device) -> int:
    return int(torch.cuda.current_stream(device).cuda_stream)


def _need(t: torch.Tensor, name: str, dtype, device: Optional[torch.device] = None) -> None:
    if not isinstance(t, torch.Tensor):
        raise TypeError(f"{name} must be a torch.Tensor")
    if not t.is_cuda:
        raise RuntimeError(f"{name} must be a CUDA tensor (there is no CPU implementation)")
    dtypes = dtype if isinstance(dtype, tuple) else (dtype,)
    if t.dtype not in dtypes:
        raise TypeError(f"{name} must have dtype {dtypes}, got {t.dtype}")
    if not t.is_contiguous():
        raise ValueError(f"{name} must be contiguous")
    if device is not None and t.device != device:
        raise RuntimeError(f"{name} is on {t.device}, expected {device}")


def _check_matrix(dec, w_comp, row_off, ter_minmax) -> Tuple[torch.device, int]:
    _need(dec, "dec", torch.int32)
    dev = dec.device
    if dec.numel() != 2 * _lib.DICT_COUNT:
        raise ValueError("dec must hold 2 * 65536 int32 words")
    _need(w_comp, "w_comp", (torch.int16, torch.uint16), dev)
    _need(row_off, "row_off", torch.int32, dev)
    _need(ter_minmax, "ter_minmax", torch.bfloat16, dev)
    height = row_off.numel() - 1
    if height < 1 or ter_minmax.numel() != 2 * height:
        raise ValueError("row_off must have height + 1 entries and ter_minmax 2 * height")
    track_dec(dec)
    return dev, height


_MATVEC_CHECKED = {}
_TRACKED_DEC = set()


def track_dec(dec: torch.Tensor) -> None:
    """Tie the library's cache for this decoder table to the life of the tensor.

    The library keys its derived table by the address of ``dec``.  torch's allocator hands freed
    addresses out again, so when ``dec`` is garbage collected the cached table (and the remembered
    argument checks of :func:`sub1matvec`) for its address are dropped: a different table that
    later lands on the same address is derived afresh.  Overwriting a table IN PLACE is not seen;
    call ``qmoe_sub1_forget`` / ``qmoe_sub1_release`` after that."""
    import weakref
    ptr, index = dec.data_ptr(), dec.device.index
    if (ptr, index) in _TRACKED_DEC:
        return
    _TRACKED_DEC.add((ptr, index))

    def forget(ptr=ptr, index=index):
        _TRACKED_DEC.discard((ptr, index))
        for key in [k for k in _MATVEC_CHECKED if k[0] == ptr]:
            del _MATVEC_CHECKED[key]
        try:
            _lib.load().qmoe_sub1_forget(ptr, index)
        except Exception:  # interpreter shutdown
            pass

    weakref.finalize(dec, forget)


def sub1matvec(dec: torch.Tensor, w_comp: torch.Tensor, row_off: torch.Tensor,
               ter_minmax: torch.Tensor, x: torch.Tensor, y: torch.Tensor) -> None:
    """``y += bf16(W x)`` for one compressed matrix and one bf16 vector, in place.

    Same contract as the reference binding (sub1_cuda.cpp:35-45): height = ``y.numel()``, width =
    ``x.numel()`` (sub1_cuda_kernel.cu:78-79); unlike the reference, any height and any width up to
    8192 works, and unsupported input raises instead of silently doing nothing.  The argument checks
    of a (dec, w_comp, row_off, ter_minmax) quadruple are remembered by storage address and shape, so
    the per-token loop of ``Sub1Linear`` pays them once."""
    key = (dec.data_ptr(), w_comp.data_ptr(), row_off.data_ptr(), ter_minmax.data_ptr(),
           w_comp.numel(), row_off.numel())
    hit = _MATVEC_CHECKED.get(key)
    if hit is None:
        dev, height = _check_matrix(dec, w_comp, row_off, ter_minmax)
        if len(_MATVEC_CHECKED) > 65536:
            _MATVEC_CHECKED.clear()
        hit = _MATVEC_CHECKED[key] = (dev, height, _lib.load().qmoe_sub1_matvec)
    dev, height, fn = hit
    if (x.dtype is not torch.bfloat16 or y.dtype is not torch.bfloat16 or x.device != dev or y.device != dev
            or not x.is_contiguous() or not y.is_contiguous()):
        _need(x, "x", torch.bfloat16, dev)
        _need(y, "y", torch.bfloat16, dev)
    if y.numel() != height:
        raise ValueError(f"y has {y.numel()} elements but row_off describes {height} rows")
    rc = fn(key[0], key[1], key[2], key[3], x.data_ptr(), y.data_ptr(), height, x.numel(), key[4], dev.index,
            torch.cuda.current_stream(dev).cuda_stream)
    if rc:
        _lib.check(rc)


def sub1matvec_noalloc(dec: torch.Tensor, w_comp: torch.Tensor, row_off: torch.Tensor,
                       ter_minmax: torch.Tensor, x: torch.Tensor, y: torch.Tensor) -> None:
    """``sub1matvec`` for hosts that must not allocate GPU memory (an embedding framework that owns
    the device's memory, a fully pooled budget, a thread that may not block in the allocator).

    Same arguments and result.  Neither this wrapper nor the library call behind it allocates: the
    library keeps its derived dictionary in a fixed ~256 KB array that ships inside its device
    image and rebuilds it from ``dec`` on every call.  The array is shared, so do not let two of
    these calls overlap on one GPU, and make the first call on a device outside stream capture."""
    dev, height = _check_matrix(dec, w_comp, row_off, ter_minmax)
    _need(x, "x", torch.bfloat16, dev)
    _need(y, "y", torch.bfloat16, dev)
    if y.numel() != height:
        raise ValueError(f"y has {y.numel()} elements but row_off describes {height} rows")
    L = _lib.load()
    _lib.check(L.qmoe_sub1_matvec_noalloc(dec.data_ptr(), w_comp.data_ptr(), row_off.data_ptr(),
                                          ter_minmax.data_ptr(), x.data_ptr(), y.data_ptr(), height,
                                          x.numel(), w_comp.numel(), dev.index, _stream(dev)))


def sub1matmul(dec: torch.Tensor, w_comp: torch.Tensor, row_off: torch.Tensor,
               ter_minmax: torch.Tensor, x: torch.Tensor, y: torch.Tensor, flags: int = 0) -> None:
    """Batched form: ``x[t, width] -> y[t, height]``, codes decoded once per group of four tokens.
    ``flags``: ``FLAG_ACCUMULATE`` (``y +=``, else ``y =``), ``FLAG_RELU``.  Rows may be strided."""
    dev, height = _check_matrix(dec, w_comp, row_off, ter_minmax)
    for t, n in ((x, "x"), (y, "y")):
        if not (isinstance(t, torch.Tensor) and t.is_cuda and t.dtype == torch.bfloat16 and t.dim() == 2
                and t.stride(1) == 1 and t.device == dev):
            raise ValueError(f"{n} must be a 2-D bf16 CUDA tensor on {dev} with unit inner stride")
    if x.shape[0] != y.shape[0] or y.shape[1] != height:
        raise ValueError("x and y must have the same number of rows and y must have `height` columns")
    L = _lib.load()
    _lib.check(L.qmoe_sub1_matmul(dec.data_ptr(), w_comp.data_ptr(), row_off.data_ptr(),
                                  ter_minmax.data_ptr(), x.data_ptr(), y.data_ptr(), height, x.shape[1],
                                  w_comp.numel(), x.shape[0], x.stride(0) if x.shape[0] > 1 else x.shape[1],
                                  y.stride(0) if y.shape[0] > 1 else height, int(flags), dev.index,
                                  _stream(dev)))


def sub1decode(dec: torch.Tensor, w_comp: torch.Tensor, row_off: torch.Tensor, width: int,
               return_status: bool = False):
    """Ternary symbols ``uint8[height, width]`` of a compressed matrix (0, 1 = row min, 2 = row max);
    the GPU twin of decompress() (test.py:103-115).  With ``return_status`` also returns the number
    of rows whose codes do not cover exactly ``width`` weights (a host synchronisation)."""
    _need(dec, "dec", torch.int32)
    dev = dec.device
    track_dec(dec)
    _need(w_comp, "w_comp", (torch.int16, torch.uint16), dev)
    _need(row_off, "row_off", torch.int32, dev)
    height = row_off.numel() - 1
    sym = torch.empty((height, width), dtype=torch.uint8, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    L = _lib.load()
    _lib.check(L.qmoe_sub1_decode(dec.data_ptr(), w_comp.data_ptr(), row_off.data_ptr(), sym.data_ptr(),
                                  status.data_ptr(), height, int(width), w_comp.numel(), dev.index,
                                  _stream(dev)))
    if return_status:
        return sym, int(status.item())
    return sym


def sub1pack(trie: torch.Tensor, w_tern: torch.Tensor, row_off: torch.Tensor) -> torch.Tensor:
    """Greedy dictionary encoding of ``w_tern`` (int32[H, W], values 0/1/2).  As in the reference
    (sub1_cuda.cpp:47-54, sub1_cuda_kernel.cu:92-126) ``w_tern`` is clobbered, ``row_off``
    (int32[H+1]) receives the exclusive prefix sums, and a new int16 tensor with the code stream
    is returned.  Reading ``row_off[H]`` to size the output synchronises, as the reference does."""
    _need(trie, "trie", torch.int32)
    dev = trie.device
    if trie.numel() != (_lib.DICT_COUNT + 1) * 9:
        raise ValueError("trie must be int32[65537, 9]")
    _need(w_tern, "w_tern", torch.int32, dev)
    _need(row_off, "row_off", torch.int32, dev)
    if w_tern.dim() != 2 or row_off.numel() != w_tern.shape[0] + 1:
        raise ValueError("w_tern must be [H, W] and row_off must have H + 1 entries")
    height, width = w_tern.shape
    L = _lib.load()
    s = _stream(dev)
    _lib.check(L.qmoe_sub1_pack_prepare(trie.data_ptr(), w_tern.data_ptr(), row_off.data_ptr(), height, width,
                                        dev.index, s))
    n_codes = int(row_off[height].item())
    w_comp = torch.zeros(n_codes, dtype=torch.int16, device=dev)
    if n_codes:
        _lib.check(L.qmoe_sub1_pack_emit(w_tern.data_ptr(), row_off.data_ptr(), w_comp.data_ptr(), height,
                                         width, dev.index, s))
    return w_comp


def sub1pack_u8(trie: torch.Tensor, sym: torch.Tensor):
    """Batched encoder: ``sym`` uint8[M, H, W] (or [H, W]) -> (codes int16[total], row_off int32[M, H+1]
    relative to each matrix, mat_base int64[M] in codes, each a multiple of 8, n_codes int64[M]).
    One host synchronisation to size the output."""
    _need(trie, "trie", torch.int32)
    dev = trie.device
    _need(sym, "sym", torch.uint8, dev)
    if sym.dim() == 2:
        sym = sym.unsqueeze(0)
    m, height, width = sym.shape
    L = _lib.load()
    s = _stream(dev)
    tmp = torch.empty((m * height, width // 2), dtype=torch.int16, device=dev)
    row_len = torch.empty(m * height, dtype=torch.int32, device=dev)
    _lib.check(L.qmoe_sub1_pack_u8_count(trie.data_ptr(), sym.data_ptr(), tmp.data_ptr(), row_len.data_ptr(),
                                         m, height, width, dev.index, s))
    row_off = torch.zeros((m, height + 1), dtype=torch.int32, device=dev)
    row_off[:, 1:] = torch.cumsum(row_len.view(m, height), dim=1, dtype=torch.int32)
    n_codes = row_off[:, height].to(torch.int64)
    padded = (n_codes + 7) // 8 * 8
    mat_base = torch.cumsum(padded, 0) - padded
    total = int((mat_base[-1] + padded[-1]).item())
    codes = torch.zeros(total, dtype=torch.int16, device=dev)
    _lib.check(L.qmoe_sub1_pack_u8_gather(tmp.data_ptr(), row_off.data_ptr(), mat_base.data_ptr(),
                                          codes.data_ptr(), m, height, width, dev.index, s))
    return codes, row_off, mat_base, n_codes
