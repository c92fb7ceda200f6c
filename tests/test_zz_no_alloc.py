"""The allocation-free matvec entry point, called through the C ABI, against the regular one.

Why it exists: some hosts of this library may not allocate device memory at all (a framework that
owns the GPU's memory, a process whose budget is fully pooled, a thread that must not block in the
driver's allocator).  ``qmoe_sub1_matvec_noalloc`` keeps its scratch -- the derived dictionary --
in a fixed array inside the library instead of memory obtained with cudaMalloc.

This file is named to be collected last: it must pass alone in a fresh process and after every
other test has run (the shared array then holds whatever earlier calls left in it).
"""
import ctypes

import pytest
import torch

from qmoe_b200 import _lib, sub1
from util import Matrix, randn_bf16, rel_err

pytestmark = pytest.mark.gpu
TOL = 1e-2   # same bound as the other parity tests: max|err| / max|ref|


def _call(fn, dec, m, x, y):
    dev = dec.device
    _lib.check(fn(dec.data_ptr(), m.d_codes.data_ptr(), m.d_row_off.data_ptr(), m.d_minmax.data_ptr(),
                  x.data_ptr(), y.data_ptr(), m.height, m.width, m.d_codes.numel(), dev.index,
                  int(torch.cuda.current_stream(dev).cuda_stream)))


def test_noalloc_matvec_matches_regular_entry_point_twice():
    dev = torch.device("cuda", 0)
    lib = _lib.load()
    dec = sub1.DEC(dev)
    first = Matrix(3072, 768, seed=4, matrix_id=21, device=dev)
    second = Matrix(200, 1000, seed=4, matrix_id=22, device=dev)
    warm = torch.zeros(first.height, dtype=torch.bfloat16, device=dev)
    _call(lib.qmoe_sub1_matvec_noalloc, dec, first, randn_bf16(first.width).to(dev), warm)   # loads the kernels
    torch.cuda.synchronize()
    for round_, m in enumerate((first, second, first)):      # consecutive calls share the scratch array
        x = randn_bf16(m.width, seed=round_).to(dev)
        y0 = randn_bf16(m.height, seed=10 + round_).to(dev)
        want = y0.clone()
        _call(lib.qmoe_sub1_matvec, dec, m, x, want)
        torch.cuda.synchronize()
        got = y0.clone()
        torch.cuda.synchronize()
        reserved = torch.cuda.memory_reserved(dev)
        free_before = torch.cuda.mem_get_info(dev)[0]         # the driver's view: sees a cudaMalloc by anyone
        _call(lib.qmoe_sub1_matvec_noalloc, dec, m, x, got)
        _call(lib.qmoe_sub1_matvec_noalloc, dec, m, x, got)   # second call in a row: y += W x again
        torch.cuda.synchronize()
        assert torch.cuda.mem_get_info(dev)[0] == free_before, "device memory was allocated during the calls"
        _call(lib.qmoe_sub1_matvec, dec, m, x, want)
        torch.cuda.synchronize()
        assert rel_err(got, want) <= TOL
        assert rel_err(got.float().cpu() - y0.float().cpu(), 2 * m.oracle_matvec(x.cpu()).float().reshape(-1)) <= 2 * TOL
        assert torch.cuda.memory_reserved(dev) == reserved     # torch's pool was not touched either


def test_noalloc_matvec_rejects_sizes_beyond_its_maximum():
    dev = torch.device("cuda", 0)
    lib = _lib.load()
    dec = sub1.DEC(dev)
    m = Matrix(8, 64, seed=1, matrix_id=2, device=dev)
    x = randn_bf16(64).to(dev)
    y = torch.zeros(8, dtype=torch.bfloat16, device=dev)
    p = ctypes.c_void_p
    rc = lib.qmoe_sub1_matvec_noalloc(dec.data_ptr(), m.d_codes.data_ptr(), m.d_row_off.data_ptr(),
                                      m.d_minmax.data_ptr(), x.data_ptr(), y.data_ptr(), 8, _lib.MAX_WIDTH + 2,
                                      m.d_codes.numel(), 0, None)
    assert rc == _lib.ERR_UNSUPPORTED and b"maximum" in lib.qmoe_last_error()
    rc = lib.qmoe_sub1_matvec_noalloc(dec.data_ptr(), m.d_codes.data_ptr(), m.d_row_off.data_ptr(),
                                      m.d_minmax.data_ptr(), x.data_ptr(), y.data_ptr(), 8, 64, 1 << 31, 0, None)
    assert rc == _lib.ERR_UNSUPPORTED and b"maximum" in lib.qmoe_last_error()
    assert float(y.abs().max()) == 0.0
