"""Host-side checks that need no GPU: the C-ABI library loads and exports every symbol the header
declares, the native dictionary builder reproduces the reference tables, argument validation
rejects bad input before any CUDA call, and the synthetic generator's CPU twin is sane."""
import ctypes
import hashlib
import os
import re

import numpy as np
import pytest

from oracle import oracle as O
from qmoe_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "qmoe_sub1.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(qmoe_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    lib = _lib.load()
    names = _declared_symbols()
    assert len(names) >= 18
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/qmoe_sub1.h but not exported"
    # ... and the ctypes table covers exactly the header
    assert sorted(_lib.SIGNATURES) == names
    assert lib.qmoe_version() >= 100


def test_matrix_desc_layout():
    assert ctypes.sizeof(_lib.MatrixDesc) == 40
    assert _lib.MatrixDesc.height.offset == 32 and _lib.MatrixDesc.width.offset == 36


def test_native_dictionary_matches_reference_hashes(oracle_dict):
    from qmoe_b200 import sub1
    dec, trie = sub1.setup()
    assert dec.dtype.is_floating_point is False and tuple(trie.shape) == (65537, 9)
    assert hashlib.sha256(dec.numpy().tobytes()).hexdigest() == O.DEC_SHA256
    assert hashlib.sha256(trie.numpy().tobytes()).hexdigest() == O.TRIE_SHA256
    assert (dec.numpy() == oracle_dict[0]).all() and (trie.numpy() == oracle_dict[1]).all()


def test_argument_validation_without_gpu():
    lib = _lib.load()
    assert lib.qmoe_sub1_build_dictionary(None, None) == _lib.ERR_INVALID_ARG
    assert b"null" in lib.qmoe_last_error()
    # null device pointers / bad shapes are rejected before any CUDA call
    assert lib.qmoe_sub1_matvec(None, None, None, None, None, None, 8, 8, 0, 0, None) == _lib.ERR_INVALID_ARG
    fake = ctypes.c_void_p(256)
    assert lib.qmoe_sub1_matvec(fake, fake, fake, fake, fake, fake, 0, 8, 1, 0, None) == _lib.ERR_INVALID_ARG
    assert lib.qmoe_sub1_matvec(fake, fake, fake, fake, fake, fake, 8, 1 << 20, 1, 0, None) == _lib.ERR_UNSUPPORTED
    assert lib.qmoe_sub1_matvec(fake, ctypes.c_void_p(257), fake, fake, fake, fake, 8, 8, 1, 0, None) \
        == _lib.ERR_INVALID_ARG
    assert lib.qmoe_moe_rank(fake, fake, fake, fake, 4, 2, 3, 1, 0, None) == _lib.ERR_INVALID_ARG
    assert lib.qmoe_moe_work_bytes(4, 16, 768, 3072) > 64
    with pytest.raises(_lib.QmoeError):
        _lib.check(lib.qmoe_sub1_pack_prepare(None, None, None, 1, 2, 0, None))


def test_interleaved_store_arguments_are_validated_without_gpu():
    lib = _lib.load()
    fake = ctypes.c_void_p(256)
    # heights must be multiples of 32 and rows consecutive: checked on the host copy of the descriptors
    descs = (_lib.MatrixDesc * 2)(_lib.MatrixDesc(0, 10, 0, 0, 64, 32), _lib.MatrixDesc(16, 10, 65, 64, 33, 64))
    rc = lib.qmoe_moe_interleave_count(fake, fake, ctypes.addressof(descs), 2, fake, 0, None)
    assert rc == _lib.ERR_UNSUPPORTED and b"multiples of 32" in lib.qmoe_last_error()
    descs = (_lib.MatrixDesc * 2)(_lib.MatrixDesc(0, 10, 0, 0, 64, 32), _lib.MatrixDesc(16, 10, 65, 96, 32, 64))
    assert lib.qmoe_moe_interleave_count(fake, fake, ctypes.addressof(descs), 2, fake, 0, None) == _lib.ERR_UNSUPPORTED
    assert lib.qmoe_moe_interleave_count(None, fake, ctypes.addressof(descs), 2, fake, 0, None) == _lib.ERR_INVALID_ARG
    assert lib.qmoe_moe_interleave_emit(fake, fake, fake, 2, fake, None, ctypes.c_void_p(8), 0, None) \
        == _lib.ERR_INVALID_ARG                                   # copy not 16-byte aligned
    # grouped FFN over an interleaved store: null store, null member, widths that are not multiples of 32
    args = (fake, None, fake, fake, fake)
    tail = (fake, fake, fake, fake, fake, 4, 8)
    assert lib.qmoe_moe_grouped_ffn_interleaved(*args, None, *tail, 64, 96, 0, None) == _lib.ERR_INVALID_ARG
    store = _lib.InterleavedStore(256, 256, 256, None, None)
    assert lib.qmoe_moe_grouped_ffn_interleaved(*args, ctypes.addressof(store), *tail, 64, 96, 0, None) \
        == _lib.ERR_INVALID_ARG
    store = _lib.InterleavedStore(256, 256, 256, 256, None)
    assert lib.qmoe_moe_grouped_ffn_interleaved(*args, ctypes.addressof(store), *tail, 64, 100, 0, None) \
        == _lib.ERR_UNSUPPORTED
    assert lib.qmoe_decode_attention(fake, fake, fake, fake, fake, 4, 512, 64, 0, None) == _lib.ERR_UNSUPPORTED
    assert lib.qmoe_rms_norm(None, fake, fake, 1, 8, 1e-6, 0, None) == _lib.ERR_INVALID_ARG
    assert lib.qmoe_sub1_remap_tables(None, None, fake, fake, 0, None) == _lib.ERR_INVALID_ARG


def test_cpu_tensors_are_rejected():
    import torch
    from qmoe_b200 import sub1_cuda
    dec = torch.zeros(131072, dtype=torch.int32)
    with pytest.raises(RuntimeError):
        sub1_cuda.sub1matvec(dec, torch.zeros(4, dtype=torch.int16), torch.zeros(3, dtype=torch.int32),
                             torch.zeros(4, dtype=torch.bfloat16), torch.zeros(8, dtype=torch.bfloat16),
                             torch.zeros(2, dtype=torch.bfloat16))


def test_sub1linear_buffers_match_reference_keys():
    from qmoe_b200.sub1 import Sub1Linear
    lin = Sub1Linear(6, 17)
    sd = lin.state_dict()
    assert list(sd) == ["w_comp", "row_off", "ter_minmax", "weight"]
    assert sd["w_comp"].dtype.is_signed and sd["w_comp"].numel() == 17
    assert sd["row_off"].numel() == 7 and sd["ter_minmax"].numel() == 12 and sd["weight"].numel() == 0


def test_synthetic_symbols_distribution_and_determinism():
    from qmoe_b200 import synth
    a = synth.ternary_numpy(1 << 18, seed=0, first_index=synth.matrix_first_index(5), p_zero=0.9)
    b = synth.ternary_numpy(1 << 18, seed=0, first_index=synth.matrix_first_index(5), p_zero=0.9)
    assert (a == b).all()
    frac = np.bincount(a, minlength=3) / a.size
    assert abs(frac[0] - 0.9) < 5e-3 and abs(frac[1] - 0.05) < 3e-3 and abs(frac[2] - 0.05) < 3e-3
    # a window of the stream equals the same indices generated on their own
    c = synth.ternary_numpy(64, seed=0, first_index=synth.matrix_first_index(5) + 1024, p_zero=0.9)
    assert (c == a[1024:1088]).all()
    assert (synth.ternary_numpy(4096, 1, 0, 0.9) != synth.ternary_numpy(4096, 2, 0, 0.9)).any()
