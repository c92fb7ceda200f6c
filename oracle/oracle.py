"""ctypes front end of the CPU oracle (``sub1_oracle.c``).  TEST INFRASTRUCTURE ONLY.

Only the test-suite, the smoke check and the CPU-baseline leg of the benchmark import this module;
the GPU product path never does.  Parity status: pinned (see the header of ``sub1_oracle.c``).

Besides the C restatement this module carries a second, independent numpy decoder
(:func:`numpy_decode_matrix`) that follows the reference's table layout directly
(sub1.py:60-72, sub1_cuda_kernel.cu:153-154,188-189); the tests check the two against each other
and against the golden vectors produced by the reference's own Python.
"""
from __future__ import annotations

import ctypes
import os
import subprocess
from typing import Tuple

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SRC = os.path.join(_HERE, "sub1_oracle.c")
_OUT_DIR = os.path.join(_HERE, "_build")
_LIB = os.path.join(_OUT_DIR, "libsub1_oracle.so")

DICT_COUNT = 65536
TRIE_ROOT = 65536

# SHA-256 of the tables produced by the reference's own setup() (sub1.py:29-102).
DEC_SHA256 = "c09862c453fe122634070a475357ff81a679aff65829d84a56f806c02a54ed45"
TRIE_SHA256 = "fc77a88c6c9c32a0a884b2736ac78c25239a162817d133dc8457c8f0770a8b0b"


def build(force: bool = False) -> str:
    """Compile the C oracle with gcc (OpenMP) into ``oracle/_build``; returns the library path."""
    if not force and os.path.exists(_LIB) and os.path.getmtime(_LIB) >= os.path.getmtime(_SRC):
        return _LIB
    os.makedirs(_OUT_DIR, exist_ok=True)
    cmd = ["gcc", "-O3", "-march=x86-64-v2", "-fopenmp", "-shared", "-fPIC", "-std=c11",
           "-o", _LIB, _SRC, "-lm"]
    subprocess.run(cmd, check=True)
    return _LIB


_lib = None


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        path = _LIB if os.path.exists(_LIB) and os.path.getmtime(_LIB) >= os.path.getmtime(_SRC) else build()
        L = ctypes.CDLL(path)
        P = ctypes.c_void_p
        I = ctypes.c_int
        L.oracle_build_dictionary.argtypes = [P, P]
        L.oracle_build_dictionary.restype = I
        L.oracle_encode_row.argtypes = [P, P, I, P]
        L.oracle_encode_row.restype = I
        L.oracle_encode_matrix.argtypes = [P, P, I, I, P, P]
        L.oracle_encode_matrix.restype = ctypes.c_int64
        L.oracle_decode_row.argtypes = [P, P, I, I, P]
        L.oracle_decode_row.restype = I
        L.oracle_decode_matrix.argtypes = [P, P, P, I, I, P]
        L.oracle_decode_matrix.restype = I
        L.oracle_matvec.argtypes = [P, P, P, P, P, P, I, I, I]
        L.oracle_matvec.restype = I
        L.oracle_expert_ffn.argtypes = [P] * 10 + [I, I, I]
        L.oracle_expert_ffn.restype = I
        L.oracle_synth_ternary.argtypes = [P, ctypes.c_int64, ctypes.c_uint64, ctypes.c_uint64, ctypes.c_float]
        L.oracle_synth_ternary.restype = None
        L.oracle_num_threads.argtypes = []
        L.oracle_num_threads.restype = I
        L.oracle_set_num_threads.argtypes = [I]
        L.oracle_set_num_threads.restype = None
        _lib = L
    return _lib


def _p(a: np.ndarray) -> ctypes.c_void_p:
    return ctypes.c_void_p(a.ctypes.data)


_dict_cache = None


def build_dictionary() -> Tuple[np.ndarray, np.ndarray]:
    """(dec int32[131072], trie int32[65537, 9]) as the reference's setup() (sub1.py:29-102)."""
    global _dict_cache
    if _dict_cache is None:
        dec = np.zeros(2 * DICT_COUNT, dtype=np.int32)
        trie = np.zeros((DICT_COUNT + 1, 9), dtype=np.int32)
        rc = lib().oracle_build_dictionary(_p(dec), _p(trie))
        if rc != 0:
            raise RuntimeError(f"oracle_build_dictionary failed: {rc}")
        dec.setflags(write=False)
        trie.setflags(write=False)
        _dict_cache = (dec, trie)
    return _dict_cache


def encode_matrix(trie: np.ndarray, sym: np.ndarray) -> Tuple[np.ndarray, np.ndarray]:
    """Greedy longest-match encoding of a [H, W] uint8 symbol matrix (test.py:86-100,146-151).
    Returns (codes uint16[n], row_off int32[H+1])."""
    sym = np.ascontiguousarray(sym, dtype=np.uint8)
    h, w = sym.shape
    trie = np.ascontiguousarray(trie, dtype=np.int32)
    codes = np.zeros(h * ((w + 1) // 2) + 1, dtype=np.uint16)
    row_off = np.zeros(h + 1, dtype=np.int32)
    n = lib().oracle_encode_matrix(_p(trie), _p(sym), h, w, _p(codes), _p(row_off))
    return codes[:n].copy(), row_off


def decode_matrix(dec: np.ndarray, codes: np.ndarray, row_off: np.ndarray, height: int,
                  width: int) -> np.ndarray:
    """Decoded ternary symbols uint8[H, W] (test.py:103-115)."""
    dec = np.ascontiguousarray(dec, dtype=np.int32)
    codes = np.ascontiguousarray(codes).view(np.uint16)
    row_off = np.ascontiguousarray(row_off, dtype=np.int32)
    sym = np.zeros((height, width), dtype=np.uint8)
    rc = lib().oracle_decode_matrix(_p(dec), _p(codes), _p(row_off), height, width, _p(sym))
    if rc != 0:
        raise ValueError("code stream does not tile the rows exactly")
    return sym


def matvec(dec, codes, row_off, minmax_bits, x_bits, y_bits, height: int, width: int) -> None:
    """y[t, H] += bf16(W x[t]) with fp32 accumulation; all bf16 data passed as uint16 bit
    patterns; ``y_bits`` is updated in place (sub1_cuda_kernel.cu:197-200)."""
    x_bits = np.ascontiguousarray(x_bits, dtype=np.uint16).reshape(-1, width)
    tokens = x_bits.shape[0]
    assert y_bits.dtype == np.uint16 and y_bits.flags.c_contiguous and y_bits.size == tokens * height
    dec = np.ascontiguousarray(dec, dtype=np.int32)
    codes = np.ascontiguousarray(codes).view(np.uint16)
    row_off = np.ascontiguousarray(row_off, dtype=np.int32)
    minmax_bits = np.ascontiguousarray(minmax_bits, dtype=np.uint16)
    rc = lib().oracle_matvec(_p(dec), _p(codes), _p(row_off), _p(minmax_bits), _p(x_bits),
                             _p(y_bits), height, width, tokens)
    if rc != 0:
        raise ValueError("code stream does not tile the rows exactly")


def expert_ffn(dec, wi, wo, x_bits, d_model: int, d_ff: int) -> np.ndarray:
    """wo(ReLU(wi(x))) for one expert; ``wi``/``wo`` are (codes, row_off, minmax_bits) triples;
    ``x_bits`` is [t, d_model] bf16 bits.  Returns y bits [t, d_model]."""
    x_bits = np.ascontiguousarray(x_bits, dtype=np.uint16).reshape(-1, d_model)
    tokens = x_bits.shape[0]
    hidden = np.zeros((tokens, d_ff), dtype=np.uint16)
    y = np.zeros((tokens, d_model), dtype=np.uint16)
    dec = np.ascontiguousarray(dec, dtype=np.int32)
    a = [np.ascontiguousarray(wi[0]).view(np.uint16), np.ascontiguousarray(wi[1], dtype=np.int32),
         np.ascontiguousarray(wi[2], dtype=np.uint16),
         np.ascontiguousarray(wo[0]).view(np.uint16), np.ascontiguousarray(wo[1], dtype=np.int32),
         np.ascontiguousarray(wo[2], dtype=np.uint16)]
    rc = lib().oracle_expert_ffn(_p(dec), *[_p(t) for t in a], _p(x_bits), _p(hidden), _p(y),
                                 d_model, d_ff, tokens)
    if rc != 0:
        raise ValueError("code stream does not tile the rows exactly")
    return y


def synth_ternary(count: int, seed: int, first_index: int, p_zero: float) -> np.ndarray:
    """Seeded synthetic symbols uint8[count]; same stream as the GPU generator of the benchmark."""
    sym = np.empty(count, dtype=np.uint8)
    lib().oracle_synth_ternary(_p(sym), count, seed & ((1 << 64) - 1), first_index, p_zero)
    return sym


def num_threads() -> int:
    return int(lib().oracle_num_threads())


def use_all_cores() -> int:
    """Let the OpenMP loops use every core this process may run on, whatever OMP_NUM_THREADS says
    (multi-process launchers set it to 1); returns the thread count."""
    import os
    n = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    lib().oracle_set_num_threads(n)
    return num_threads()


# ---------------------------------------------------------------------------------------------
# bf16 bit helpers (numpy has no bf16): round-to-nearest-even like torch / CUDA.
# ---------------------------------------------------------------------------------------------
def f32_to_bf16_bits(a: np.ndarray) -> np.ndarray:
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32).astype(np.uint64)
    lsb = (u >> 16) & 1
    return ((u + 0x7FFF + lsb) >> 16).astype(np.uint16)


def bf16_bits_to_f32(b: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(b, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


# ---------------------------------------------------------------------------------------------
# Independent numpy decoder, straight from the table layout.
# ---------------------------------------------------------------------------------------------
def numpy_entry_digits(dec: np.ndarray) -> Tuple[np.ndarray, np.ndarray]:
    """For every code: (digits uint8[65536, 28], length-in-weights int32[65536]).  Decoded
    position t sits in word t // 14 at bit 4 + 2 * (t % 14) (sub1_cuda_kernel.cu:153-154,188-189);
    the low nibble of either word is the length in pairs (sub1.py:66,71)."""
    w = np.ascontiguousarray(dec, dtype=np.int32).view(np.uint32).reshape(-1, 2)
    t = np.arange(28)
    digits = ((w[:, t // 14] >> (4 + 2 * (t % 14)).astype(np.uint32)) & 3).astype(np.uint8)
    nweights = (2 * (w[:, 0] & 0xF)).astype(np.int32)
    return digits, nweights


def numpy_decode_matrix(dec, codes, row_off, height: int, width: int) -> np.ndarray:
    digits, nweights = numpy_entry_digits(dec)
    codes = np.ascontiguousarray(codes).view(np.uint16).astype(np.int64)
    out = np.zeros((height, width), dtype=np.uint8)
    for r in range(height):
        c = codes[row_off[r]:row_off[r + 1]]
        ln = nweights[c]
        flat = digits[c]                                   # [n, 28]
        keep = np.arange(28)[None, :] < ln[:, None]
        row = flat[keep]
        if row.size < width or row.size > width + 1:
            raise ValueError("row %d decodes to %d weights, expected %d" % (r, row.size, width))
        out[r] = row[:width]
    return out
