"""Generates tests/golden/sub1_golden.npz by running the REFERENCE's own Python.

Run where the reference checkout is available:

    [QMOE_REFERENCE=/path/to/reference] python tests/golden/make_golden.py

Nothing of the reference is copied: its functions are loaded with ``ast`` from the files where they
lie (``setup`` from sub1.py:29-102; the module-level dictionary, ``greedy`` and ``decompress`` from
test.py:29-115, whose top-level ``import sub1_cuda`` and GPU script body cannot run here) and
executed unchanged on seeded inputs.  The outputs are the golden vectors the oracle and the CUDA
kernels are pinned against.
"""
import ast
import hashlib
import heapq
import os
import random
import sys

import numpy as np
import torch

_HERE = os.path.dirname(os.path.abspath(__file__))


def _reference_dir():
    """``$QMOE_REFERENCE``, else a directory named ``reference`` beside this repository."""
    env = os.environ.get("QMOE_REFERENCE")
    return env if env else os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(_HERE))), "reference")


REF = _reference_dir()
OUT = os.path.join(os.path.dirname(os.path.abspath(__file__)), "sub1_golden.npz")


def load_setup():
    tree = ast.parse(open(os.path.join(REF, "sub1.py")).read())
    fn = [n for n in tree.body if isinstance(n, ast.FunctionDef) and n.name == "setup"][0]
    ns = {"np": np, "torch": torch, "heapq": heapq}
    exec(compile(ast.Module([fn], []), "sub1.py", "exec"), ns)
    return ns["setup"]


def load_test_namespace():
    tree = ast.parse(open(os.path.join(REF, "test.py")).read())
    body = [n for n in tree.body
            if n.lineno < 129 and not (isinstance(n, ast.Import) and n.names[0].name == "sub1_cuda")]
    ns = {}
    exec(compile(ast.Module(body, []), "test.py", "exec"), ns)
    return ns


def main():
    dec, trie = load_setup()()
    dec = dec.numpy()
    trie = trie.numpy()
    ns = load_test_namespace()
    assert (ns["dec"].astype(np.int32) == dec).all(), "test.py and sub1.py dictionaries differ"

    out = {
        "dec_sha256": np.frombuffer(hashlib.sha256(dec.tobytes()).digest(), dtype=np.uint8),
        "trie_sha256": np.frombuffer(hashlib.sha256(trie.tobytes()).digest(), dtype=np.uint8),
        # spot samples of both tables
        "dec_sample_idx": np.array([0, 1, 2, 3, 24, 25, 1000, 1001, 65534 * 2, 65534 * 2 + 1, 131070, 131071]),
        "trie_sample_rows": np.array([65536, 0, 1, 13, 14, 326, 5000, 40000, 65535]),
    }
    out["dec_sample"] = dec[out["dec_sample_idx"]]
    out["trie_sample"] = trie[out["trie_sample_rows"]]
    lens = dec[0::2] & 0xF
    out["len_hist"] = np.bincount(lens, minlength=15)

    # Encoder / decoder cases: (name, height, width, P(0)).  Pair sequences are drawn like genseq()
    # (test.py:80-84) but from a seeded generator and at the stated sparsity.
    cases = [("tiny", 4, 16, 0.5), ("small", 8, 64, 0.9), ("wide", 3, 768, 0.9), ("dense", 5, 40, 0.2),
             ("zeros", 2, 64, 1.0), ("design", 6, 256, 0.885), ("odd", 3, 31, 0.8)]
    rng = np.random.default_rng(20231026)
    names = []
    for name, h, w, pz in cases:
        q = np.array([pz, (1 - pz) / 2, (1 - pz) / 2])
        sym = rng.choice(3, size=(h, w), p=q).astype(np.uint8)
        codes, row_off = [], [0]
        for r in range(h):
            # pair = 3 * second + first (sub1_cuda_kernel.cu:223-228); odd trailing weight alone
            seq = [int(sym[r, i]) + (3 * int(sym[r, i + 1]) if i + 1 < w else 0) for i in range(0, w, 2)]
            codes.extend(ns["greedy"](seq))
            row_off.append(len(codes))
        termin = -rng.uniform(0.01, 1.0, size=h).astype(np.float32)
        termax = +rng.uniform(0.01, 1.0, size=h).astype(np.float32)
        termin = torch.from_numpy(termin).bfloat16().float().numpy()
        termax = torch.from_numpy(termax).bfloat16().float().numpy()
        ns["termin"], ns["termax"], ns["D2"] = termin, termax, w
        wdense = ns["decompress"](codes, w).reshape(h, w)
        x = torch.from_numpy(rng.standard_normal(w).astype(np.float32)).bfloat16()
        # test.py:176,180 semantics: dense bf16 matmul of the decompressed matrix
        y_bf16 = torch.matmul(torch.from_numpy(wdense).bfloat16(), x.reshape(-1, 1)).reshape(-1)
        y_f32 = torch.matmul(torch.from_numpy(wdense).bfloat16().float(), x.float().reshape(-1, 1)).reshape(-1)
        names.append(name)
        out[name + "_sym"] = sym
        out[name + "_codes"] = np.array(codes, dtype=np.uint16)
        out[name + "_row_off"] = np.array(row_off, dtype=np.int32)
        out[name + "_termin"] = termin
        out[name + "_termax"] = termax
        out[name + "_wdense"] = wdense.astype(np.float32)
        out[name + "_x"] = x.float().numpy()
        out[name + "_y_bf16"] = y_bf16.float().numpy()
        out[name + "_y_f32"] = y_f32.numpy()
    out["cases"] = np.array(names)
    np.savez_compressed(OUT, **out)
    print("wrote", OUT, os.path.getsize(OUT), "bytes")


if __name__ == "__main__":
    main()
