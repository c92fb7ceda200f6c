"""``sub1_cuda.install()``: the documented way to let unmodified reference code ``import sub1_cuda``.

Without a GPU: after install() the name resolves to this package's module with the reference's two
callables (sub1_cuda.cpp:56-59), and -- where the reference checkout is present -- the reference's
own ``Sub1Linear`` class (sub1.py:114-166, loaded with ``ast`` and executed unchanged) builds on top
of it with the same buffers, dtypes and state-dict keys as :class:`qmoe_b200.sub1.Sub1Linear`.
With a GPU and the checkout: that class's own ``make`` and ``forward`` run on the new kernels and
are compared with the oracle.  With a GPU alone: the reference's call protocol (zero ``y``, one
``sub1matvec`` per token, sub1.py:132-143) through the installed name.
"""
import ast
import importlib
import os
import sys

import numpy as np
import pytest
import torch

from qmoe_b200 import sub1, sub1_cuda
from util import Matrix, randn_bf16, rel_err

TOL = 1e-2


def _reference_sub1_py():
    here = os.path.dirname(os.path.abspath(__file__))
    env = os.environ.get("QMOE_REFERENCE")
    ref = env if env else os.path.join(os.path.dirname(os.path.dirname(here)), "reference")
    path = os.path.join(ref, "sub1.py")
    return path if os.path.exists(path) else None


def _reference_sub1linear(dec_of, trie):
    """The reference's Sub1Linear class object, its module globals DEC / TRIE supplied by us."""
    path = _reference_sub1_py()
    if path is None:
        pytest.skip("reference checkout absent (set QMOE_REFERENCE)")
    tree = ast.parse(open(path).read())
    cls = [n for n in tree.body if isinstance(n, ast.ClassDef) and n.name == "Sub1Linear"][0]
    sub1_cuda.install()
    ns = {"torch": torch, "nn": torch.nn, "sub1_cuda": importlib.import_module("sub1_cuda"),
          "DEC": dec_of, "TRIE": trie}
    exec(compile(ast.Module([cls], []), "sub1.py", "exec"), ns)
    return ns["Sub1Linear"]


def test_install_registers_the_reference_module_name():
    sub1_cuda.install()
    mod = importlib.import_module("sub1_cuda")
    assert mod is sys.modules["qmoe_b200.sub1_cuda"]
    assert callable(mod.sub1matvec) and callable(mod.sub1pack)


def test_reference_sub1linear_has_our_buffers():
    ref_cls = _reference_sub1linear({}, None)
    theirs, ours = ref_cls(96, 1000), sub1.Sub1Linear(96, 1000)
    sd_t, sd_o = theirs.state_dict(), ours.state_dict()
    assert list(sd_t) == list(sd_o)
    for k in sd_t:
        assert sd_t[k].dtype == sd_o[k].dtype and sd_t[k].shape == sd_o[k].shape, k


@pytest.mark.gpu
def test_reference_call_protocol_through_the_installed_name():
    dev = torch.device("cuda", 0)
    sub1_cuda.install()
    import sub1_cuda as installed                       # what `import sub1_cuda` in reference code gets
    m = Matrix(768, 3072, seed=2, matrix_id=5, device=dev)
    x = randn_bf16(3, m.width, seed=1).to(dev)
    y = torch.zeros((3, m.height), dtype=torch.bfloat16, device=dev)    # sub1.py:133-135
    dec = sub1.DEC(dev)
    for i in range(3):                                                   # sub1.py:139-142
        installed.sub1matvec(dec, m.d_codes, m.d_row_off, m.d_minmax, x[i], y[i])
    assert rel_err(y, m.oracle_matvec(x.cpu())) <= TOL


@pytest.mark.gpu
def test_reference_sub1linear_make_and_forward_on_the_new_kernels():
    dev = torch.device("cuda", 0)
    ref_cls = _reference_sub1linear({dev.index: sub1.DEC(dev)}, sub1.TRIE(dev))
    m = Matrix(768, 3072, seed=3, matrix_id=9)
    dense = torch.from_numpy(m.dense()).bfloat16().to(dev)
    lin = ref_cls.make(dense)                            # the reference's make() -> our sub1pack
    assert (lin.w_comp.cpu().numpy().view(np.uint16) == m.codes).all()
    assert (lin.row_off.cpu().numpy() == m.row_off).all()
    x = randn_bf16(2, m.width, seed=4).to(dev)
    y = lin(x)                                           # the reference's forward() -> our sub1matvec
    assert rel_err(y, m.oracle_matvec(x.cpu())) <= TOL
