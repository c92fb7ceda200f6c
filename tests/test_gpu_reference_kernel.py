"""The new kernels against the REFERENCE's own CUDA kernels (built unmodified into oracle/_ref by
oracle/build_ref.py) on the same device tensors.  Skipped when that build is absent."""

import numpy as np
import pytest
import torch

from oracle import build_ref  # noqa: E402  (as a package member: putting oracle/ itself on sys.path would
                              # shadow the package with oracle/oracle.py in child processes of later tests)

from qmoe_b200 import sub1, sub1_cuda  # noqa: E402
from util import Matrix, randn_bf16, rel_err  # noqa: E402

pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(build_ref.built_path() is None, reason="oracle/_ref not built")]

REFERENCE_SHAPES = [(768, 3072), (3072, 768), (1024, 4096), (4096, 1024), (2080, 6144), (6144, 2080)]


@pytest.fixture(scope="module")
def ref():
    return build_ref.load()


@pytest.mark.parametrize("shape", REFERENCE_SHAPES)
def test_matvec_equals_reference_kernel(ref, shape):
    """The six shapes the reference kernel is instantiated for (sub1_cuda_kernel.cu:82-87)."""
    h, w = shape
    dev = torch.device("cuda", 0)
    dec = sub1.DEC(dev)
    m = Matrix(h, w, seed=1, matrix_id=100 + h, device=dev)
    x = randn_bf16(w, seed=3).to(dev)
    y0 = randn_bf16(h, seed=4).to(dev)
    theirs = y0.clone()
    torch.cuda.synchronize()
    ref.sub1matvec(dec, m.d_codes, m.d_row_off, m.d_minmax, x, theirs)   # legacy default stream
    torch.cuda.synchronize()
    ours = y0.clone()
    sub1_cuda.sub1matvec(dec, m.d_codes, m.d_row_off, m.d_minmax, x, ours)
    torch.cuda.synchronize()
    # both accumulate in fp32 (different summation order), round to bf16, then add in bf16
    assert rel_err(ours, theirs) <= 1e-2
    assert float((ours == theirs).float().mean()) > 0.9


@pytest.mark.parametrize("shape", [(64, 256), (3072, 768)])
def test_pack_equals_reference_kernel(ref, shape):
    h, w = shape
    dev = torch.device("cuda", 0)
    trie = sub1.TRIE(dev)
    rng = np.random.default_rng(5)
    sym = torch.from_numpy(rng.choice(3, size=(h, w), p=[.9, .05, .05]).astype(np.int32)).to(dev)
    a_tern, b_tern = sym.clone(), sym.clone()
    a_off = torch.zeros(h + 1, dtype=torch.int32, device=dev)
    b_off = torch.zeros(h + 1, dtype=torch.int32, device=dev)
    torch.cuda.synchronize()
    theirs = ref.sub1pack(trie, a_tern, a_off)
    torch.cuda.synchronize()
    ours = sub1_cuda.sub1pack(trie, b_tern, b_off)
    torch.cuda.synchronize()
    assert torch.equal(ours, theirs) and torch.equal(a_off, b_off)
    # same in-place side effect on w_tern: each row's codes at the head of the row
    n = (b_off[1:] - b_off[:-1]).cpu()
    for r in (0, h // 2, h - 1):
        assert torch.equal(a_tern[r, : int(n[r])], b_tern[r, : int(n[r])])
