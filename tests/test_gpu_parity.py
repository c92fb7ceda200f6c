"""GPU parity tests: the sm_100a kernels, called through the C ABI, against the CPU oracle.

Bars: decoded symbols and encoder output bit-exact; matvec / FFN outputs within 1e-2 of the oracle's
decode-then-matmul (fp32 accumulation, bf16 output) measured as max|err| / max|ref| per call."""
import numpy as np
import pytest
import torch

from oracle import oracle as O
from qmoe_b200 import _lib, sub1, sub1_cuda, synth
from util import Matrix, randn_bf16, rel_err

pytestmark = pytest.mark.gpu

REFERENCE_SHAPES = [(768, 3072), (3072, 768), (1024, 4096), (4096, 1024), (2080, 6144), (6144, 2080)]
TOL = 1e-2


@pytest.fixture(scope="module")
def dev():
    return torch.device("cuda", 0)


@pytest.fixture(scope="module")
def dec(dev):
    return sub1.DEC(dev)


def test_device_dictionary_matches_oracle(dev, dec, oracle_dict):
    assert (dec.cpu().numpy() == oracle_dict[0]).all()
    assert (sub1.TRIE(dev).cpu().numpy() == oracle_dict[1]).all()


@pytest.mark.parametrize("case", ["tiny", "small", "wide", "dense", "zeros", "design", "odd"])
def test_decode_golden_bit_exact(golden, dev, dec, case):
    sym = golden[case + "_sym"]
    h, w = sym.shape
    codes = torch.from_numpy(golden[case + "_codes"].view(np.int16)).to(dev)
    row_off = torch.from_numpy(golden[case + "_row_off"]).to(dev)
    got, bad = sub1_cuda.sub1decode(dec, codes, row_off, w, return_status=True)
    assert bad == 0
    assert (got.cpu().numpy() == sym).all()


@pytest.mark.parametrize("case", ["tiny", "small", "wide", "dense", "zeros", "design", "odd"])
def test_matvec_golden(golden, dev, dec, case):
    sym = golden[case + "_sym"]
    h, w = sym.shape
    codes = torch.from_numpy(golden[case + "_codes"].view(np.int16)).to(dev)
    row_off = torch.from_numpy(golden[case + "_row_off"]).to(dev)
    mm = torch.from_numpy(np.stack([golden[case + "_termin"], golden[case + "_termax"]], 1).reshape(-1))
    x = torch.from_numpy(golden[case + "_x"]).bfloat16().to(dev)
    y = torch.zeros(h, dtype=torch.bfloat16, device=dev)
    sub1_cuda.sub1matvec(dec, codes, row_off, mm.bfloat16().to(dev), x, y)
    ref = torch.from_numpy(golden[case + "_y_f32"])
    assert rel_err(y, ref) <= TOL


@pytest.mark.parametrize("shape", REFERENCE_SHAPES)
def test_reference_shapes_decode_and_matvec(dev, dec, shape):
    h, w = shape
    m = Matrix(h, w, seed=0, matrix_id=h, device=dev)
    got, bad = sub1_cuda.sub1decode(dec, m.d_codes, m.d_row_off, w, return_status=True)
    assert bad == 0
    assert torch.equal(got.cpu(), torch.from_numpy(m.sym))          # bit-exact decode
    x = randn_bf16(w, seed=1)
    y0 = randn_bf16(h, seed=2)
    y = y0.clone().to(dev)
    sub1_cuda.sub1matvec(dec, m.d_codes, m.d_row_off, m.d_minmax, x.to(dev), y)   # y += W x
    ref = m.oracle_matvec(x, y0).reshape(-1)
    assert rel_err(y, ref) <= TOL
    # dense fp32 check, independent of the oracle's decoder
    dense = torch.from_numpy(m.dense()) @ x.float()
    assert rel_err(y.float().cpu() - y0.float(), dense) <= 2 * TOL


@pytest.mark.parametrize("tokens", [1, 2, 3, 4, 5, 9])
@pytest.mark.parametrize("flags", [0, _lib.FLAG_RELU, _lib.FLAG_ACCUMULATE])
def test_matmul_batched(dev, dec, tokens, flags):
    h, w = 352, 512
    m = Matrix(h, w, seed=3, matrix_id=7, device=dev)
    x = randn_bf16(tokens, w, seed=tokens)
    y0 = randn_bf16(tokens, h, seed=100 + tokens)
    ybuf = torch.zeros(tokens, h + 8, dtype=torch.bfloat16, device=dev)   # strided rows
    y = ybuf[:, :h]
    y.copy_(y0)
    sub1_cuda.sub1matmul(dec, m.d_codes, m.d_row_off, m.d_minmax, x.to(dev), y, flags)
    ref = m.oracle_matvec(x, y0 if flags & _lib.FLAG_ACCUMULATE else None)
    if flags & _lib.FLAG_RELU:
        ref = torch.relu(ref)
    assert rel_err(y, ref) <= TOL
    assert float(ybuf[:, h:].abs().max()) == 0.0                           # nothing written past a row


def test_matvec_unaligned_stream_and_odd_height(dev, dec):
    h, w = 37, 130
    m = Matrix(h, w, seed=5, matrix_id=11, device=dev)
    pad = torch.zeros(m.d_codes.numel() + 3, dtype=torch.int16, device=dev)
    for shift in (1, 2, 3):
        pad[shift:shift + m.d_codes.numel()] = m.d_codes
        view = pad[shift:shift + m.d_codes.numel()]
        x = randn_bf16(w, seed=shift)
        y = torch.zeros(h, dtype=torch.bfloat16, device=dev)
        sub1_cuda.sub1matvec(dec, view, m.d_row_off, m.d_minmax, x.to(dev), y)
        assert rel_err(y, m.oracle_matvec(x).reshape(-1)) <= TOL
        assert torch.equal(sub1_cuda.sub1decode(dec, view, m.d_row_off, w).cpu(), torch.from_numpy(m.sym))


def test_rows_of_zeros_and_one_sided_rows(dev, dec):
    h, w = 64, 256
    rng = np.random.default_rng(3)
    sym = rng.choice(3, size=(h, w), p=[.9, .05, .05]).astype(np.uint8)
    sym[0] = 0                       # all-zero row
    sym[1][sym[1] == 1] = 0          # only max
    sym[2][sym[2] == 2] = 0          # only min
    sym[3] = 2                       # fully dense row
    mm = synth.row_scales(h, 0, 0)
    mm[2 * 1] = 0.0                  # min == 0 on the max-only row
    m = Matrix(h, w, sym=sym, minmax=mm, device=dev)
    assert torch.equal(sub1_cuda.sub1decode(dec, m.d_codes, m.d_row_off, w).cpu(), torch.from_numpy(sym))
    x = randn_bf16(2, w, seed=9)
    y = torch.empty(2, h, dtype=torch.bfloat16, device=dev)
    sub1_cuda.sub1matmul(dec, m.d_codes, m.d_row_off, m.d_minmax, x.to(dev), y)
    assert rel_err(y, m.oracle_matvec(x)) <= TOL
    assert float(y[:, 0].abs().max()) == 0.0


def test_corrupt_stream_is_reported_not_faulted(dev, dec):
    h, w = 16, 64
    m = Matrix(h, w, seed=1, matrix_id=3, device=dev)
    bad_codes = m.d_codes.clone()
    _, nweights = O.numpy_entry_digits(O.build_dictionary()[0])
    bad_codes[0] = 0 if nweights[m.codes[0]] != 2 else 13   # another length: row 0 no longer tiles
    _, bad = sub1_cuda.sub1decode(dec, bad_codes, m.d_row_off, w, return_status=True)
    assert bad >= 1
    bad_off = m.d_row_off.clone()
    bad_off[5] = 10 ** 6             # span outside the stream: clamped, counted, no out-of-bounds read
    _, bad = sub1_cuda.sub1decode(dec, m.d_codes, bad_off, w, return_status=True)
    assert bad >= 1
    y = torch.zeros(h, dtype=torch.bfloat16, device=dev)
    sub1_cuda.sub1matvec(dec, bad_codes, bad_off, m.d_minmax, randn_bf16(w).to(dev), y)
    torch.cuda.synchronize()


def test_nonconforming_table_uses_digit_path(dev, oracle_dict):
    """A table with an entry of four non-zeros cannot use the sparse form; results must still match
    a decode done straight from that table."""
    dec_np = oracle_dict[0].copy()
    digits, nweights = O.numpy_entry_digits(dec_np)
    code = int(np.where((nweights >= 8) & ((digits != 0).sum(1) == 3))[0][0])
    free = int(np.where(digits[code][:nweights[code]] == 0)[0][0])
    word, bit = free // 14, 4 + 2 * (free % 14)
    dec_np[2 * code + word] = np.int32(np.uint32(dec_np[2 * code + word]) | np.uint32(2 << bit))
    dec2 = torch.from_numpy(dec_np).to(dev)
    h, w = 8, int(nweights[code]) + 28
    codes = np.full((h, 2), code, dtype=np.uint16)
    zeros28 = int(np.where((nweights == 28) & ((digits != 0).sum(1) == 0))[0][0])
    codes[::2, 1] = zeros28          # a conforming all-zero entry of 28 weights after / before it
    codes[1::2, 0] = zeros28
    row_off = (np.arange(h + 1) * 2).astype(np.int32)
    want = O.numpy_decode_matrix(dec_np, codes.reshape(-1), row_off, h, w)
    d_codes = torch.from_numpy(codes.reshape(-1).view(np.int16)).to(dev)
    d_off = torch.from_numpy(row_off).to(dev)
    got, bad = sub1_cuda.sub1decode(dec2, d_codes, d_off, w, return_status=True)
    assert bad == 0 and (got.cpu().numpy() == want).all()
    mm = synth.row_scales(h, 1, 1)
    x = randn_bf16(w, seed=4)
    y = torch.zeros(h, dtype=torch.bfloat16, device=dev)
    sub1_cuda.sub1matvec(dec2, d_codes, d_off, mm.to(dev), x.to(dev), y)
    deq = np.concatenate([np.zeros((h, 1), np.float32), mm.float().numpy().reshape(-1, 2)], 1)
    dense = torch.from_numpy(np.take_along_axis(deq, want.astype(np.int64), 1)) @ x.float()
    assert rel_err(y, dense) <= TOL
    _lib.check(_lib.load().qmoe_sub1_release(0))


@pytest.mark.parametrize("shape", [(32, 64), (96, 768), (33, 130), (1, 2), (64, 31)])
def test_pack_matches_oracle_bit_exact(dev, oracle_dict, shape):
    h, w = shape
    rng = np.random.default_rng(h * 1000 + w)
    sym = rng.choice(3, size=(h, w), p=[.88, .06, .06]).astype(np.uint8)
    codes, row_off = O.encode_matrix(oracle_dict[1], sym)
    w_tern = torch.from_numpy(sym.astype(np.int32)).to(dev)
    d_off = torch.full((h + 1,), 123, dtype=torch.int32, device=dev)
    w_comp = sub1_cuda.sub1pack(sub1.TRIE(dev), w_tern, d_off)
    assert w_comp.dtype == torch.int16
    assert (w_comp.cpu().numpy().view(np.uint16) == codes).all()
    assert (d_off.cpu().numpy() == row_off).all()
    # the reference leaves each row's codes at the head of the row of w_tern
    head = w_tern.cpu().numpy()
    for r in (0, h - 1):
        n = row_off[r + 1] - row_off[r]
        assert (head[r, :n] == codes[row_off[r]:row_off[r + 1]]).all()


def test_pack_u8_batched_matches_oracle(dev, oracle_dict):
    m, h, w = 3, 48, 160
    rng = np.random.default_rng(11)
    sym = rng.choice(3, size=(m, h, w), p=[.9, .05, .05]).astype(np.uint8)
    codes, row_off, base, n_codes = sub1_cuda.sub1pack_u8(sub1.TRIE(dev), torch.from_numpy(sym).to(dev))
    codes = codes.cpu().numpy().view(np.uint16)
    for i in range(m):
        c, ro = O.encode_matrix(oracle_dict[1], sym[i])
        assert int(base[i]) % 8 == 0 and int(n_codes[i]) == len(c)
        assert (row_off[i].cpu().numpy() == ro).all()
        assert (codes[int(base[i]):int(base[i]) + len(c)] == c).all()


def test_synth_kernel_matches_numpy_twin(dev):
    for count, first in ((1000, 0), (4099, synth.matrix_first_index(9)), (5, 8)):
        got = synth.ternary_cuda(count, 42, first, 0.9, dev).cpu().numpy()
        assert (got == synth.ternary_numpy(count, 42, first, 0.9)).all()


def test_sub1linear_make_and_forward(dev):
    h, w = 96, 256
    m = Matrix(h, w, seed=2, matrix_id=5)
    dense = torch.from_numpy(m.dense()).bfloat16().to(dev)
    lin = sub1.Sub1Linear.make(dense)
    assert (lin.w_comp.cpu().numpy().view(np.uint16) == m.codes).all()
    assert (lin.row_off.cpu().numpy() == m.row_off).all()
    assert torch.equal(lin.ter_minmax.cpu(), m.minmax)
    x = randn_bf16(5, w, seed=8).to(dev)
    y = lin(x)
    ref = m.oracle_matvec(x.cpu())
    assert rel_err(y, ref) <= TOL
    assert rel_err(lin.forward_per_token(x), ref) <= TOL
    sd = {k: v.cpu() for k, v in lin.state_dict().items()}
    lin2 = sub1.Sub1Linear(h, sd["w_comp"].numel())
    lin2.load_state_dict(sd)
    assert torch.equal(lin2.to(dev)(x), y)
