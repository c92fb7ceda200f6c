"""The CPU oracle against the golden vectors produced by the reference's own Python
(tests/golden/make_golden.py) and, when the reference checkout is present, against the reference
functions themselves."""
import hashlib
import os

import numpy as np
import pytest

from oracle import oracle as O


def test_dictionary_hashes(golden, oracle_dict):
    dec, trie = oracle_dict
    assert hashlib.sha256(dec.tobytes()).hexdigest() == O.DEC_SHA256
    assert hashlib.sha256(trie.tobytes()).hexdigest() == O.TRIE_SHA256
    assert bytes(golden["dec_sha256"]).hex() == O.DEC_SHA256
    assert bytes(golden["trie_sha256"]).hex() == O.TRIE_SHA256


def test_dictionary_samples(golden, oracle_dict):
    dec, trie = oracle_dict
    assert (dec[golden["dec_sample_idx"]] == golden["dec_sample"]).all()
    assert (trie[golden["trie_sample_rows"]] == golden["trie_sample"]).all()
    # known answers recorded from the reference's setup()
    assert dec[:4].tolist() == [1, 1, 2, 2]
    assert dec[24:26].tolist() == [0x11, 0x1]
    assert dec[-2:].tolist() == [0x0102000D, 0x20D]
    assert trie[65536].tolist() == [0, 12, 13, 14, 326, 327, 15, 328, 329]
    lens = dec[0::2] & 0xF
    assert np.bincount(lens, minlength=15).tolist() == golden["len_hist"].tolist()
    assert np.bincount(lens, minlength=15)[1:].tolist() == [9, 65, 233, 577, 1161, 2049, 3305, 4993, 7177,
                                                            9921, 13289, 17345, 3843, 1569]


def test_entries_have_at_most_three_nonzeros(oracle_dict):
    digits, nweights = O.numpy_entry_digits(oracle_dict[0])
    assert (digits != 3).all()
    assert ((digits != 0).sum(1) <= 3).all()
    # digits past the entry's length are zero
    assert (digits * (np.arange(28)[None, :] >= nweights[:, None])).sum() == 0


@pytest.mark.parametrize("case", ["tiny", "small", "wide", "dense", "zeros", "design", "odd"])
def test_encode_decode_matches_reference(golden, oracle_dict, case):
    dec, trie = oracle_dict
    sym = golden[case + "_sym"]
    h, w = sym.shape
    codes, row_off = O.encode_matrix(trie, sym)
    assert codes.tolist() == golden[case + "_codes"].tolist()
    assert row_off.tolist() == golden[case + "_row_off"].tolist()
    back = O.decode_matrix(dec, golden[case + "_codes"], golden[case + "_row_off"], h, w)
    assert (back == sym).all()
    assert (O.numpy_decode_matrix(dec, codes, row_off, h, w) == sym).all()
    # reference decompress(): symbols mapped to {0, min_r, max_r}
    deq = np.stack([np.zeros(h, np.float32), golden[case + "_termin"], golden[case + "_termax"]], 1)
    assert (np.take_along_axis(deq, sym.astype(np.int64), 1) == golden[case + "_wdense"]).all()


@pytest.mark.parametrize("case", ["tiny", "small", "wide", "dense", "zeros", "design", "odd"])
def test_matvec_matches_reference_dense_matmul(golden, oracle_dict, case):
    dec, _ = oracle_dict
    sym = golden[case + "_sym"]
    h, w = sym.shape
    minmax = O.f32_to_bf16_bits(np.stack([golden[case + "_termin"], golden[case + "_termax"]], 1).reshape(-1))
    x = O.f32_to_bf16_bits(golden[case + "_x"])
    y = np.zeros(h, dtype=np.uint16)
    O.matvec(dec, golden[case + "_codes"], golden[case + "_row_off"], minmax, x, y, h, w)
    got = O.bf16_bits_to_f32(y)
    ref = golden[case + "_y_f32"]          # fp32-accumulated dense matmul of the decompressed matrix
    scale = max(np.abs(ref).max(), 1e-6)
    # tolerance: max error relative to max|y| <= 1e-2 (bf16 output rounding is 2^-9 relative)
    assert np.abs(got - ref).max() / scale <= 1e-2
    assert np.abs(got - golden[case + "_y_bf16"]).max() / scale <= 2e-2
    # accumulate semantics: a second call doubles the result up to bf16 rounding
    O.matvec(dec, golden[case + "_codes"], golden[case + "_row_off"], minmax, x, y, h, w)
    assert np.abs(O.bf16_bits_to_f32(y) - 2 * ref).max() / scale <= 2e-2


def test_bad_stream_is_rejected(oracle_dict):
    dec, trie = oracle_dict
    sym = np.zeros((2, 32), dtype=np.uint8)
    codes, row_off = O.encode_matrix(trie, sym)
    with pytest.raises(ValueError):
        O.decode_matrix(dec, codes, row_off, 2, 34)


def test_round_trip_reference_shapes(oracle_dict):
    dec, trie = oracle_dict
    rng = np.random.default_rng(0)
    for h, w in [(3072, 768), (768, 3072)]:
        sym = rng.choice(3, size=(h, w), p=[.9, .05, .05]).astype(np.uint8)
        codes, row_off = O.encode_matrix(trie, sym)
        assert (O.decode_matrix(dec, codes, row_off, h, w) == sym).all()
        bits = 16 * len(codes) / (h * w)
        assert 0.68 < bits < 0.70           # ~0.69 bit/weight at P(0)=0.90


def _make_golden_module():
    import importlib.util
    spec = importlib.util.spec_from_file_location(
        "make_golden", os.path.join(os.path.dirname(__file__), "golden", "make_golden.py"))
    mg = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mg)
    return mg


def test_against_live_reference(oracle_dict):
    """Runs the reference's greedy()/decompress() (loaded with ast, executed unchanged) next to the
    oracle on fresh random rows.  Needs the reference checkout ($QMOE_REFERENCE, or a directory named
    ``reference`` beside the repository); skipped where it is absent."""
    mg = _make_golden_module()
    if not os.path.exists(os.path.join(mg.REF, "test.py")):
        pytest.skip("reference checkout absent (set QMOE_REFERENCE)")
    ns = mg.load_test_namespace()
    dec, trie = oracle_dict
    assert (ns["dec"].astype(np.int32) == dec).all()
    rng = np.random.default_rng(7)
    for w in (2, 30, 128, 770):
        sym = rng.choice(3, size=(1, w), p=[.85, .1, .05]).astype(np.uint8)
        seq = [int(sym[0, i]) + 3 * int(sym[0, i + 1]) for i in range(0, w, 2)]
        ref_codes = ns["greedy"](seq)
        codes, _ = O.encode_matrix(trie, sym)
        assert codes.tolist() == ref_codes
        ns["termin"], ns["termax"], ns["D2"] = [-1.0], [2.0], w
        dense = ns["decompress"](ref_codes, w)
        assert (np.array([0, -1.0, 2.0], np.float32)[sym[0]] == dense).all()
