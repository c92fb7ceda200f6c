"""The benchmark configurations at their full shapes (seeded synthetic stand-ins for the Switch
checkpoints): config 2 (switch-base-128 layer, 128 tokens), config 3 (switch-large-128 layer, 512
tokens, uniform and skewed router) and one switch-c-2048 expert.

Checks: (1) size-independent property over EVERY matrix of a layer -- encode on the GPU, decode on
the GPU, compare with the generated symbols bit for bit; (2) the GPU encoder's streams equal the CPU
oracle's for sampled experts; (3) layer outputs of tokens routed to sampled experts equal the
oracle's decode-then-matmul FFN times the router probability within 1e-2 (max|err| / max|ref|)."""
import numpy as np
import pytest
import torch

from oracle import oracle as O
from qmoe_b200 import sub1, sub1_cuda, synth
from util import rel_err

pytestmark = pytest.mark.gpu
SEED = 0
TOL = 1e-2


def _oracle_expert(d_model, d_ff, e):
    _, trie = O.build_dictionary()
    mats = []
    for which, (h, w) in enumerate(((d_ff, d_model), (d_model, d_ff))):
        m = 2 * e + which
        sym = O.synth_ternary(h * w, SEED, synth.matrix_first_index(m), 0.9).reshape(h, w)
        codes, row_off = O.encode_matrix(trie, sym)
        mm = synth.row_scales(h, SEED, m)
        mats.append((sym, codes, row_off, mm))
    return mats


def _oracle_ffn(mats, x_bf16, d_model, d_ff):
    dec, _ = O.build_dictionary()
    bits = lambda t: t.contiguous().view(torch.int16).numpy().view(np.uint16)  # noqa: E731
    wi, wo = mats
    y = O.expert_ffn(dec, (wi[1], wi[2], bits(wi[3])), (wo[1], wo[2], bits(wo[3])), bits(x_bf16), d_model, d_ff)
    return torch.from_numpy(y.view(np.int16)).view(torch.bfloat16)


def _check_layer(name, n_tokens, hot_experts=0, hot_fraction=0.0, sample=6):
    d_model, d_ff, n_exp = synth.SHAPES[name]
    dev = torch.device("cuda", 0)
    store = synth.build_store(d_model, d_ff, list(range(n_exp)), SEED, dev)
    dec = sub1.DEC(dev)

    # (1) every matrix of the layer: encode -> decode round trip, bit-exact
    for m in range(2 * n_exp):
        d = store.host_descs[m]
        w_comp, row_off, _ = store.matrix(m)
        got, bad = sub1_cuda.sub1decode(dec, w_comp.contiguous(), row_off.contiguous(), d.width, return_status=True)
        want = synth.ternary_cuda(d.height * d.width, SEED, synth.matrix_first_index(m), 0.9, dev)
        assert bad == 0
        assert torch.equal(got.reshape(-1), want), f"matrix {m} does not round-trip"

    hidden = synth.tokens(n_tokens, d_model, SEED + 1)
    logits = synth.router_logits(n_tokens, n_exp, SEED + 2, hot_experts=hot_experts, hot_fraction=hot_fraction)
    out, (_, index) = sub1.FasterMLP(None, store)(hidden.reshape(1, n_tokens, d_model).to(dev),
                                                  router_logits=logits.reshape(1, n_tokens, n_exp).to(dev))
    out = out.reshape(n_tokens, d_model).cpu()
    index = index.reshape(-1).cpu()
    probs = torch.softmax(logits, -1).bfloat16()
    assert torch.equal(index, probs.argmax(-1))

    counts = torch.bincount(index, minlength=n_exp)
    order = torch.argsort(counts, descending=True).tolist()
    chosen = order[:2] + [e for e in order if counts[e] == 1][:sample - 2]      # busiest + singles
    for e in chosen:
        mats = _oracle_expert(d_model, d_ff, e)
        # (2) GPU encoder == oracle encoder on this expert
        for which in (0, 1):
            w_comp, row_off, mm = store.matrix(2 * e + which)
            assert (w_comp.cpu().numpy().view(np.uint16) == mats[which][1]).all()
            assert (row_off.cpu().numpy() == mats[which][2]).all()
            assert torch.equal(mm.cpu(), mats[which][3])
        # (3) outputs of this expert's tokens
        tok = torch.nonzero(index == e).reshape(-1)
        ref = _oracle_ffn(mats, hidden[tok], d_model, d_ff).float() * probs[tok, e].float().unsqueeze(1)
        assert rel_err(out[tok], ref.bfloat16()) <= TOL, f"expert {e} with {len(tok)} tokens"
    return counts


def test_config2_switch_base_128_layer():
    counts = _check_layer("switch-base-128", 128)
    assert int(counts.max()) <= 8


def test_config3_switch_large_128_layer_uniform():
    _check_layer("switch-large-128", 512, sample=4)


@pytest.mark.parametrize("tile_min", [0, 16])
def test_config3_switch_large_128_layer_skewed_router(tile_min):
    """Hot experts (32+ tokens) through the per-row kernel (tile path off) and through the
    tensor-core tile path (threshold 16)."""
    from qmoe_b200 import _lib
    before = _lib.load().qmoe_moe_set_tile_min_tokens(tile_min)
    try:
        counts = _check_layer("switch-large-128", 512, hot_experts=8, hot_fraction=0.5, sample=4)
    finally:
        _lib.load().qmoe_moe_set_tile_min_tokens(before)
    assert int(counts.max()) >= 32          # the hot experts: many token groups per expert


def test_config4_one_switch_c_2048_expert():
    d_model, d_ff, _ = synth.SHAPES["switch-c-2048"]
    dev = torch.device("cuda", 0)
    e = 1234
    store = synth.build_store(d_model, d_ff, [e], SEED, dev)
    mats = _oracle_expert(d_model, d_ff, e)
    for which in (0, 1):
        w_comp, row_off, _ = store.matrix(which)
        assert (w_comp.cpu().numpy().view(np.uint16) == mats[which][1]).all()
        got = sub1_cuda.sub1decode(sub1.DEC(dev), w_comp.contiguous(), row_off.contiguous(), mats[which][0].shape[1])
        assert (got.cpu().numpy() == mats[which][0]).all()
    for n in (1, 3, 6):
        xs = synth.tokens(n, d_model, 7 + n)
        offsets = torch.tensor([0, n], dtype=torch.int32, device=dev)
        ys = sub1.grouped_ffn(store, offsets, xs.to(dev), n)
        assert rel_err(ys, _oracle_ffn(mats, xs, d_model, d_ff)) <= TOL
