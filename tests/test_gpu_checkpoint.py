"""A compressed-checkpoint directory on the GPU: written with the GPU encoder through the
reference's ``add_expert`` / ``save_experts`` / ``finalize`` protocol (sub1.py:196-214), read back as
expert slices onto the device (what sub1.py:250,284-292 does for a whole model), and run through
the single-GPU layer and the single-rank expert-parallel layer against the CPU oracle."""
import numpy as np
import pytest
import torch

from oracle import oracle as O
from qmoe_b200 import checkpoint as ck
from qmoe_b200 import sub1, synth
from qmoe_b200.ep import ExpertParallelMLP
from util import rel_err

pytestmark = pytest.mark.gpu
TOL = 1e-2   # max|got - ref| / max|ref|


def _dense_ternary(h, w, seed, dev):
    """bf16 [h, w] with values {min_r, 0, max_r} per row: what Sub1Linear.make compresses."""
    sym = synth.ternary_numpy(h * w, seed, 0, 0.9).reshape(h, w)
    mm = synth.row_scales(h, seed, 1).float().reshape(h, 2)
    deq = torch.cat([torch.zeros(h, 1), mm], 1)
    dense = torch.gather(deq, 1, torch.from_numpy(sym.astype(np.int64))).bfloat16()
    return dense.to(dev), dense


def test_directory_written_on_the_gpu_loads_as_slices_and_runs(tmp_path):
    dev = torch.device("cuda", 0)
    d_model, d_ff, n_exp, n_tok = 128, 256, 4, 24
    layer = "decoder.block.1.layer.2.mlp"
    g = torch.Generator().manual_seed(3)
    router = (torch.randn(n_exp, d_model, generator=g) / d_model ** 0.5).bfloat16()
    w = ck.Sub1CheckpointWriter(str(tmp_path), config={"d_model": d_model, "d_ff": d_ff, "num_experts": n_exp,
                                                       "expert_capacity": 1024},
                                nonexpert_state={f"{layer}.router.classifier.weight": router})
    syms = {}
    for j in range(n_exp):
        wi, s_wi = _dense_ternary(d_ff, d_model, 10 + j, dev)
        wo, s_wo = _dense_ternary(d_model, d_ff, 20 + j, dev)
        syms[j] = (s_wi, s_wo)
        w.add_expert(ck.expert_name(layer, j), wi, wo)            # GPU encoder (Sub1Linear.make)
    w.save_experts()
    w.finalize()

    cfg = ck.read_config(str(tmp_path))
    assert cfg["torch_dtype"] == "bfloat16" and cfg["num_experts"] == n_exp
    noexp = ck.read_nonexpert(str(tmp_path), dev)
    router_dev = noexp[f"{layer}.router.classifier.weight"]
    assert router_dev.is_cuda and torch.equal(router_dev.cpu(), router)

    # two disjoint slices, as two expert-parallel ranks would read them, and the whole layer
    lo, _, idx_lo = ck.load_expert_store(str(tmp_path), "exp00.pt", experts=[0, 1], device=dev)
    hi, _, idx_hi = ck.load_expert_store(str(tmp_path), "exp00.pt", experts=[2, 3], device=dev)
    full, name, idx = ck.load_expert_store(str(tmp_path), "exp00.pt", device=dev)
    assert name == layer and idx == [0, 1, 2, 3] and idx_lo == [0, 1] and idx_hi == [2, 3]
    assert lo.codes.is_cuda and lo.il_codes is not None and (lo.n_experts, hi.n_experts) == (2, 2)

    # the streams read back decode to the weights that were compressed, bit for bit (compared as
    # values: make() marks the zeros of a row without negative entries as "row minimum" = 0)
    from qmoe_b200 import sub1_cuda
    for store, base in ((lo, 0), (hi, 2)):
        for local in range(2):
            for which in (0, 1):
                w_comp, row_off, mm = store.matrix(2 * local + which)
                width = d_model if which == 0 else d_ff
                got = sub1_cuda.sub1decode(sub1.DEC(dev), w_comp.contiguous(), row_off.contiguous(), width)
                deq = torch.cat([torch.zeros(got.shape[0], 1), mm.float().cpu().reshape(-1, 2)], 1)
                values = torch.gather(deq, 1, got.cpu().long()).bfloat16()
                assert torch.equal(values, syms[base + local][which])

    hidden = synth.tokens(n_tok, d_model, seed=5)
    layer_1gpu = sub1.FasterMLP(router_dev.float(), full, expert_capacity=cfg["expert_capacity"])
    out, (logits, index) = layer_1gpu(hidden.reshape(1, n_tok, d_model).to(dev))
    ep = ExpertParallelMLP(router_dev.float(), full, n_exp, expert_capacity=cfg["expert_capacity"])
    out_ep, _ = ep(hidden.to(dev), seq_len=n_tok)
    torch.cuda.synchronize()
    out = out.reshape(n_tok, d_model).cpu()
    assert torch.equal(out, out_ep.cpu()), "single-GPU layer and single-rank expert-parallel layer differ"

    # oracle: decode-then-matmul FFN of the chosen expert times the router probability
    dec, _ = O.build_dictionary()
    probs = torch.softmax(logits.reshape(n_tok, n_exp).float().cpu(), -1).bfloat16()
    index = index.reshape(-1).cpu()
    assert torch.equal(index, probs.argmax(-1))
    bits = lambda t: t.contiguous().cpu().view(torch.int16).numpy().view(np.uint16)  # noqa: E731
    ref = torch.empty_like(hidden)
    for t in range(n_tok):
        e = int(index[t])
        mats = []
        for which in (0, 1):
            w_comp, row_off, mm = full.matrix(2 * e + which)
            mats.append((bits(w_comp), row_off.cpu().numpy(), bits(mm)))
        y = O.expert_ffn(dec, mats[0], mats[1], bits(hidden[t:t + 1]), d_model, d_ff)
        ref[t] = (probs[t, e].float() * torch.from_numpy(y.view(np.int16)).view(torch.bfloat16)[0].float()).bfloat16()
    assert rel_err(out, ref) <= TOL
    # the two slices together give the full layer's expert outputs
    for store, base in ((lo, 0), (hi, 2)):
        tok = torch.nonzero((index >= base) & (index < base + 2)).reshape(-1)
        if len(tok) == 0:
            continue
        order = tok[torch.argsort(index[tok], stable=True)]
        counts = [int((index[order] == base + k).sum()) for k in range(2)]
        offsets = torch.tensor([0, counts[0], counts[0] + counts[1]], dtype=torch.int32, device=dev)
        ys = sub1.grouped_ffn(store, offsets, hidden[order].to(dev).contiguous(), len(order)).cpu()
        want = ref[order].float() / probs[order, index[order]].float().unsqueeze(1)
        assert rel_err(ys, want.bfloat16()) <= 2 * TOL
