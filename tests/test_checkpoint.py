"""Compressed-checkpoint directory: written in the reference's file / key layout (sub1.py:170-214)
and read back as per-rank expert slices.  CPU only."""
import os

import numpy as np
import torch

from qmoe_b200 import checkpoint as ck
from qmoe_b200.sub1 import Sub1Linear
from util import Expert


def _linear(m):
    lin = Sub1Linear(m.height, len(m.codes))
    lin.w_comp = torch.from_numpy(m.codes.view(np.int16).copy())
    lin.row_off = torch.from_numpy(m.row_off.copy())
    lin.ter_minmax = m.minmax.clone()
    return lin


def test_write_and_read_back_expert_slices(tmp_path):
    d_model, d_ff = 64, 96
    layers = ["encoder.block.1.layer.1.mlp", "decoder.block.1.layer.2.mlp"]
    experts = {(li, j): Expert(d_model, d_ff, seed=li + 1, expert_id=j) for li in range(2) for j in range(4)}
    w = ck.Sub1CheckpointWriter(str(tmp_path), config={"d_model": d_model, "d_ff": d_ff, "num_experts": 4},
                                nonexpert_state={"shared.weight": torch.randn(8, d_model)})
    for li, layer in enumerate(layers):
        for j in range(4):
            e = experts[(li, j)]
            w.add_packed(ck.expert_name(layer, j), _linear(e.wi), _linear(e.wo))
        w.save_experts()
    w.finalize()

    assert sorted(os.listdir(tmp_path)) == ["config.json", "exp00.pt", "exp01.pt", "noexp.pt", "sizes.pt"]
    assert ck.expert_files(str(tmp_path)) == ["exp00.pt", "exp01.pt"]
    sizes = ck.read_sizes(str(tmp_path))
    assert sizes["decoder.block.1.layer.2.mlp.experts.expert_3.wo"] == len(experts[(1, 3)].wo.codes)
    raw = torch.load(tmp_path / "exp00.pt")
    key = "encoder.block.1.layer.1.mlp.experts.expert_2.wi."
    assert {k[len(key):] for k in raw if k.startswith(key)} == {"w_comp", "row_off", "ter_minmax", "weight"}
    assert raw[key + "w_comp"].dtype == torch.int16 and raw[key + "row_off"].dtype == torch.int32
    assert raw[key + "ter_minmax"].dtype == torch.bfloat16 and not raw[key + "w_comp"].is_cuda
    assert torch.load(tmp_path / "noexp.pt")["shared.weight"].dtype == torch.bfloat16

    # an expert-parallel rank reads only its slice, in the order it asks for
    store, layer, idx = ck.load_expert_store(str(tmp_path), "exp01.pt", experts=[2, 3])
    assert layer == layers[1] and idx == [2, 3]
    assert (store.n_experts, store.d_model, store.d_ff) == (2, d_model, d_ff)
    for local, j in enumerate(idx):
        for which, m in enumerate((experts[(1, j)].wi, experts[(1, j)].wo)):
            w_comp, row_off, mm = store.matrix(2 * local + which)
            assert (w_comp.numpy().view(np.uint16) == m.codes).all()
            assert (row_off.numpy() == m.row_off).all() and torch.equal(mm, m.minmax)
            d = store.host_descs[2 * local + which]
            assert d.code_base % 8 == 0 and (d.height, d.width) == (m.height, m.width)

    lin = ck.load_linear(raw, "encoder.block.1.layer.1.mlp.experts.expert_2.wi")
    assert (lin.w_comp.numpy().view(np.uint16) == experts[(0, 2)].wi.codes).all()
    full, _, idx_all = ck.load_expert_store(str(tmp_path), "exp00.pt")
    assert idx_all == [0, 1, 2, 3] and full.n_experts == 4
