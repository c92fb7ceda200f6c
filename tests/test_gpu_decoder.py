"""The decoder stack used for end-to-end generation timing: its MoE blocks against a dense torch
re-statement built from the decoded experts, and CUDA-graph decoding against eager decoding."""
import pytest
import torch
import torch.nn.functional as F

from qmoe_b200 import sub1, sub1_cuda
from qmoe_b200.decoder import SwitchDecoderLM, _rms_norm

pytestmark = pytest.mark.gpu


def _dense_expert(store, m, dev):
    d = store.host_descs[m]
    w_comp, row_off, mm = store.matrix(m)
    sym = sub1_cuda.sub1decode(sub1.DEC(dev), w_comp.contiguous(), row_off.contiguous(), d.width).long()
    deq = torch.stack([torch.zeros(d.height, device=dev), mm[0::2].float(), mm[1::2].float()], 1)
    return torch.gather(deq, 1, sym)                       # fp32 [H, W] of {0, min_r, max_r}


def _reference_forward(model, ids):
    """Same stack in plain torch; MoE = decode-then-matmul with fp32 accumulation, bf16 between."""
    dev = model.dev
    n = ids.shape[0]
    x = model.embed[ids]
    causal = torch.tril(torch.ones(n, n, dtype=torch.bool, device=dev))
    for b in model.blocks:
        hn = _rms_norm(x, b["ln1"])
        qkv = (hn @ b["wqkv"].t()).view(n, 3, model.h, model.hd)
        q, k, v = (qkv[:, j].transpose(0, 1).unsqueeze(0) for j in range(3))
        att = F.scaled_dot_product_attention(q, k, v, attn_mask=causal[None, None])
        x = x + att[0].transpose(0, 1).reshape(n, -1) @ b["wo"].t()
        hm = _rms_norm(x, b["ln2"]).contiguous()
        moe = b["moe"]
        probs = torch.softmax(hm.float() @ moe.router.w32.t(), -1).bfloat16()
        choice = probs.argmax(-1)
        y = torch.empty_like(hm)
        for t in range(n):
            e = int(choice[t])
            wi, wo = _dense_expert(moe.store, 2 * e, dev), _dense_expert(moe.store, 2 * e + 1, dev)
            hid = torch.relu((wi @ hm[t].float()).bfloat16()).float()
            y[t] = (probs[t, e].float() * (wo @ hid).bfloat16().float()).bfloat16()
        x = x + y
    return (_rms_norm(x, model.final_norm) @ model.lm_head.t()).float()


def test_decoder_blocks_match_dense_reference_and_graph_decoding():
    dev = torch.device("cuda", 0)
    model = SwitchDecoderLM(d_model=128, d_ff=256, n_experts=8, n_layers=2, n_heads=4, vocab=512,
                            max_len=32, device=dev, seed=3, drop_reference_layout=False)
    g = torch.Generator().manual_seed(1)
    ids = torch.randint(0, 512, (12,), generator=g).to(dev)
    logits = model.forward(ids, torch.arange(12, device=dev))
    ref = _reference_forward(model, ids)
    err = float((logits - ref).abs().max() / ref.abs().max())
    assert err <= 2e-2, err                                  # two blocks of bf16 arithmetic
    eager = model.generate(ids, 10, use_graph=False)
    graphed = model.generate(ids, 10, use_graph=True)
    assert model.last_generate_used_graph
    assert torch.equal(eager, graphed)
    assert eager.shape == (10,) and int(eager.max()) < 512
    # the same model holding only the interleaved copies of its experts (how the benchmark runs it)
    for b in model.blocks:
        b["moe"].store.drop_reference_layout()
    assert torch.equal(model.forward(ids, torch.arange(12, device=dev)), logits)
    assert torch.equal(model.generate(ids, 10, use_graph=True), eager)
