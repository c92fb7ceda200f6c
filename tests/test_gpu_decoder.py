"""The decoder stack used for end-to-end generation timing: its MoE blocks against a dense torch
re-statement built from the decoded experts, and CUDA-graph decoding against eager decoding."""
import pytest
import torch
import torch.nn.functional as F

from qmoe_b200 import sub1, sub1_cuda
from qmoe_b200.decoder import SwitchDecoderLM, _rms_norm

pytestmark = pytest.mark.gpu


def _dense_expert(store, m, dev):
    """Dense weights of one matrix, decoded with this package's own ``sub1decode``.  That is sound
    here only because the decoder is pinned elsewhere, bit for bit against the CPU oracle and the
    reference's golden vectors (test_gpu_parity.py, test_gpu_configs.py); this file checks the stack
    around the experts, not the decoding."""
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
    # single-token step through the fused kernels (RMS norm, attention with cache update, combine +
    # residual) against the batched path: token 11 after a prefill of tokens 0..10
    model.forward(ids[:11], torch.arange(11, device=dev))
    one = model.forward(ids[11:12], torch.full((1,), 11, dtype=torch.int64, device=dev))
    assert float((one[0] - logits[11]).abs().max() / logits[11].abs().max()) <= 2e-2
    model.fused_decode = False
    unfused = model.forward(ids[11:12], torch.full((1,), 11, dtype=torch.int64, device=dev))
    model.fused_decode = True
    assert float((one - unfused).abs().max() / unfused.abs().max()) <= 2e-2
    eager = model.generate(ids, 10, use_graph=False)
    graphed = model.generate(ids, 10, use_graph=True)
    assert model.last_generate_used_graph
    assert torch.equal(eager, graphed)
    assert eager.shape == (10,) and int(eager.max()) < 512
    # teacher-forced input (what the benchmark feeds): eager and graph replay agree, the forced ids
    # are what the steps consume, and the trace counts one expert per block and decode step
    forced = torch.randint(0, 512, (9,), generator=g)
    f_eager = model.generate(ids, 10, use_graph=False, forced=forced)
    assert torch.equal(model.generate(ids, 10, use_graph=True, forced=forced), f_eager)
    assert torch.equal(f_eager[:1], eager[:1]) and not torch.equal(f_eager, eager)
    model.trace_experts(True)
    assert torch.equal(model.generate(ids, 10, use_graph=False, forced=forced), f_eager)
    trace = model.expert_trace()
    model.trace_experts(False)
    assert trace.shape == (2, 8) and trace.sum(1).tolist() == [9, 9]
    # forced routing: every step goes where the schedule says, eager and graph replay agree
    sched = torch.randint(0, 8, (9, 2), generator=g)
    model.set_forced_routing(sched)
    model.trace_experts(True)
    r_eager = model.generate(ids, 10, use_graph=False, forced=forced)
    want = torch.stack([torch.bincount(sched[:, i], minlength=8) for i in range(2)])
    assert torch.equal(model.expert_trace().long(), want)
    model.trace_experts(False)
    assert torch.equal(model.generate(ids, 10, use_graph=True, forced=forced), r_eager)
    model.set_forced_routing(None)
    assert torch.equal(model.generate(ids, 10, use_graph=True, forced=forced), f_eager)
    # the same model holding only the interleaved copies of its experts (how the benchmark runs it)
    for b in model.blocks:
        b["moe"].store.drop_reference_layout()
    assert torch.equal(model.forward(ids, torch.arange(12, device=dev)), logits)
    assert torch.equal(model.generate(ids, 10, use_graph=True), eager)


def test_fused_rms_norm_matches_torch_formulation():
    from qmoe_b200 import sub1
    from qmoe_b200.decoder import _rms_norm
    dev = torch.device("cuda", 0)
    g = torch.Generator().manual_seed(5)
    for rows, d in ((1, 2080), (3, 130), (2, 7)):
        x = (torch.randn(rows, d, generator=g) * 3).bfloat16().to(dev)
        w = (1 + 0.1 * torch.randn(d, generator=g)).bfloat16().to(dev)
        got, want = sub1.rms_norm(x, w), _rms_norm(x, w)
        assert float((got.float() - want.float()).abs().max()) <= 2 ** -6 * float(want.float().abs().max())


@pytest.mark.parametrize("hd,max_len", [(65, 48), (128, 300), (200, 40), (16, 9000)])
def test_decode_attention_matches_masked_sdpa(hd, max_len):
    import torch.nn.functional as F
    from qmoe_b200 import sub1
    dev = torch.device("cuda", 0)
    g = torch.Generator().manual_seed(6)
    heads = 4
    k_cache = torch.randn(heads, max_len, hd, generator=g).bfloat16().to(dev)
    v_cache = torch.randn(heads, max_len, hd, generator=g).bfloat16().to(dev)
    for p in (0, 1, 17, max_len - 1):
        qkv = torch.randn(3, heads, hd, generator=g).bfloat16().to(dev)
        k_ref, v_ref = k_cache.clone(), v_cache.clone()
        k_ref[:, p], v_ref[:, p] = qkv[1], qkv[2]
        pos = torch.full((1,), p, dtype=torch.int64, device=dev)
        got = sub1.decode_attention(qkv.contiguous(), k_cache, v_cache, pos).reshape(heads, hd)
        assert torch.equal(k_cache, k_ref) and torch.equal(v_cache, v_ref)          # cache updated in place
        want = F.scaled_dot_product_attention(qkv[0].float().unsqueeze(1), k_ref[:, :p + 1].float(),
                                              v_ref[:, :p + 1].float())[:, 0]
        assert float((got.float() - want).abs().max()) <= 2e-2 * max(float(want.abs().max()), 1e-3)


def test_decode_attention_unscaled_with_position_bias_and_position_status():
    """T5 / Switch style: scores are not scaled and a per-head bias over the key positions is added;
    a position outside the cache is refused and counted when a status word is given."""
    import torch.nn.functional as F
    from qmoe_b200 import sub1
    dev = torch.device("cuda", 0)
    g = torch.Generator().manual_seed(8)
    heads, hd, max_len = 4, 64, 40
    k_cache = (0.3 * torch.randn(heads, max_len, hd, generator=g)).bfloat16().to(dev)
    v_cache = torch.randn(heads, max_len, hd, generator=g).bfloat16().to(dev)
    bias = torch.randn(heads, max_len, generator=g).to(dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    for p in (0, 9, max_len - 1):
        qkv = (0.3 * torch.randn(3, heads, hd, generator=g)).bfloat16().to(dev)
        k_ref, v_ref = k_cache.clone(), v_cache.clone()
        k_ref[:, p], v_ref[:, p] = qkv[1], qkv[2]
        pos = torch.full((1,), p, dtype=torch.int64, device=dev)
        got = sub1.decode_attention(qkv.contiguous(), k_cache, v_cache, pos, scale=1.0, bias=bias,
                                    status=status).reshape(heads, hd)
        assert torch.equal(k_cache, k_ref) and torch.equal(v_cache, v_ref)
        want = F.scaled_dot_product_attention(qkv[0].float().unsqueeze(1), k_ref[:, :p + 1].float(),
                                              v_ref[:, :p + 1].float(), attn_mask=bias[:, None, :p + 1],
                                              scale=1.0)[:, 0]
        assert float((got.float() - want).abs().max()) <= 2e-2 * max(float(want.abs().max()), 1e-3)
    assert int(status.item()) == 0
    before_k = k_cache.clone()
    for bad in (-1, max_len):
        sub1.decode_attention(qkv.contiguous(), k_cache, v_cache,
                              torch.full((1,), bad, dtype=torch.int64, device=dev), scale=1.0, status=status)
    assert int(status.item()) == 2 and torch.equal(k_cache, before_k)      # refused, nothing written


def test_one_token_matrix_vector_kernel_variants():
    from qmoe_b200 import sub1
    from qmoe_b200.decoder import _rms_norm
    dev = torch.device("cuda", 0)
    g = torch.Generator().manual_seed(8)
    for n, k in ((6240, 2080), (37, 64), (1, 8), (300, 4096)):
        x = torch.randn(1, k, generator=g).bfloat16().to(dev)
        w = (torch.randn(n, k, generator=g) * 0.05).bfloat16().to(dev)
        ln = (1 + 0.1 * torch.randn(k, generator=g)).bfloat16().to(dev)
        res = torch.randn(1, n, generator=g).bfloat16().to(dev)
        ref = x.float() @ w.float().t()
        scale = float(ref.abs().max())
        assert float((sub1.gemv(x, w).float() - ref).abs().max()) <= 1e-2 * scale
        assert float((sub1.gemv(x, w, f32_out=True) - ref).abs().max()) <= 1e-4 * scale
        got = sub1.gemv(x, w, residual=res).float()
        assert float((got - (res.float() + ref.bfloat16().float())).abs().max()) <= 2e-2 * max(scale, 1.0)
        xn = _rms_norm(x, ln)
        y, normed = sub1.gemv(x, w, ln_weight=ln, f32_out=True, want_normed=True)
        assert float((normed.float() - xn.float()).abs().max()) <= 2 ** -6 * float(xn.float().abs().max())
        ref_n = normed.float() @ w.float().t()
        assert float((y - ref_n).abs().max()) <= 1e-4 * float(ref_n.abs().max())
