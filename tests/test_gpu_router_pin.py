"""Pins the routing kernels against HuggingFace's own ``SwitchTransformersTop1Router``.

The reference calls that router at sub1.py:310 (transformers 4.28: returns mask, probs, logits).
The transformers installed here is 5.x, whose router returns (probs, one-hot index, max prob) and
keeps a singleton axis in the one-hot tensor, so that its ``cumsum(dim=-2)`` runs over that axis and
its capacity mask never drops a token.  What both versions share, and what is compared here on the
same logits, is: softmax in fp32, cast to the input dtype (bf16), the expert = first index of the
largest bf16 probability, and that probability as the scaling factor.  The 4.28 capacity rule
(``cumsum`` over the sequence axis ``<= expert_capacity``) is then applied with the same two torch
calls to the installed router's own one-hot output and compared with ``qmoe_moe_rank``.

The router's classifier is set to the identity (hidden size = number of experts) so that the
hidden states ARE the logits, exactly, and both sides see the same fp32 numbers.
"""
import pytest
import torch

from qmoe_b200 import sub1

pytestmark = pytest.mark.gpu


def _hf_router(n_experts, capacity):
    try:
        from transformers import SwitchTransformersConfig
        from transformers.models.switch_transformers.modeling_switch_transformers import (
            SwitchTransformersTop1Router)
    except Exception as exc:  # pragma: no cover
        pytest.skip(f"transformers' Switch router cannot be imported: {exc}")
    cfg = SwitchTransformersConfig(num_experts=n_experts, d_model=n_experts, expert_capacity=capacity,
                                   router_bias=False, router_jitter_noise=0.0)
    router = SwitchTransformersTop1Router(cfg).eval()
    with torch.no_grad():
        router.classifier.weight.copy_(torch.eye(n_experts))
    return router


def _hf_route(logits_bf16, capacity):
    """(expert index [B, S], bf16 max probability [B, S], kept mask [B, S] under the 4.28 rule)."""
    router = _hf_router(logits_bf16.shape[-1], capacity)
    with torch.no_grad():
        out = router(logits_bf16)
    probs = out[0]
    one_hot = [t for t in out if t.dtype == torch.int64][0]
    one_hot = one_hot.reshape(*logits_bf16.shape)            # 5.x keeps a singleton axis; 4.28 has none
    assert int(one_hot.sum(-1).max()) <= 1
    priority = torch.cumsum(one_hot, dim=-2)                 # transformers 4.28, over the sequence
    kept = (one_hot * (priority <= capacity)).sum(-1).bool()
    # 5.x never drops; where 4.28 keeps everything the two agree
    return one_hot.argmax(-1), probs.reshape(logits_bf16.shape[:-1]), kept


def _cases():
    g = torch.Generator().manual_seed(0)
    few = torch.randn(3, 40, 16, generator=g)
    few[0, 0, :] = 0.0                                        # all equal: the first index wins
    few[0, 1, 3] = few[0, 1, 9] = 5.0                         # two-way tie
    few[1, :, :] = 0.0
    few[1, :, 5] = 4.0                                        # a whole sequence on one expert: overflow
    # two logits one bf16 step apart, the smaller at the lower index: their fp32 probabilities differ
    # but round to the same bf16 value, so the router takes the lower index, unlike an fp32 argmax
    few[2, :8, :] = -10.0
    few[2, :8, 11] = 0.25
    few[2, :8, 4] = 0.25 - 2.0 ** -9
    many = torch.randn(2, 64, 2048, generator=g)              # the expert count of switch-c-2048
    peaked = torch.randn(2, 32, 128, generator=g) * 4.0
    return [("ties and overflow", few, (1, 2, 5, 1024)), ("2048 experts", many, (1, 1024)),
            ("peaked", peaked, (2, 1024))]


@pytest.mark.parametrize("name,logits,capacities", _cases(), ids=[c[0] for c in _cases()])
def test_route_and_capacity_rule_equal_the_installed_switch_router(name, logits, capacities):
    dev = torch.device("cuda", 0)
    logits = logits.bfloat16()                                # bf16 hidden states, as the bf16 model has
    b, s, e = logits.shape
    choice, prob = sub1.route_top1(logits.float().reshape(-1, e).to(dev).contiguous())
    for cap in capacities:
        index, probs, kept = _hf_route(logits, cap)
        assert torch.equal(choice.cpu().long(), index.reshape(-1)), f"{name}: expert index"
        assert torch.equal(prob.cpu(), probs.reshape(-1)), f"{name}: bf16 router probability"
        bucket, rank, counts, _ = sub1.rank_buckets(choice, e, seq_len=s, capacity=cap)
        assert torch.equal(bucket.cpu() >= 0, kept.reshape(-1)), f"{name}: kept mask at capacity {cap}"
        want = torch.zeros(e, dtype=torch.int64)
        want.index_add_(0, index.reshape(-1)[kept.reshape(-1)], torch.ones(int(kept.sum()), dtype=torch.int64))
        assert torch.equal(counts.cpu().long(), want)
    if name == "ties and overflow":
        # the argmax is taken over the bf16 probabilities, not over fp32 ones
        fp32_arg = torch.softmax(logits.float(), -1).argmax(-1).reshape(-1)
        assert int((fp32_arg != choice.cpu().long()).sum()) >= 8
