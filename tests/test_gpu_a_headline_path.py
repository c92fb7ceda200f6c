"""The path the benchmark's headline number is timed on, checked against the oracle.

``bench.py`` times a switch-c-2048 layer: d_model 2080, d_ff 6144, hundreds of active experts with
one to a few tokens each.  With that many (expert, token group) pairs the work list cuts every matrix
into items of up to 1024 rows for the persistent row-per-thread kernel (groups of one to four
tokens); ``wo`` has 2080 = 2 * 1024 + 32 rows, so its last 32 rows are not part of such an item
and are done one row per warp by the CTA that takes the matrix's last item.  No small layer and no
single expert reaches that branch, so this file runs a SLICE of the benchmark's layer: 160 experts
of the real shape, 300 uniformly routed tokens (one to six tokens per active expert).

Checks: the work list holds row-per-thread items for rows 0..2047 of which one per (expert, token
group) also covers the remainder; outputs of the busiest experts and of single-token experts equal
the oracle FFN (decode-then-matmul, fp32 accumulation, bf16 hidden activation) within 1e-2 of
max|ref|, with rows 2048..2079 checked on their own; the interleaved store and the row-by-row store
give the same bits where both walk a row with one thread.  File name chosen so that the file is
collected before the other GPU tests.
"""
import numpy as np
import pytest
import torch

from oracle import oracle as O
from qmoe_b200 import _lib, sub1, synth
from util import rel_err

pytestmark = pytest.mark.gpu
SEED = 0
TOL = 1e-2          # max|got - ref| / max|ref|
N_EXPERTS = 160
N_TOKENS = 300


def _oracle_expert(d_model, d_ff, e):
    _, trie = O.build_dictionary()
    mats = []
    for which, (h, w) in enumerate(((d_ff, d_model), (d_model, d_ff))):
        m = 2 * e + which
        sym = O.synth_ternary(h * w, SEED, synth.matrix_first_index(m), 0.9).reshape(h, w)
        codes, row_off = O.encode_matrix(trie, sym)
        mats.append((codes, row_off, synth.row_scales(h, SEED, m)))
    return mats


def _oracle_ffn(mats, x_bf16, d_model, d_ff):
    dec, _ = O.build_dictionary()
    bits = lambda t: t.contiguous().view(torch.int16).numpy().view(np.uint16)  # noqa: E731
    wi, wo = mats
    y = O.expert_ffn(dec, (wi[0], wi[1], bits(wi[2])), (wo[0], wo[1], bits(wo[2])), bits(x_bf16), d_model, d_ff)
    return torch.from_numpy(y.view(np.int16)).view(torch.bfloat16)


def _sorted_tokens(dev, store, hidden, logits):
    """Route as FasterMLP does and return (offsets, xs sorted by expert, slot, choice)."""
    choice, _prob = sub1.route_top1(logits.to(dev).contiguous())
    bucket, rank, _counts, offsets = sub1.rank_buckets(choice, store.n_experts, hidden.shape[0], 1024)
    xs = torch.empty((hidden.shape[0], store.d_model), dtype=torch.bfloat16, device=dev)
    slot = sub1.permute_rows(bucket, rank, offsets, hidden.to(dev), xs)
    return offsets, xs, slot, choice


def test_switch_c_2048_slice_grouped_path_against_the_oracle():
    d_model, d_ff, _ = synth.SHAPES["switch-c-2048"]
    dev = torch.device("cuda", 0)
    L = _lib.load()
    store = synth.build_store(d_model, d_ff, list(range(N_EXPERTS)), SEED, dev)
    assert store.il_codes is not None, "the benchmark runs on the interleaved copy"
    hidden = synth.tokens(N_TOKENS, d_model, SEED + 1)
    logits = synth.router_logits(N_TOKENS, N_EXPERTS, SEED + 2)
    offsets, xs, slot, choice = _sorted_tokens(dev, store, hidden, logits)

    nbytes = int(L.qmoe_moe_work_bytes(N_EXPERTS, N_TOKENS, d_model, d_ff))
    work = torch.zeros(nbytes, dtype=torch.uint8, device=dev)
    ys = sub1.grouped_ffn(store, offsets, xs, N_TOKENS, work=work)
    torch.cuda.synchronize()
    assert sub1.tile_timeouts(dev) == 0

    # the work list of this step: row-per-thread items of at most 1024 rows for rows 0..2047 of wo and
    # all rows of wi; the last item of every (expert, token group) of wo carries the 32 remainder rows
    # (2080 = 2 * 1024 + 32) for its CTA's warps
    plan = sub1.work_plan(work, N_TOKENS, d_ff)
    counts = torch.bincount(choice.cpu().long(), minlength=N_EXPERTS)
    assert plan["group_tokens"] == 4
    groups = int(sum((int(c) + 3) // 4 for c in counts))
    assert plan["wi_items"] >= groups * (d_ff // 1024) and plan["wi_items"] % groups == 0
    assert plan["wo_items"] >= groups * (d_model // 1024) and plan["wo_items"] % groups == 0
    assert 32 <= plan["wi_rows_per_item"] <= 1024 and 32 <= plan["wo_rows_per_item"] <= 1024
    assert plan["wi_warp_items"] == 0 and plan["wo_warp_items"] == 0
    assert plan["wo_items_with_remainder"] == groups, "rows 2048..2079 of wo are not covered"

    # this step is small enough for the single launch that runs the items of wi and wo together; the
    # benchmark's full layer takes one launch per linear: same bits
    was = L.qmoe_moe_set_fused_phases(0)
    try:
        ys_two = sub1.grouped_ffn(store, offsets, xs, N_TOKENS)
        torch.cuda.synchronize()
    finally:
        L.qmoe_moe_set_fused_phases(was)
    assert was == 1 and torch.equal(ys, ys_two), "one launch for both linears differs from one launch per linear"
    # a step declared as large as the benchmark's (2048 token slots) takes one launch per linear whose
    # CTAs claim their items two ahead and stage the next item's activations early: same bits
    ys_big = sub1.grouped_ffn(store, offsets, xs, 2048)
    torch.cuda.synchronize()
    assert torch.equal(ys_big[:N_TOKENS], ys), "the large-step launches differ from the fused launch"

    # the same step on a store without the interleaved copy (row-by-row streams, one thread per row)
    plain = sub1.ExpertStore(store.codes, store.row_off, store.minmax, store.host_descs, d_model, d_ff,
                             interleave=False)
    ys_plain = sub1.grouped_ffn(plain, offsets, xs, N_TOKENS)
    torch.cuda.synchronize()
    main = d_model - d_model % 1024
    assert torch.equal(ys[:, :main], ys_plain[:, :main]), "interleaved and row-by-row stores differ in rows < 2048"
    # remainder rows: summed by 32 lanes instead of one thread, so the last fp32 bits may differ
    assert rel_err(ys[:, main:], ys_plain[:, main:]) <= 2e-3

    ys_c, xs_c = ys.cpu(), xs.cpu()
    off = offsets.cpu().tolist()
    order = torch.argsort(counts, descending=True).tolist()
    singles = [e for e in order if counts[e] == 1][:2]
    doubles = [e for e in order if counts[e] == 2][:1]
    chosen = order[:2] + doubles + singles
    assert int(counts[order[0]]) >= 4 and singles, "routing of this seed changed"
    for e in chosen:
        mats = _oracle_expert(d_model, d_ff, e)
        rows = slice(off[e], off[e + 1])
        ref = _oracle_ffn(mats, xs_c[rows], d_model, d_ff)
        assert rel_err(ys_c[rows], ref) <= TOL, f"expert {e} with {int(counts[e])} tokens"
        tail = ref[:, main:].float()
        err = float((ys_c[rows][:, main:].float() - tail).abs().max() / max(float(ref.float().abs().max()), 1e-12))
        assert err <= TOL, f"rows {main}..{d_model - 1} of expert {e}"
        assert float(tail.abs().max()) > 0.0
