"""GPU parity of the top-1 MoE layer (route, group, grouped expert FFN, combine) against the
reference's FasterMLP semantics evaluated on the CPU with the oracle as expert FFN."""
import numpy as np
import pytest
import torch

from qmoe_b200 import sub1, synth
from util import Expert, reference_moe, reference_router, rel_err, store_from_experts

pytestmark = pytest.mark.gpu
TOL = 1e-2


@pytest.fixture(scope="module")
def dev():
    return torch.device("cuda", 0)


@pytest.fixture(scope="module")
def small_layer(dev):
    d_model, d_ff, n_exp = 128, 320, 8
    experts = [Expert(d_model, d_ff, seed=0, expert_id=e) for e in range(n_exp)]
    return experts, store_from_experts(experts, dev)


def test_route_matches_switch_router(dev):
    g = torch.Generator().manual_seed(0)
    logits = torch.randn(3, 40, 16, generator=g)
    logits[0, 0, :] = 0.0                       # exact tie: first index wins
    logits[0, 1, 3] = logits[0, 1, 9] = 5.0     # two-way tie
    choice, prob = sub1.route_top1(logits.reshape(-1, 16).to(dev).contiguous())
    mask, probs = reference_router(logits, capacity=10 ** 6)
    assert torch.equal(choice.cpu().long(), mask.argmax(-1).reshape(-1))
    assert torch.equal(prob.cpu(), probs.reshape(-1))
    for cap in (1, 2, 5):
        mask, _ = reference_router(logits, capacity=cap)
        bucket, rank, counts, offsets = sub1.rank_buckets(choice, 16, seq_len=40, capacity=cap)
        kept = mask.sum(-1).reshape(-1).bool()
        assert torch.equal(bucket.cpu() >= 0, kept)
        assert torch.equal(counts.cpu().long(), mask.sum(dim=(0, 1)))
        assert offsets.cpu().tolist() == [0] + torch.cumsum(mask.sum(dim=(0, 1)), 0).tolist()
        # ranks are stable: token order inside every bucket
        b, r = bucket.cpu().numpy(), rank.cpu().numpy()
        for e in range(16):
            assert r[b == e].tolist() == list(range(int((b == e).sum())))


@pytest.mark.parametrize("batch,seq,capacity", [(1, 24, 1024), (2, 16, 1024), (2, 16, 2), (1, 1, 1024)])
def test_moe_layer_matches_reference(dev, small_layer, batch, seq, capacity):
    experts, store = small_layer
    hidden = synth.tokens(batch * seq, store.d_model, seed=batch * 100 + seq).reshape(batch, seq, -1)
    logits = synth.router_logits(batch * seq, store.n_experts, seed=seq).reshape(batch, seq, -1)
    layer = sub1.FasterMLP(None, store, expert_capacity=capacity)
    out, (lg, index) = layer(hidden.to(dev), router_logits=logits.to(dev))
    ref = reference_moe(hidden, logits, experts, capacity)
    assert out.shape == hidden.shape and out.dtype == torch.bfloat16
    assert rel_err(out, ref) <= TOL
    mask, _ = reference_router(logits, capacity)
    assert torch.equal(index.cpu(), mask.argmax(-1))


def test_moe_layer_skewed_router_and_idle_experts(dev, small_layer):
    experts, store = small_layer
    n = 40
    hidden = synth.tokens(n, store.d_model, seed=5).reshape(1, n, -1)
    logits = synth.router_logits(n, store.n_experts, seed=6, hot_experts=2, hot_fraction=0.75).reshape(1, n, -1)
    logits[..., 5:] -= 30.0                     # experts 5..7 receive nothing
    out, _ = sub1.FasterMLP(None, store)(hidden.to(dev), router_logits=logits.to(dev))
    assert rel_err(out, reference_moe(hidden, logits, experts, 1024)) <= TOL


def test_moe_layer_with_router_weight(dev, small_layer):
    experts, store = small_layer
    g = torch.Generator().manual_seed(3)
    wr = torch.randn(store.n_experts, store.d_model, generator=g) * 0.5
    hidden = synth.tokens(12, store.d_model, seed=9).reshape(1, 12, -1)
    layer = sub1.FasterMLP(wr, store)
    out, (lg, _) = layer(hidden.to(dev))
    logits = hidden.float() @ wr.t()
    assert rel_err(lg, logits) <= 1e-3
    assert rel_err(out, reference_moe(hidden, lg.cpu(), experts, 1024)) <= TOL


def test_grouped_ffn_direct_with_empty_and_large_groups(dev, small_layer):
    """offsets with empty experts and a 9-token expert (three token groups)."""
    experts, store = small_layer
    counts = [0, 9, 1, 0, 4, 0, 2, 0]
    n = sum(counts)
    xs = synth.tokens(n, store.d_model, seed=2)
    offsets = torch.tensor([0] + np.cumsum(counts).tolist(), dtype=torch.int32, device=dev)
    ys = sub1.grouped_ffn(store, offsets, xs.to(dev), n + 3)        # max_slots larger than used
    pos = 0
    for e, c in enumerate(counts):
        if c:
            assert rel_err(ys[pos:pos + c], experts[e].oracle_ffn(xs[pos:pos + c])) <= TOL
        pos += c


def test_tensor_core_tile_path_for_heavily_loaded_experts(dev, small_layer):
    """Experts with >= 16 tokens go through the tcgen05 tile kernel (64-token blocks, 128-row blocks,
    partial last blocks in both directions); the others stay on the per-row kernel."""
    from qmoe_b200 import _lib
    experts, store = small_layer
    counts = [0, 70, 1, 16, 0, 33, 3, 64]
    n = sum(counts)
    xs = synth.tokens(n, store.d_model, seed=11)
    offsets = torch.tensor([0] + np.cumsum(counts).tolist(), dtype=torch.int32, device=dev)
    nbytes = int(_lib.load().qmoe_moe_work_bytes(store.n_experts, n, store.d_model, store.d_ff))
    work = torch.zeros(nbytes, dtype=torch.uint8, device=dev)
    before = _lib.load().qmoe_moe_set_tile_min_tokens(16)
    try:
        ys = sub1.grouped_ffn(store, offsets, xs.to(dev), n, work=work)
        torch.cuda.synchronize()
    finally:
        _lib.load().qmoe_moe_set_tile_min_tokens(before)
    header = work[:64].view(torch.int32).cpu()
    assert sub1.tile_timeouts(dev) == 0              # no bounded wait gave up
    assert int(header[4]) == 5 * 3 and int(header[5]) == 5 * 1   # 2+1+1+1 token blocks x row blocks
    pos = 0
    for e, c in enumerate(counts):
        if c:
            assert rel_err(ys[pos:pos + c], experts[e].oracle_ffn(xs[pos:pos + c])) <= TOL, (e, c)
        pos += c


def _plain_copy(store, **kw):
    """The same store without / with a differently built interleaved copy."""
    from qmoe_b200.sub1 import ExpertStore
    return ExpertStore(store.codes, store.row_off, store.minmax, store.host_descs, store.d_model, store.d_ff, **kw)


def test_interleaved_copy_holds_the_same_codes(dev, small_layer):
    """Undo the lane interleaving, the row order and the renumbering on the host: every row's codes
    come back."""
    _, store = small_layer
    assert store.il_codes is not None
    il = store.il_codes.cpu().numpy().view(np.uint16).reshape(-1, 8)          # [16-byte entry, 8 codes]
    base = store.blk_base.cpu().numpy()
    inverse = np.empty(65536, np.int64)
    inverse[store.remap.cpu().numpy()] = np.arange(65536)
    codes = store.codes.cpu().numpy().view(np.uint16)
    row_off = store.row_off.cpu().numpy()
    rows = store.il_rows.cpu().numpy()
    for d in store.host_descs:
        # inside every 1024 positions the rows of the matrix, each once, longest first
        mine_rows = rows[d.minmax_base:d.minmax_base + d.height]
        lengths = np.diff(row_off[d.rowoff_base:d.rowoff_base + d.height + 1])
        for s0 in range(0, d.height, 1024):
            seg = mine_rows[s0:s0 + 1024]
            assert sorted(seg.tolist()) == list(range(s0, min(s0 + 1024, d.height)))
            assert (np.diff(lengths[seg]) <= 0).all()
        for pos in range(d.height):
            row = int(mine_rows[pos])
            b, e = row_off[d.rowoff_base + row], row_off[d.rowoff_base + row + 1]
            gblk, lane = (d.minmax_base + pos) // 32, pos % 32
            chunks = (base[gblk + 1] - base[gblk]) // 32
            mine = il[base[gblk] + lane:base[gblk] + 32 * chunks:32].reshape(-1)
            assert len(mine) >= e - b
            assert (inverse[mine[:e - b]] == codes[d.code_base + b:d.code_base + e]).all()
            assert (mine[e - b:] == store.remap.cpu().numpy()[0] % 65536).all()   # padding = code 0, renumbered


@pytest.mark.parametrize("variant", ["row_by_row", "interleaved_plain_numbers", "interleaved_only"])
def test_interleaved_and_row_by_row_stores_give_identical_results(dev, small_layer, variant):
    """Same codes, same order of accumulation: the layouts must agree bit for bit."""
    experts, store = small_layer
    counts = [3, 9, 1, 0, 4, 2, 2, 5]
    n = sum(counts)
    xs = synth.tokens(n, store.d_model, seed=5).to(dev)
    offsets = torch.tensor([0] + np.cumsum(counts).tolist(), dtype=torch.int32, device=dev)
    want = sub1.grouped_ffn(store, offsets, xs, n)
    if variant == "row_by_row":
        other = _plain_copy(store, interleave=False)
        assert other.il_codes is None
    elif variant == "interleaved_plain_numbers":
        other = _plain_copy(store, interleave=False)
        other.interleave(renumber=False, sort_rows=False)
        assert other.il_rows is None
    else:
        other = _plain_copy(store)
        other.drop_reference_layout()
        assert other.codes is None and other.compressed_bytes == store.compressed_bytes
        with pytest.raises(RuntimeError):
            other.matrix(0)
    got = sub1.grouped_ffn(other, offsets, xs, n)
    assert torch.equal(got[:n], want[:n])
    assert rel_err(got[:counts[0]], experts[0].oracle_ffn(xs[:counts[0]].cpu())) <= TOL


def test_remap_tables_reject_a_non_permutation(dev):
    from qmoe_b200 import _lib
    remap = torch.arange(65536, dtype=torch.int32, device=dev)
    remap[7] = 8                                                  # two codes onto one number
    tab = torch.empty(65536, dtype=torch.int32, device=dev)
    dec_out = torch.empty(131072, dtype=torch.int32, device=dev)
    rc = _lib.load().qmoe_sub1_remap_tables(sub1.DEC(dev).data_ptr(), remap.data_ptr(), tab.data_ptr(),
                                            dec_out.data_ptr(), dev.index, None)
    assert rc == _lib.ERR_INVALID_ARG
    assert b"permutation" in _lib.load().qmoe_last_error()


@pytest.mark.parametrize("interleave", [True, False])
def test_grouped_ffn_with_a_table_that_needs_the_digit_path(dev, interleave):
    """A decoder table with an entry of four non-zeros (not expressible in the sparse form): the
    grouped kernels must fall back to digit-by-digit decoding of that entry, in the row-by-row and in
    the interleaved, renumbered layout, for groups of one, two and three tokens."""
    from oracle import oracle as O
    from qmoe_b200 import _lib
    from qmoe_b200.sub1 import ExpertStore
    dec_np = O.build_dictionary()[0].copy()
    digits, nweights = O.numpy_entry_digits(dec_np)
    bad = int(np.where((nweights >= 8) & (nweights <= 28) & ((digits != 0).sum(1) == 3))[0][0])
    free = int(np.where(digits[bad][:nweights[bad]] == 0)[0][0])
    word, bit = free // 14, 4 + 2 * (free % 14)
    dec_np[2 * bad + word] = np.int32(np.uint32(dec_np[2 * bad + word]) | np.uint32(2 << bit))
    all_zero = np.where((digits != 0).sum(1) == 0)[0]
    zero_run = {int(nweights[c]): int(c) for c in all_zero[::-1]}     # runs of 2..28 zeros
    some = [int(c) for c in np.where((nweights == 12) & ((digits != 0).sum(1) == 2))[0][:4]]

    def row(width, r):
        codes, left = [], width
        for c in ([bad] if r % 2 == 0 else []) + [some[r % len(some)]]:
            codes.append(c)
            left -= int(nweights[c])
        while left > 0:
            n = min(left, 28)
            codes.append(zero_run[n])
            left -= n
        assert left == 0
        return codes[::-1] if r % 3 == 0 else codes

    # wi: 1024 rows one per thread plus 32 one per warp in k_matmul_grouped; wo (64 rows, few in
    # total): k_matmul_grouped_warp
    d_model, d_ff, n_exp = 64, 1056, 40
    parts, dense = [], []
    for h, w in ((d_ff, d_model), (d_model, d_ff)):
        rows = [row(w, r) for r in range(h)]
        codes = np.array([c for rc in rows for c in rc], dtype=np.uint16)
        row_off = np.concatenate([[0], np.cumsum([len(rc) for rc in rows])]).astype(np.int32)
        mm = synth.row_scales(h, 3, h)
        sym = O.numpy_decode_matrix(dec_np, codes, row_off, h, w)
        deq = np.concatenate([np.zeros((h, 1), np.float32), mm.float().numpy().reshape(-1, 2)], 1)
        dense.append(torch.from_numpy(np.take_along_axis(deq, sym.astype(np.int64), 1)))
        parts.append((torch.from_numpy(codes.view(np.int16)).to(dev), torch.from_numpy(row_off).to(dev), mm.to(dev), h, w))
    dec2 = torch.from_numpy(dec_np).to(dev)
    base = ExpertStore.from_matrices(parts * n_exp, d_model, d_ff)    # experts with the same two matrices
    store = ExpertStore(base.codes, base.row_off, base.minmax, base.host_descs, d_model, d_ff,
                        interleave=interleave, dec=dec2)
    assert (store.il_codes is not None) == interleave
    counts = [1 + e % 3 for e in range(n_exp)]
    n = sum(counts)
    xs = synth.tokens(n, d_model, seed=9)
    offsets = torch.tensor([0] + np.cumsum(counts).tolist(), dtype=torch.int32, device=dev)
    ys = sub1.grouped_ffn(store, offsets, xs.to(dev), n).cpu()
    hidden = torch.relu((xs.float() @ dense[0].t()).bfloat16())
    want = (hidden.float() @ dense[1].t()).bfloat16()
    assert rel_err(ys, want) <= TOL
    _lib.check(_lib.load().qmoe_sub1_release(0))


def test_tile_path_reports_a_wait_that_ran_out(dev, small_layer):
    """Every wait of the tile kernel on an MMA-completion barrier is bounded.  With the bound lowered
    to a single poll the first such wait gives up although nothing hangs: the CTA stops, writes
    zeros for the rows it did not finish, and the library's sticky status word reports it until it
    is read with reset.  (The clean-up waits before tensor memory is released keep the full bound.)"""
    from qmoe_b200 import _lib
    experts, store = small_layer
    L = _lib.load()
    counts = [0, 70, 0, 0, 0, 0, 0, 0]
    n = sum(counts)
    xs = synth.tokens(n, store.d_model, seed=12).to(dev)
    offsets = torch.tensor([0] + np.cumsum(counts).tolist(), dtype=torch.int32, device=dev)
    assert sub1.tile_timeouts(dev, reset=True) == 0
    before = L.qmoe_moe_set_tile_min_tokens(16)
    L.qmoe_moe_set_tile_wait_limit(1)
    try:
        ys = sub1.grouped_ffn(store, offsets, xs, n)
        torch.cuda.synchronize()
    finally:
        L.qmoe_moe_set_tile_wait_limit(0)
        L.qmoe_moe_set_tile_min_tokens(before)
    assert torch.isfinite(ys.float()).all()
    assert sub1.tile_timeouts(dev) > 0                     # sticky: still there on a second read
    with pytest.raises(_lib.QmoeError):
        sub1.check_tile_status(dev)                        # raises and clears
    assert sub1.tile_timeouts(dev) == 0
    # the same step with the default bound completes and matches the oracle
    before = L.qmoe_moe_set_tile_min_tokens(16)
    try:
        ys = sub1.grouped_ffn(store, offsets, xs, n)
        torch.cuda.synchronize()
    finally:
        L.qmoe_moe_set_tile_min_tokens(before)
    assert sub1.tile_timeouts(dev) == 0
    assert rel_err(ys, experts[1].oracle_ffn(xs.cpu())) <= TOL


def test_aliased_store_reuses_the_matrices_of_its_experts(dev, small_layer):
    """``ExpertStore.aliased``: a longer descriptor table over the same arrays; expert e behaves as
    expert e % n (the benchmark measures its L2-resident ceiling on such a store)."""
    experts, store = small_layer
    n = store.n_experts
    big = store.aliased(3 * n)
    assert big.n_experts == 3 * n and big.il_codes is store.il_codes and big.codes is store.codes
    counts = [1, 0, 2] * n
    t = sum(counts)
    xs = synth.tokens(t, store.d_model, seed=21).to(dev)
    offsets = torch.tensor([0] + np.cumsum(counts).tolist(), dtype=torch.int32, device=dev)
    ys = sub1.grouped_ffn(big, offsets, xs, t).cpu()
    off = offsets.cpu().tolist()
    for e in range(3 * n):
        if counts[e]:
            rows = slice(off[e], off[e + 1])
            assert rel_err(ys[rows], experts[e % n].oracle_ffn(xs.cpu()[rows])) <= TOL, f"expert {e}"


@pytest.mark.parametrize("n,capacity", [(1, 1024), (5, 1024), (32, 1024), (32, 2), (7, 0)])
def test_one_launch_routing_of_few_tokens_equals_the_general_kernels(dev, n, capacity):
    n_exp, d = 300, 96                                    # not a multiple of the CTA size
    g = torch.Generator().manual_seed(n * 31 + capacity)
    logits = torch.randn(n, n_exp, generator=g)
    hot = torch.randint(0, 6, (n,), generator=g)          # few experts: collisions, capacity drops
    logits[torch.arange(n), hot] += 8.0
    logits = logits.to(dev).contiguous()
    hidden = torch.randn(n, d, generator=g).bfloat16().to(dev)
    choice, prob = sub1.route_top1(logits)
    bucket, rank, _, offsets = sub1.rank_buckets(choice, n_exp, n, capacity)
    xs = torch.zeros_like(hidden)
    slot = sub1.permute_rows(bucket, rank, offsets, hidden, xs)
    prob2, offsets2, slot2, xs2 = sub1.route_small(logits, hidden, n_exp, capacity)
    assert torch.equal(choice.cpu(), hot.to(torch.int32))
    assert torch.equal(offsets2, offsets) and torch.equal(slot2, slot)
    assert (prob2.float() - prob.float()).abs().max() <= 2 ** -7 * prob.float().max()
    kept = int(offsets[-1])
    assert torch.equal(xs2[:kept], xs[:kept])
    assert kept == int((slot >= 0).sum())
