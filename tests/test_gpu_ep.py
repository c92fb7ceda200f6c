"""Expert-parallel layer on GPUs: the single-rank path on one GPU, and two ranks (when the box has
two GPUs) against the single-GPU FasterMLP on the same seeded layer, once with the NCCL exchange and
once with rows stored straight into the peer's memory."""
import os
import socket
import sys

import pytest
import torch

from qmoe_b200 import sub1, synth
from util import rel_err

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))
D_MODEL, D_FF, N_EXP, N_TOK, SEED = 256, 512, 8, 64, 3


def _single_gpu_reference(dev):
    store = synth.build_store(D_MODEL, D_FF, list(range(N_EXP)), SEED, dev)
    hidden = synth.tokens(N_TOK, D_MODEL, SEED)
    logits = synth.router_logits(N_TOK, N_EXP, SEED)
    return store, hidden, logits


def test_ep_single_rank_equals_fastermlp():
    from qmoe_b200.ep import ExpertParallelMLP
    dev = torch.device("cuda", 0)
    store, hidden, logits = _single_gpu_reference(dev)
    want, _ = sub1.FasterMLP(None, store)(hidden.to(dev).unsqueeze(0), router_logits=logits.to(dev).unsqueeze(0))
    got, _ = ExpertParallelMLP(None, store, N_EXP)(hidden.to(dev), router_logits=logits.to(dev))
    assert torch.equal(got, want.squeeze(0))
    # a pair capacity below the worst case drops the overflow: those tokens pass through as prob * x
    got2, _ = ExpertParallelMLP(None, store, N_EXP, pair_capacity=N_TOK // 2)(hidden.to(dev),
                                                                              router_logits=logits.to(dev))
    assert torch.equal(got2[: N_TOK // 2], want.squeeze(0)[: N_TOK // 2])


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out_dir, exchange):
    sys.path.insert(0, HERE)
    sys.path.insert(0, os.path.dirname(HERE))
    import torch.distributed as dist
    from qmoe_b200.ep import ExpertParallelMLP
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    dev = torch.device("cuda", rank)
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        local = N_EXP // world
        store = synth.build_store(D_MODEL, D_FF, list(range(rank * local, (rank + 1) * local)), SEED, dev)
        per = N_TOK // world
        hidden = synth.tokens(N_TOK, D_MODEL, SEED)[rank * per:(rank + 1) * per].contiguous().to(dev)
        logits = synth.router_logits(N_TOK, N_EXP, SEED)[rank * per:(rank + 1) * per].contiguous().to(dev)
        layer = ExpertParallelMLP(None, store, N_EXP, exchange=exchange)
        out, _ = layer(hidden, router_logits=logits)
        out2, _ = layer(hidden, router_logits=logits)          # second step reuses nothing stale
        for _ in range(3):                                     # the exchange buffers are reused every step
            out3, _ = layer(hidden, router_logits=logits)
        torch.cuda.synchronize()
        assert layer.exchange == exchange
        assert torch.equal(out, out2) and torch.equal(out, out3)
        assert layer.peer_timeouts() == 0 and layer.overflow_count() == 0
        # a pair capacity that is too small: tokens beyond it pass through and are counted; with
        # exact=True the step is run again at the worst-case capacity and equals the full result
        tight = ExpertParallelMLP(None, store, N_EXP, exchange=exchange, pair_capacity=8)
        dropped, _ = tight(hidden, router_logits=logits)
        n_over = tight.overflow_count()
        total = torch.tensor([n_over], device=dev)
        dist.all_reduce(total)
        assert int(total.item()) > 0, "the seed no longer overflows a capacity of 8"
        assert int((dropped != out).any(dim=1).sum()) == n_over
        exact = ExpertParallelMLP(None, store, N_EXP, exchange=exchange, pair_capacity=8, exact=True)
        for _ in range(2):
            again, _ = exact(hidden, router_logits=logits)
            assert torch.equal(again, out)
        assert exact.peer_timeouts() == 0
        torch.save(out.cpu(), os.path.join(out_dir, f"r{rank}.pt"))
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("exchange", ["nccl", "peer"])
def test_ep_two_ranks_equal_single_gpu(tmp_path, exchange):
    import torch.multiprocessing as mp
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path), exchange), nprocs=world, join=True)
    dev = torch.device("cuda", 0)
    store, hidden, logits = _single_gpu_reference(dev)
    want, _ = sub1.FasterMLP(None, store)(hidden.to(dev).unsqueeze(0), router_logits=logits.to(dev).unsqueeze(0))
    got = torch.cat([torch.load(os.path.join(str(tmp_path), f"r{r}.pt")) for r in range(world)])
    # same kernels, same per-expert token order (stable ranking) -> identical results
    assert rel_err(got, want.squeeze(0)) <= 1e-2
    assert torch.equal(got, want.squeeze(0).cpu())


def test_peer_entry_points_on_one_gpu():
    """The kernels of the peer exchange with every "peer" buffer in this GPU's own memory: two
    emulated ranks' blocks side by side, rows stored through the block table, results stored through
    the per-slot addresses; equal to the slot-array path."""
    dev = torch.device("cuda", 0)
    store, hidden, logits = _single_gpu_reference(dev)
    hidden, logits = hidden.to(dev), logits.to(dev)
    n, d, G = N_TOK, D_MODEL, 2
    cap = n
    local = N_EXP // G
    choice, prob = sub1.route_top1(logits.float().contiguous())
    overflow = torch.zeros(1, dtype=torch.int32, device=dev)
    expert, slot, send = sub1.ep_dispatch(choice, hidden, N_EXP, G, n, 1024, cap, overflow)
    # "receive buffers" of the two destinations, each with room for two source blocks; this rank is source 1
    recv = torch.zeros((G, G * cap, d + 8), dtype=torch.bfloat16, device=dev)
    recv[:, :, d:].view(torch.int32)[..., 0] = -1
    blocks = torch.tensor([recv[q, cap].data_ptr() for q in range(G)], dtype=torch.int64).to(dev)
    expert2, slot2 = sub1.ep_dispatch_peer(choice, hidden, N_EXP, G, n, 1024, cap, overflow, blocks)
    torch.cuda.synchronize()
    assert torch.equal(expert, expert2) and torch.equal(slot, slot2) and int(overflow.item()) == 0
    for q in range(G):
        part = send[q * cap:(q + 1) * cap]
        ids = part[:, d:].view(torch.int32)[..., 0]
        assert torch.equal(recv[q, cap:, d:].view(torch.int32)[..., 0], ids)
        used = ids >= 0                                     # unused slots of `send` hold no row
        assert bool(used.any()) and torch.equal(recv[q, cap:][used][:, :d], part[used][:, :d])
        assert bool((recv[q, :cap, d:].view(torch.int32)[..., 0] == -1).all())

    # destination 0 groups what it received from "source 1" and stores results through addresses
    e_store = synth.build_store(D_MODEL, D_FF, list(range(local)), SEED, dev)
    rows = recv[0]
    offsets, slot_of_row, row_of_slot = sub1.plan_rows(local, rows=rows, d_model=d)
    ret = torch.zeros((G * cap, d), dtype=torch.bfloat16, device=dev)
    sub1.grouped_ffn_rows(e_store, offsets, rows, row_of_slot, ret, row_of_slot, G * cap)
    back = torch.zeros((G, cap, d), dtype=torch.bfloat16, device=dev)   # one return block per source rank
    out_blocks = torch.tensor([back[q].data_ptr() for q in range(G)], dtype=torch.int64).to(dev)
    offsets2, sor2, ros2, ptrs = sub1.plan_rows_peer(local, rows, d, out_blocks, cap, 2 * d)
    sub1.grouped_ffn_scatter(e_store, offsets2, rows, ros2, ptrs, G * cap)
    torch.cuda.synchronize()
    assert torch.equal(offsets, offsets2) and torch.equal(slot_of_row, sor2)
    m = int(offsets[-1])
    assert m > 0 and torch.equal(row_of_slot[:m], ros2[:m])
    assert torch.equal(back.reshape(G * cap, d), ret)


def test_peer_barrier_alone_and_its_time_limit():
    """One rank: nothing to wait for.  Two ranks emulated by two flag blocks on one GPU where the
    other rank never runs: the wait ends at its time limit and is counted; the context stays usable."""
    import time
    from qmoe_b200 import _lib
    dev = torch.device("cuda", 0)
    L = _lib.load()
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    flags = torch.zeros((2, 4), dtype=torch.int32, device=dev)
    table = torch.tensor([flags[0].data_ptr()], dtype=torch.int64).to(dev)
    stream = torch.cuda.current_stream(dev).cuda_stream
    _lib.check(L.qmoe_moe_peer_barrier(table.data_ptr(), 0, 1, 0, 1000, status.data_ptr(), 0, stream))
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    table2 = torch.tensor([flags[0].data_ptr(), flags[1].data_ptr()], dtype=torch.int64).to(dev)
    t0 = time.time()
    _lib.check(L.qmoe_moe_peer_barrier(table2.data_ptr(), 0, 2, 1, 50, status.data_ptr(), 0, stream))
    torch.cuda.synchronize()
    assert time.time() - t0 < 5.0
    assert int(status.item()) == 1
    assert int(flags[1, 1 * 2 + 0].item()) == 1          # the flag this rank raised for the absent one
    # a flag that is already there is taken at once
    flags.zero_()
    flags[0, 1 * 2 + 1] = 1
    status.zero_()
    _lib.check(L.qmoe_moe_peer_barrier(table2.data_ptr(), 0, 2, 1, 1000, status.data_ptr(), 0, stream))
    torch.cuda.synchronize()
    assert int(status.item()) == 0 and int(flags[0, 3].item()) == 0
    assert torch.ones(4, device=dev).sum().item() == 4.0
