"""Expert-parallel layer on GPUs: the single-rank path on one GPU, and two NCCL ranks (when the box
has two GPUs) against the single-GPU FasterMLP on the same seeded layer."""
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


def _worker(rank, world, port, out_dir):
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
        layer = ExpertParallelMLP(None, store, N_EXP)
        out, _ = layer(hidden, router_logits=logits)
        out2, _ = layer(hidden, router_logits=logits)          # second step reuses nothing stale
        torch.cuda.synchronize()
        assert torch.equal(out, out2)
        torch.save(out.cpu(), os.path.join(out_dir, f"r{rank}.pt"))
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_ep_two_nccl_ranks_equal_single_gpu(tmp_path):
    import torch.multiprocessing as mp
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    dev = torch.device("cuda", 0)
    store, hidden, logits = _single_gpu_reference(dev)
    want, _ = sub1.FasterMLP(None, store)(hidden.to(dev).unsqueeze(0), router_logits=logits.to(dev).unsqueeze(0))
    got = torch.cat([torch.load(os.path.join(str(tmp_path), f"r{r}.pt")) for r in range(world)])
    # same kernels, same per-expert token order (stable ranking) -> identical results
    assert rel_err(got, want.squeeze(0)) <= 1e-2
    assert torch.equal(got, want.squeeze(0).cpu())
