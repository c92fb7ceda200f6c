"""Expert-parallel layer among CPU ranks (gloo, world_size 2): the dispatch / combine exchanges and
all slot arithmetic of qmoe_b200.ep, with the device ops replaced by the torch-CPU test double and
the oracle as expert FFN.  The result must equal the single-process reference layer."""
import os
import socket
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

HERE = os.path.dirname(os.path.abspath(__file__))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, capacity, result_dir):
    sys.path.insert(0, HERE)
    sys.path.insert(0, os.path.dirname(HERE))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import cpu_ops
        from qmoe_b200 import synth
        from qmoe_b200.ep import ExpertParallelMLP
        from util import Expert, reference_moe
        d_model, d_ff, n_exp, n_tok = 64, 96, 4, 12
        experts = [Expert(d_model, d_ff, seed=1, expert_id=e) for e in range(n_exp)]
        local = n_exp // world
        store = cpu_ops.CpuStore(experts[rank * local:(rank + 1) * local])
        hidden = synth.tokens(n_tok, d_model, seed=3)
        logits = synth.router_logits(n_tok, n_exp, seed=4)
        per = n_tok // world
        layer = ExpertParallelMLP(None, store, n_exp, expert_capacity=capacity, ops=cpu_ops)
        out, (_, index) = layer(hidden[rank * per:(rank + 1) * per].contiguous(),
                                router_logits=logits[rank * per:(rank + 1) * per].contiguous(), seq_len=per)
        # reference: every rank's tokens form their own sequence of length `per`
        ref = reference_moe(hidden.reshape(world, per, d_model), logits.reshape(world, per, n_exp), experts,
                            capacity)[rank]
        err = float((out.float() - ref.float()).abs().max() / ref.float().abs().max())
        torch.save({"err": err, "index": index}, os.path.join(result_dir, f"r{rank}.pt"))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("capacity", [1024, 2])
def test_expert_parallel_two_cpu_ranks(tmp_path, capacity):
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), capacity, str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        res = torch.load(os.path.join(str(tmp_path), f"r{r}.pt"))
        assert res["err"] <= 1e-2, res


def test_single_rank_path_without_process_group():
    sys.path.insert(0, HERE)
    import cpu_ops
    from qmoe_b200 import synth
    from qmoe_b200.ep import ExpertParallelMLP
    from util import Expert, reference_moe
    d_model, d_ff, n_exp, n_tok = 64, 96, 3, 7
    experts = [Expert(d_model, d_ff, seed=2, expert_id=e) for e in range(n_exp)]
    layer = ExpertParallelMLP(None, cpu_ops.CpuStore(experts), n_exp, ops=cpu_ops)
    hidden = synth.tokens(n_tok, d_model, seed=5)
    logits = synth.router_logits(n_tok, n_exp, seed=6)
    out, _ = layer(hidden, router_logits=logits)
    ref = reference_moe(hidden.unsqueeze(0), logits.unsqueeze(0), experts, 1024)[0]
    assert float((out.float() - ref.float()).abs().max() / ref.float().abs().max()) <= 1e-2
