"""CUDA-graph replay helpers: a captured step and the double-buffered host-to-host pipeline."""
import pytest
import torch

from qmoe_b200.graph import GraphedStep, PipelinedStep

pytestmark = pytest.mark.gpu


def test_pipelined_step_returns_every_result_in_order():
    dev = torch.device("cuda", 0)
    weight = torch.arange(1, 65, dtype=torch.float32, device=dev)

    def fn(x):
        y = x * weight
        for _ in range(20):                       # long enough for copies to overlap it
            y = y + torch.tanh(x) * 0.0
        return y + 1.0

    example = torch.zeros(4096, 64, device=dev)
    g = GraphedStep(fn, example)
    pipe = PipelinedStep(g)
    ins = [torch.full((4096, 64), float(i), dtype=torch.float32).pin_memory() for i in range(7)]
    outs = [torch.empty(4096, 64, dtype=torch.float32).pin_memory() for _ in range(7)]
    for i in range(7):
        pipe.submit(ins[i], outs[i])
    pipe.drain()
    torch.cuda.synchronize(dev)
    for i in range(7):
        assert torch.equal(outs[i], ins[i] * weight.cpu() + 1.0), i
    # a second batch through the same object, same host output buffer every step
    out = torch.empty(4096, 64, dtype=torch.float32).pin_memory()
    for i in range(5):
        ev = pipe.submit(ins[i], out)
    ev.synchronize()
    assert torch.equal(out, ins[4] * weight.cpu() + 1.0)
    g.close()
