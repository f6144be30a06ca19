"""GPU checks of the expert-parallel layer's single-rank form (no collectives): with one rank it owns every
expert, so it must reproduce the plain layer bit for bit -- eagerly and with the kernels between the two
collectives replayed from a CUDA graph."""

import pytest
import torch

from zmlx_b200 import synthetic
from zmlx_b200.ep import EPMoELayer
from zmlx_b200.layer import MoELayer

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.mark.parametrize("name,T,graphs", [("c2", 1, False), ("c2", 1, True), ("c2", 8, True), ("c1", 3, True)])
def test_single_rank_expert_parallel_layer_equals_the_plain_layer(name, T, graphs):
    cfg = synthetic.CONFIGS[name]
    params = synthetic.make_layer(cfg, device=DEV)
    plain = MoELayer(cfg, params, max_tokens=8, fused=False)
    ep = EPMoELayer(cfg, params, rank=0, world=1, max_tokens=8, segment_graphs=graphs)
    side = torch.cuda.Stream(device=DEV)
    for step in range(4):  # pass 0 eager, pass 1 captures, passes 2-3 replay
        x = synthetic.make_tokens(cfg, T, step=step, device="cpu").to(DEV)
        want = plain(x).clone()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            got = ep(x).clone()
        torch.cuda.current_stream().wait_stream(side)
        assert torch.equal(got, want), f"step {step}"
    assert (len(ep._graphs) == 1) == graphs
