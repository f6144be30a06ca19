"""CPU, world size 2 over gloo: host logic of the expert-parallel layer (partition, token all-gather, local
index remap, exact reduce-scatter of per-slot rows, ordered combine) with the oracle standing in for the kernels.
The result of every rank must equal the single-process oracle layer bit for bit."""

import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import fast as F
from oracle import semantics as S
from tests.helpers import params_to_numpy, t2n
from zmlx_b200 import ep, synthetic


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, T: int, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.set_num_threads(1)
        cfg = synthetic.CONFIGS["c2"].scaled(n_experts=8, d_model=128, d_ff=64, top_k=2)
        params = synthetic.make_layer(cfg)  # same seed on every rank: replicated model
        lo, hi = ep.expert_range(cfg.n_experts, world, rank)
        local = params_to_numpy(ep.shard_params(params, lo, hi))
        full = params_to_numpy(params)
        x = synthetic.make_tokens(cfg, T, step=rank)  # every rank brings its own tokens
        x_all = ep.gather_tokens(x, world)
        assert x_all.shape == (world * T, cfg.d_model)
        xn = t2n(x_all)
        logits = S.bf16(xn @ full["router_w"].T)
        idx, w = S.qwen3_gating(logits, cfg.top_k)
        li = t2n(ep.localize_indices(torch.from_numpy(idx.astype(np.int32)), lo, hi))
        assert ((li >= 0) == ((idx >= lo) & (idx < hi))).all()
        # local experts only; rows of non-local pairs stay zero
        TA, K = idx.shape
        y = np.zeros((TA * K, cfg.d_model), dtype=np.float32)
        sel = np.nonzero(li.reshape(-1) >= 0)[0]
        if sel.size:
            lhs = (sel // K).astype(np.int32)
            rhs = li.reshape(-1)[sel]
            g = F.gather_qmm_rows(xn, local["gate_w"], local["gate_s"], local["gate_b"], lhs, rhs)
            u = F.gather_qmm_rows(xn, local["up_w"], local["up_s"], local["up_b"], lhs, rhs)
            h = F.swiglu_cpu_contract(g, u)
            y[sel] = F.gather_qmm_rows(h, local["down_w"], local["down_s"], local["down_b"],
                                       np.arange(sel.size, dtype=np.int32), rhs)
        y_mine = ep.exchange_slot_rows(torch.from_numpy(y).to(torch.bfloat16), world)
        out = S.moe_combine(t2n(y_mine).reshape(T, K, -1), w[rank * T:(rank + 1) * T], mode="no_fma")
        # single-process oracle on this rank's own tokens
        ref, idx1, w1 = S.moe_layer(t2n(x), logits[rank * T:(rank + 1) * T], full, family="qwen3", top_k=cfg.top_k)
        ret[rank] = bool(np.array_equal(out, ref) and np.array_equal(idx1, idx[rank * T:(rank + 1) * T]))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("T", [1, 3])
def test_expert_parallel_host_logic_world2(T):
    world = 2
    port = _free_port()
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    procs = [ctx.Process(target=_worker, args=(r, world, port, T, ret)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    assert dict(ret) == {0: True, 1: True}


def test_partition_helpers():
    assert ep.expert_range(128, 8, 3) == (48, 64)
    with pytest.raises(ValueError):
        ep.expert_range(10, 4, 0)
    idx = torch.tensor([[0, 5, 7, 2]], dtype=torch.int32)
    assert ep.localize_indices(idx, 4, 8).tolist() == [[-1, 1, 3, -1]]
