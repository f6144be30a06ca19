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


# ------------------------------------------------------------------------------------------------------------------
# The one-launch expert-parallel block exchanges rows by peer stores into per-rank inboxes (no collective).  Its
# host-visible protocol -- inbox layout, launch parities, tagged words, home rows, bounded polls -- is restated
# here with shared-memory tensors standing in for peer-mapped device memory and the oracle for the kernels.

_POLL_LIMIT_S = 1.0


def _poll(inbox: torch.Tensor, lo: int, n: int, launch: int):
    """The kernel's bounded wait: poll until every word of the range carries this launch's tag, at most a second."""
    import time
    t0 = time.monotonic()
    while True:
        ok, rows = ep.unpack_words(inbox[lo:lo + n], launch)
        if ok:
            return rows
        if time.monotonic() - t0 > _POLL_LIMIT_S:
            return None
        time.sleep(0.001)


def _peer_worker(rank: int, world: int, port: int, T: int, inboxes, silent_rank: int, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.set_num_threads(1)
        cfg = synthetic.CONFIGS["c2"].scaled(n_experts=8, d_model=128, d_ff=64, top_k=2)
        d, K = cfg.d_model, cfg.top_k
        params = synthetic.make_layer(cfg)
        lo, hi = ep.expert_range(cfg.n_experts, world, rank)
        local, full = params_to_numpy(ep.shard_params(params, lo, hi)), params_to_numpy(params)
        lay = ep.inbox_layout(T, world, d, K)
        status, good = 0, True
        for launch in range(3):  # both launch parities, and a tag that differs from the one two launches before
            par = launch & 1
            x = synthetic.make_tokens(cfg, T, step=10 * launch + rank)
            if rank != silent_rank:
                # ---- own token rows -> row rank * T + t of the token part of every rank's inbox
                words = ep.pack_words(x, launch).reshape(-1)
                for r in range(world):
                    o = lay["x"][par] + rank * T * d
                    inboxes[r][o:o + T * d] = words
            # ---- wait for the token rows of every rank (bounded)
            rows = _poll(inboxes[rank], lay["x"][par], T * world * d, launch)
            if rows is None:
                status = -6  # ZMOE_ERR_TIMEOUT: the kernel sets the status word and returns
                break
            xn = t2n(rows.reshape(T * world, d))
            logits = S.bf16(xn @ full["router_w"].T)
            idx, w = S.qwen3_gating(logits, K)
            # ---- local experts only; each projected row goes to its home rank's inbox as tagged words
            for row in range(T * world * K):
                e = int(idx.reshape(-1)[row])
                if not (lo <= e < hi):
                    continue
                lhs = np.array([row // K], dtype=np.int32)
                rhs = np.array([e - lo], dtype=np.int32)
                g = F.gather_qmm_rows(xn, local["gate_w"], local["gate_s"], local["gate_b"], lhs, rhs)
                u = F.gather_qmm_rows(xn, local["up_w"], local["up_s"], local["up_b"], lhs, rhs)
                h = F.swiglu_cpu_contract(g, u)
                y = F.gather_qmm_rows(h, local["down_w"], local["down_s"], local["down_b"],
                                      np.zeros(1, dtype=np.int32), rhs)
                home, hrow = ep.home_of_row(row, T, K)
                o = lay["y"][par] + hrow * d
                inboxes[home][o:o + d] = ep.pack_words(torch.from_numpy(y).to(torch.bfloat16), launch).reshape(-1)
            # ---- the home rank combines its own tokens' rows as they arrive
            yrows = _poll(inboxes[rank], lay["y"][par], T * K * d, launch)
            if yrows is None:
                status = -6
                break
            out = S.moe_combine(t2n(yrows.reshape(T, K, d)), w[rank * T:(rank + 1) * T], mode="no_fma")
            ref, idx1, _ = S.moe_layer(t2n(x), logits[rank * T:(rank + 1) * T], full, family="qwen3", top_k=K)
            good = good and bool(np.array_equal(out, ref)) and bool(np.array_equal(idx1, idx[rank * T:(rank + 1) * T]))
        ret[rank] = (status, good)
    finally:
        dist.destroy_process_group()


def _run_peer(T: int, silent_rank: int):
    world = 2
    cfg = synthetic.CONFIGS["c2"].scaled(n_experts=8, d_model=128, d_ff=64, top_k=2)
    lay = ep.inbox_layout(T, world, cfg.d_model, cfg.top_k)
    inboxes = [torch.zeros(lay["words"], dtype=torch.int64).share_memory_() for _ in range(world)]
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    port = _free_port()
    procs = [ctx.Process(target=_peer_worker, args=(r, world, port, T, inboxes, silent_rank, ret)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=180)
        assert p.exitcode == 0
    return dict(ret)


@pytest.mark.parametrize("T", [1, 2])
def test_peer_store_exchange_protocol_world2(T):
    """Every rank's result equals the single-process oracle block bit for bit, over three launches."""
    assert _run_peer(T, silent_rank=-1) == {0: (0, True), 1: (0, True)}


def test_peer_store_exchange_reports_a_rank_that_never_posts():
    """Failure made on the host: rank 1 pushes no token rows.  Rank 0's bounded wait runs out and it reports the
    time-out status instead of hanging; rank 1 itself sees its own rows missing too (it reads them from its inbox
    like everyone else's)."""
    got = _run_peer(1, silent_rank=1)
    assert got[0][0] == -6 and got[1][0] == -6


def test_inbox_layout_and_home_rows():
    lay = ep.inbox_layout(2, 4, 64, 8)
    assert lay["x"] == [0, 2 * 4 * 64] and lay["y"][0] == 2 * lay["x"][1]
    assert lay["words"] * 4 == lay["bytes"]
    assert ep.home_of_row(0, 2, 8) == (0, 0) and ep.home_of_row(8 * 2 + 3, 2, 8) == (1, 3)
    assert ep.home_of_row(8 * 3 + 7, 2, 8) == (1, 15)
    assert ep.launch_tag(0) == 1 << 16 and ep.launch_tag(65535) == 1 << 16 and ep.launch_tag(2) != ep.launch_tag(0)
