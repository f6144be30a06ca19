"""Worker of tests/test_gpu_ep.py, one process per GPU under torch.distributed.run: the expert-parallel block in
one launch per rank (zmlx_b200.ep.PeerMoELayer) against the one-GPU block on the same tokens and against the CPU
oracle.  Prints one JSON line per rank."""

import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import numpy as np  # noqa: E402
import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

from tests.helpers import oracle_layer, t2n  # noqa: E402
from zmlx_b200 import ep, synthetic  # noqa: E402
from zmlx_b200.layer import MoELayer  # noqa: E402


def main() -> None:
    name, T = sys.argv[1], int(sys.argv[2])
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    cfg = synthetic.CONFIGS[name]
    full = synthetic.make_layer(cfg, device=dev)  # same seed on every rank: one model
    lo, hi = ep.expert_range(cfg.n_experts, world, rank)
    peer = ep.PeerMoELayer(cfg, ep.shard_params(full, lo, hi), rank=rank, world=world, tokens=T)
    one = MoELayer(cfg, full, max_tokens=8)
    rec = {"rank": rank, "steps": []}
    for step in range(4):  # both launch parities, twice
        x = synthetic.make_tokens(cfg, T, step=10 * step + rank).to(dev)  # every rank brings its own tokens
        got = peer(x).clone()
        want = one(x).clone()
        torch.cuda.synchronize()
        peer.check_status()
        rms = float(want.float().pow(2).mean().sqrt())
        item = {"indices_equal": bool(torch.equal(peer.indices[:T], one.indices[:T])),
                "weights_equal": bool(torch.equal(peer.weights[:T], one.weights[:T])),
                "max_err_over_rms": float((got.float() - want.float()).abs().max()) / max(rms, 1e-30),
                "equal_frac": float((got == want).float().mean())}
        if step == 0:
            ref, _ = oracle_layer(cfg, full, x, one.router_logits(T), peer.indices[:T])
            item["oracle_err_over_rms"] = float(np.abs(t2n(got) - ref).max() / max(float(np.sqrt((ref ** 2).mean())), 1e-30))
        rec["steps"].append(item)
    dist.barrier()
    peer.close()
    print("EPREC " + json.dumps(rec), flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
