"""Run by tests/test_gpu_variants.py in a child process: the kernel variant is chosen by an environment variable
that libzmoe reads once per process.  Compares one MoE block against the separate-kernel path of a second layer
object in the same process (which the parent suite checks against the oracle) and prints one JSON line."""

import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402

from zmlx_b200 import synthetic  # noqa: E402
from zmlx_b200.layer import MoELayer  # noqa: E402


def main() -> None:
    name, T, fused = sys.argv[1], int(sys.argv[2]), sys.argv[3] == "fused"
    dev = "cuda:0"
    cfg = synthetic.CONFIGS[name]
    params = synthetic.make_layer(cfg, device=dev)
    x = synthetic.make_tokens(cfg, T, device="cpu").to(dev)
    a = MoELayer(cfg, params, max_tokens=max(T, 8), fused=fused)
    out = a(x).clone()
    again = a(x).clone()
    torch.cuda.synchronize()  # a launch whose waits ran out must still end and leave the context usable
    usable = bool((torch.arange(8, device=dev) + 1).sum().item() == 36)
    rec = {"finite": bool(torch.isfinite(out.float()).all()), "repeatable": bool(torch.equal(out, again)),
           "status": a.fused_status(T) if fused else 0, "context_usable": usable,
           "out": out.float().cpu().flatten().tolist(), "indices": a.indices[:T].cpu().flatten().tolist()}
    print(json.dumps(rec))


if __name__ == "__main__":
    main()
