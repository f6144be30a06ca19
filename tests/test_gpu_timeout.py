"""Failure detection of the one-launch block without a GPU fault: a wait that cannot be satisfied must run out,
end the launch by itself, be reported through the workspace's status word and leave the CUDA context usable."""

import json
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

_CHILD = r"""
import json, sys
sys.path.insert(0, {root!r})
import torch
from zmlx_b200 import _lib, synthetic
from zmlx_b200.layer import MoELayer

dev = "cuda:0"
cfg = synthetic.CONFIGS["c2"]
params = synthetic.make_layer(cfg, device=dev)
x = synthetic.make_tokens(cfg, 1, device="cpu").to(dev)
# debug hook: expert 0's router logit is never published, so every CTA's bounded wait for it runs out
bad = MoELayer(cfg, params, max_tokens=8, fused=True, debug_withhold_logit=True)
bad(x)
torch.cuda.synchronize()  # the launch must end by itself (about a second)
status = bad.fused_status(1)
raised = False
try:
    bad.check_status()
except _lib.ZmoeError as e:
    raised = e.code == _lib.ERR_TIMEOUT
cleared = bad.fused_status(1) == 0
# the context is still usable, and a healthy layer on the same device still gives finite results
usable = bool((torch.arange(8, device=dev) + 1).sum().item() == 36)
good = MoELayer(cfg, params, max_tokens=8, fused=True)
out = good(x)
good.check_status()
print(json.dumps({{"status": status, "raised": raised, "cleared": cleared, "usable": usable,
                  "finite": bool(torch.isfinite(out.float()).all())}}))
"""


def test_a_wait_that_runs_out_ends_the_launch_with_the_status_word_set():
    res = subprocess.run([sys.executable, "-c", _CHILD.format(root=ROOT)], capture_output=True, text=True,
                         timeout=600)
    assert res.returncode == 0, res.stderr[-2000:]
    rec = json.loads(res.stdout.strip().splitlines()[-1])
    assert rec["status"] == 1
    assert rec["raised"], "check_status() must map the status word to ZMOE_ERR_TIMEOUT"
    assert rec["cleared"] and rec["usable"] and rec["finite"]
