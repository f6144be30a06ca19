"""Kernel variants that an environment variable selects once per process (the opt-in bulk-copy streaming matmul,
the bulk-copy form of the one-launch block): each runs in a child process and must agree with the default path of
this process, which the rest of the suite checks against the oracle."""

import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from tests.helpers import assert_close_rel, t2n
from zmlx_b200 import synthetic
from zmlx_b200.layer import MoELayer

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))
DEV = "cuda:0"


def _child(env: dict, name: str, T: int, mode: str) -> dict:
    full = dict(os.environ)
    full.update(env)
    res = subprocess.run([sys.executable, os.path.join(HERE, "variant_check.py"), name, str(T), mode],
                         capture_output=True, text=True, env=full, timeout=600)
    assert res.returncode == 0, res.stderr[-2000:]
    return json.loads(res.stdout.strip().splitlines()[-1])


def _reference(name: str, T: int):
    cfg = synthetic.CONFIGS[name]
    layer = MoELayer(cfg, synthetic.make_layer(cfg, device=DEV), max_tokens=max(T, 8), fused=False)
    out = layer(synthetic.make_tokens(cfg, T, device="cpu").to(DEV)).clone()
    return t2n(out), layer.indices[:T].cpu().numpy().flatten()


@pytest.mark.parametrize("env,name,T,mode", [
    ({"ZMOE_LD_BULK": "1"}, "c2", 1, "fused"),
    ({"ZMOE_LD_BULK": "1"}, "c1", 1, "fused"),
    ({"ZMOE_LD_BULK": "0", "ZMOE_LD_NO_BULK": "1"}, "c2", 1, "fused"),
    ({"ZMOE_STREAM": "1"}, "c2", 1, "separate"),
])
def test_variant_agrees_with_the_default_kernels(env, name, T, mode):
    rec = _child(env, name, T, mode)
    assert rec["finite"] and rec["repeatable"] and rec["status"] == 0
    want, idx = _reference(name, T)
    assert np.array_equal(np.asarray(rec["indices"]), idx)
    got = np.asarray(rec["out"], dtype=np.float32).reshape(want.shape)
    assert_close_rel(got, want, 2e-2, f"{name} T={T} {env}")


def test_a_wait_that_runs_out_ends_the_launch_with_the_status_word_set():
    """Failure detection without a GPU fault: with ZMOE_LD_TEST_WITHHOLD=1 one router logit is never published, so
    every CTA's bounded wait for it runs out; the launch must end by itself (about a second), report it in the
    workspace's status word and leave the CUDA context usable."""
    rec = _child({"ZMOE_LD_TEST_WITHHOLD": "1"}, "c2", 1, "fused")
    assert rec["status"] == 1
    assert rec["context_usable"]
