"""The configuration entry points (Llama depth-sharded + pruning, Mixtral expert parallel, VGG-16 pipeline)
run end to end on CPU ranks at tiny scale."""

import json
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("config,port", [("llama8b_depth", 29701), ("mixtral_ep", 29702), ("vgg16_pp", 29703)])
def test_config_entry_point_tiny(config, port):
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "4", "--master-addr",
           "127.0.0.1", "--master-port", str(port), os.path.join(ROOT, "examples", "run_config.py"), "--config", config,
           "--scale", "tiny", "--steps", "2", "--warmup", "1"]
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="")
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    line = [ln for ln in r.stdout.splitlines() if ln.startswith("{")][-1]
    out = json.loads(line)
    assert out["config"] == config and out["value"] > 0 and out["loss"] == out["loss"]
