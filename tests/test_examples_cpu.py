"""The configuration entry points (Llama depth-sharded + pruning, Mixtral expert parallel, VGG-16 pipeline)
run end to end on CPU ranks at tiny scale, and so do the two tutorial scripts: a tensor-parallel MLP that is
stopped and continued on another grid, and a pipelined ViT that has to converge."""

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


def _torchrun(nproc, port, script, *args, env=None):
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(nproc),
           "--master-addr", "127.0.0.1", "--master-port", str(port), os.path.join(ROOT, "examples", script), *args]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=900,
                       env=dict(os.environ, CUDA_VISIBLE_DEVICES="", **(env or {})))
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    return json.loads([ln for ln in r.stdout.splitlines() if ln.startswith("{")][-1])


def test_tensor_parallel_tutorial_continues_on_another_grid(tmp_path):
    folder = str(tmp_path / "ckpt")
    a = _torchrun(4, 29711, "train_mlp_tensor_parallel.py", "--G-intra-r", "2", "--G-intra-d", "2", "--steps", "30",
                  "--save", folder)
    assert a["steps"] == 30 and a["last_loss"] < 0.75 * a["first_loss"]
    b = _torchrun(2, 29712, "train_mlp_tensor_parallel.py", "--G-intra-c", "2", "--steps", "30", "--resume", folder)
    assert b["first_step"] == 30 and b["steps"] == 60
    # no restart bump: the continued run starts about where the first one stopped and keeps improving
    assert b["first_loss"] < 1.1 * a["last_loss"] and b["last_loss"] < a["last_loss"]


def test_pipelined_vit_tutorial_converges():
    out = _torchrun(4, 29713, "train_vit_pipeline.py", env={"G_inter": "2", "G_data": "2"})
    assert out["steps"] == 32 and out["final_loss"] < 0.1 < out["first_loss"]


def test_language_model_example_learns_a_text_file(tmp_path):
    corpus = tmp_path / "corpus.txt"
    corpus.write_text("the quick brown fox jumps over the lazy dog. pack my box with five dozen liquor jugs. " * 300)
    out = _torchrun(4, 29714, "train_lm.py", "--G-intra-r", "2", "--G-intra-d", "2", "--data", str(corpus), "--steps",
                    "30", "--seq-len", "64")
    assert out["vocab"] == 256 and out["steps"] == 30 and out["last_loss"] < 0.3 * out["first_loss"]


def test_token_windows():
    import numpy as np
    import torch

    from axonn_b200.utils.data import TokenWindows, load_tokens

    stream = np.arange(103, dtype=np.int64)
    ds = TokenWindows(stream, seq_len=10)
    assert len(ds) == 10                                    # windows of 11 tokens starting every 10
    x, y = ds[9]
    assert x.tolist() == list(range(90, 100)) and y.tolist() == list(range(91, 101)) and x.dtype == torch.long
    assert len(TokenWindows(stream, seq_len=10, stride=1)) == 93
    with pytest.raises(ValueError):
        TokenWindows(stream, seq_len=10, vocab=100)         # id 102 does not fit
    with pytest.raises(ValueError):
        TokenWindows(stream[:5], seq_len=10)
    with pytest.raises(IndexError):
        ds[10]


def test_load_tokens_formats(tmp_path):
    import numpy as np

    from axonn_b200.utils.data import load_tokens

    ids = np.array([1, 500, 65535, 7], dtype=np.uint16)
    ids.tofile(tmp_path / "a.bin")
    np.save(tmp_path / "a.npy", ids.astype(np.int32).reshape(2, 2))
    (tmp_path / "a.txt").write_bytes(b"abc")
    assert load_tokens(str(tmp_path / "a.bin")).tolist() == ids.tolist()
    assert load_tokens(str(tmp_path / "a.npy")).tolist() == ids.tolist()
    assert load_tokens(str(tmp_path / "a.txt")).tolist() == [97, 98, 99]
