"""Tensor-parallel batch-1 decode on 2 GPUs (skipped where fewer are visible): the frames of
the sharded run must equal the single-GPU frames code for code, greedy and sampled."""
import json
import os
import socket
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


def _gpus():
    import torch
    return torch.cuda.device_count()


def run_tp(world, mode, n_slow, frames, prompt=64):
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    out = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(world),
                          "--master-addr", "127.0.0.1", "--master-port", str(port), os.path.join(HERE, "tp_parity_worker.py"),
                          mode, str(n_slow), str(frames), str(prompt)], capture_output=True, text=True, env=env, timeout=1500)
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-4000:]
    line = [l for l in out.stdout.splitlines() if l.startswith("RESULT ")][-1]
    return json.loads(line[len("RESULT "):])


@pytest.mark.parametrize("mode", ["int4", "int8"])
def test_tp2_two_layer_equals_single_gpu(mode):
    if _gpus() < 2:
        pytest.skip("needs 2 GPUs")
    res = run_tp(2, mode, 2, 24)
    for tag, r in res["runs"].items():
        assert r["persistent"] == 1 and r["single_persistent"] == 1, tag
        assert r["ranks_agree"], tag
        assert r["frames_tp"] == r["frames_single"] and r["frames_identical"] == r["frames_single"], (tag, r)
