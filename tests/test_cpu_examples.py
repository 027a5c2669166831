"""The scripts under examples/ run as written (CPU), including a 2-rank gloo FSDP job."""
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(args, timeout=300):
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="", OMP_NUM_THREADS="2")
    return subprocess.run([sys.executable] + args, cwd=ROOT, env=env, capture_output=True, text=True,
                          timeout=timeout)


@pytest.mark.parametrize("script,expect", [
    ("examples/xor_mlp.py", "checkpoint round trip: exact"),
    ("examples/tiny_gpt.py", "final cross-entropy"),
    ("examples/int4_and_onnx.py", "bytes of ONNX"),
    ("examples/fsdp_gpt.py", "local mode, world 1"),
])
def test_example_runs(script, expect):
    r = _run([script])
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-3000:]
    assert expect in r.stdout


def test_fsdp_example_on_two_gloo_ranks():
    r = _run(["-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
              "--master-port", "29631", "examples/fsdp_gpt.py"])
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-3000:]
    assert "cpu mode, world 2" in r.stdout
    first = float(r.stdout.split("step 0: loss ")[1].split()[0])
    last = float(r.stdout.split("step 25: loss ")[1].split()[0])
    assert last < first
