"""Spawns the multi-GPU fused-kernel checks when at least two GPUs are visible."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(script, nproc, extra_env=None, timeout=600):
    env = dict(os.environ)
    env.update(extra_env or {})
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
           "--master-addr", "127.0.0.1", "--master-port", "29541", script]
    return subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=timeout)


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2,
                    reason="needs >= 2 GPUs")
@pytest.mark.parametrize("tp_pair", ["1", "0"])
def test_fused_collective_kernels_match_nccl(tp_pair):
    """``tp_pair``: the tensor-parallel kernels on the CTA-pair GEMM body (default) or on the one-CTA body."""
    n = min(torch.cuda.device_count(), 4)
    r = _run(os.path.join(ROOT, "tests", "multi_gpu", "fused_checks.py"), n,
             {"RB_TP_PAIR": tp_pair, "RB_TP_PAIR_RS": tp_pair, "RB_TP_PAIR_MAX_WORLD": "8"})
    assert r.returncode == 0, r.stdout[-4000:] + r.stderr[-4000:]
    assert "ALL FUSED CHECKS PASSED" in r.stdout


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2,
                    reason="needs >= 2 GPUs")
def test_context_parallel_attention_matches_full_sequence():
    n = min(torch.cuda.device_count(), 4)
    r = _run(os.path.join(ROOT, "tests", "multi_gpu", "cp_checks.py"), n)
    assert r.returncode == 0, r.stdout[-4000:] + r.stderr[-4000:]
    assert "ALL CP CHECKS PASSED" in r.stdout


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2,
                    reason="needs >= 2 GPUs")
def test_fsdp_reshard_after_forward_matches_resident_flow():
    n = min(torch.cuda.device_count(), 4)
    r = _run(os.path.join(ROOT, "tests", "multi_gpu", "reshard_checks.py"), n)
    assert r.returncode == 0, r.stdout[-4000:] + r.stderr[-4000:]
    assert "ALL RESHARD CHECKS PASSED" in r.stdout
