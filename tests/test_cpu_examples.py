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


def test_launcher_trains_checkpoints_and_resumes_with_fewer_ranks(tmp_path):
    """python -m rumus_b200.launch: 2 gloo ranks write checkpoints, 1 rank resumes from the newest
    verified one (re-sharded optimizer state) and finishes; metrics land in JSONL files."""
    import json
    ck, met = str(tmp_path / "ck"), str(tmp_path / "metrics")
    r = _run(["-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
              "--master-port", "29633", "-m", "rumus_b200.launch", "--config", "tiny-decoder-cpu",
              "--steps", "12", "--ckpt-dir", ck, "--ckpt-every", "6", "--metrics-dir", met, "--log-every", "3"])
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-3000:]
    out = json.loads([l for l in r.stdout.splitlines() if l.startswith("{")][-1])
    assert out["steps"] == 12 and out["world"] == 2 and out["mode"] == "cpu"
    assert sorted(os.listdir(ck)) == ["step-12", "step-6"]
    assert sorted(os.listdir(met)) == ["metrics-rank0.jsonl", "metrics-rank1.jsonl"]
    r = _run(["-m", "rumus_b200.launch", "--config", "tiny-decoder-cpu", "--steps", "18", "--ckpt-dir", ck,
              "--resume", "--log-every", "3"])
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-3000:]
    out2 = json.loads([l for l in r.stdout.splitlines() if l.startswith("{")][-1])
    assert out2["resumed_from"].endswith("step-12") and out2["steps"] == 18 and out2["world"] == 1
    assert out2["last_loss"] < out["first_logged_loss"]


def test_launcher_vision_config_from_yaml(tmp_path):
    import json
    cfg = tmp_path / "small_resnet.yaml"
    cfg.write_text("name: small-resnet\n"
                   "model: {family: resnet50, kwargs: {num_classes: 10, layers: [1, 1, 1, 1], width: 8}}\n"
                   "precision: {compute: fp32, master_weights: false, loss_scaling: true, init_scale: 128.0}\n"
                   "optimizer: sgd\nlr: 0.05\nmomentum: 0.9\nseqs_per_gpu: 2\nsteps: 3\n")
    r = _run(["-m", "rumus_b200.launch", "--config", str(cfg), "--image-size", "32", "--log-every", "1"])
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-3000:]
    out = json.loads([l for l in r.stdout.splitlines() if l.startswith("{")][-1])
    assert out["family"] == "resnet50" and out["steps"] == 3 and out["last_loss"] == out["last_loss"]


def test_launcher_llama_tp2_pp2_on_four_gloo_ranks(tmp_path):
    import json
    cfg = tmp_path / "llama_small.yaml"
    cfg.write_text("name: llama-small\n"
                   "model: {family: llama, kwargs: {vocab_size: 64, seq_len: 16, d_model: 32, num_heads: 2, "
                   "num_kv_heads: 2, num_layers: 2, ffn_dim: 64}}\n"
                   "parallel: {tp: 2, pp: 2, micro_batches: 2, backend: nccl}\n"
                   "precision: {compute: fp32, master_weights: false}\n"
                   "lr: 0.01\nglobal_batch: 4\nsteps: 12\n")
    dense = str(tmp_path / "out" / "model.safetensors")
    r = _run(["-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=4", "--master-addr", "127.0.0.1",
              "--master-port", "29635", "-m", "rumus_b200.launch", "--config", str(cfg), "--log-every", "4",
              "--export-dense", dense], timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-3000:]
    out = json.loads([l for l in r.stdout.splitlines() if l.startswith("{")][-1])
    assert out["parallelism"] == "tp2xpp2xdp1" and out["steps"] == 12
    assert out["last_loss"] < out["first_logged_loss"]
    assert abs(out["bubble_fraction_ideal"] - 1 / 3) < 1e-9
    from rumus_b200.io import load_safetensors
    sd = load_safetensors(dense)
    assert sd["blocks.1.mlp.down_proj.weight"].shape == (64, 32) and sd["head.weight"].shape == (32, 64)
