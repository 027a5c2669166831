#!/usr/bin/env python
"""Headline benchmark: GPT-style 1.3B FSDP training throughput (tokens/s over the whole job).

  python bench.py --gpus N --steps K --warmup W            (N = 1)
  python -m torch.distributed.run --nproc-per-node N ... bench.py --gpus N --steps K --warmup W

Model/config: 24 layers, d_model 2048, 16 heads, FFN 8192 GELU, vocab 50304, seq 2048, 8 sequences
per GPU, bf16 compute with fp32 master weights + Adam moments, FlashAttention, FSDP over N GPUs
(weak scaling).  Synthetic uniform-random tokens from a seed, random-init weights.

Two measurements, both over exactly K optimizer steps after W warm-up steps, bracketed by a
barrier + device synchronize, timed with CUDA events, max over ranks:
  * value : inputs already on the device (kernel-side throughput);
  * e2e   : through the public API, every step copies that step's tokens from pinned host memory
            and reads the loss back to the host.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def reference_arm(args):
    print(json.dumps({
        "impl": "reference",
        "unavailable": "reference is a Rust/WGSL cargo workspace: pip install finds no setup.py/pyproject, "
                       "no cargo/rustc offline, and its wgpu GPU path needs a graphics stack that is "
                       "unavailable on this box"}))
    return 0


class ClockSampler:
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device_index: int):
        self.proc = None
        self.idx = device_index
        self.path = f"/tmp/rb_clocks_{os.getpid()}.csv"

    def start(self):
        try:
            self.f = open(self.path, "w")
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-lms", "200", "-i", str(self.idx)], stdout=self.f, stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        self.f.close()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        try:
            for line in open(self.path):
                parts = [x.strip() for x in line.split(",")]
                if len(parts) < 9:
                    continue
                try:
                    sm.append(float(parts[1])); mx.append(float(parts[2]))
                except ValueError:
                    continue
                for n, v in zip(names, parts[5:9]):
                    if v.lower().startswith("active"):
                        reasons.add(n)
            os.unlink(self.path)
        except Exception:
            pass
        if sm:
            hi = [x for x in sm if x >= 0.5 * max(sm)]
            out["sm_mhz"] = statistics.median(hi)
            out["sm_max_mhz"] = max(mx)
            out["samples"] = len(sm)
        out["reasons"] = sorted(reasons)
        return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=8)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours")
    ap.add_argument("--mode", default=None, help="fused | nccl (multi-GPU communication path)")
    ap.add_argument("--reshard", action="store_true",
                    help="FSDP keeps only parameter shards between a block's forward and backward")
    ap.add_argument("--phases", action="store_true", help="also report forward/backward/tail device times")
    ap.add_argument("--trace-export", default=None,
                    help="write a torch.profiler Chrome trace of two extra steps (with the NVTX-named "
                         "ranges of the fused paths) to this path")
    ap.add_argument("--kernel-profile", action="store_true",
                    help="after the timed runs, print a per-kernel breakdown of two extra steps (stderr)")
    ap.add_argument("--layers", type=int, default=None, help="debug only: invalidates the number")
    ap.add_argument("--seqs-per-gpu", type=int, default=8)
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm(args)
    args.warmup = max(args.warmup, 3)

    import torch
    import torch.distributed as dist
    from rumus_b200.models import GPT, GPTConfig
    from rumus_b200.ops import _lib, native
    from rumus_b200.parallel import FSDP

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    assert world == args.gpus, f"--gpus {args.gpus} but WORLD_SIZE={world}"
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)

    cfg = GPTConfig.gpt_1p3b()
    if args.layers:
        cfg.num_layers = args.layers
    B, S = args.seqs_per_gpu, cfg.seq_len
    torch.manual_seed(1234)
    model = GPT(cfg, device=dev, dtype=torch.bfloat16)
    model.init_weights(0.02, seed=0)
    native.lib().rb_init_device()
    engine = FSDP(model, lr=1e-4, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.0, adamw=False,
                  mode=args.mode, reshard_after_forward=args.reshard)

    gen = torch.Generator(device="cpu").manual_seed(1000 + rank)
    n_batches = args.warmup + args.steps
    host_tokens = [torch.randint(0, cfg.vocab_size, (B, S + 1), generator=gen).pin_memory()
                   for _ in range(n_batches)]

    def train_step_device(tok):
        engine.zero_grad()
        loss = model(tok[:, :-1], tok[:, 1:])
        loss.backward()
        engine.step()
        return loss

    def train_step_e2e(tok_host):
        """Public-API step: pinned host tokens in, host float loss out."""
        tok = tok_host.to(dev, non_blocking=True)
        loss = train_step_device(tok)
        return float(loss.item())

    def sync_all():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, batches):
        sync_all()
        sampler = ClockSampler(local_rank) if rank == 0 else None
        if sampler:
            sampler.start()
        _lib.reset_launch_count()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        last = None
        for b in batches:
            last = fn(b)
        e1.record()
        sync_all()
        ms = e0.elapsed_time(e1)
        launches = _lib.launch_count()
        clocks = sampler.stop() if sampler else None
        t = torch.tensor([ms], device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item()), launches, clocks, last

    # ---- device-resident inputs ----
    dev_tokens = [t.to(dev) for t in host_tokens]
    for i in range(args.warmup):
        train_step_device(dev_tokens[i])
    ms, launches, clocks, last_loss = timed(train_step_device, dev_tokens[args.warmup:])
    status = native.read_status()
    tokens = world * B * S * args.steps
    value = tokens / (ms / 1e3)
    # ---- end to end (H2D tokens + D2H loss every step) ----
    train_step_e2e(host_tokens[0])
    ms_e2e, _, _, last_e2e = timed(train_step_e2e, host_tokens[args.warmup:])
    e2e_value = tokens / (ms_e2e / 1e3)

    phases = None
    if args.phases:
        # per-phase device times of a few extra steps (forward / backward / optimizer+comm tail)
        acc = [0.0, 0.0, 0.0]
        n_ph = 3
        for i in range(n_ph):
            ev = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
            sync_all()
            tok = dev_tokens[args.warmup + i % max(1, args.steps)]
            engine.zero_grad()
            if i == n_ph - 1 and world > 1 and hasattr(engine, "start_trace"):
                engine.start_trace()
            ev[0].record()
            loss = model(tok[:, :-1], tok[:, 1:])
            ev[1].record()
            loss.backward()
            ev[2].record()
            engine.step()
            ev[3].record()
            torch.cuda.synchronize()
            for k in range(3):
                acc[k] += ev[k].elapsed_time(ev[k + 1]) / n_ph
        phases = {"forward_ms": acc[0], "backward_ms": acc[1], "step_tail_ms": acc[2]}
        if world > 1 and hasattr(engine, "stop_trace"):
            tr = engine.stop_trace(ev[0])
            phases["unit_trace_ms"] = [[n, round(a, 2), round(b_, 2), round(c, 2)] for n, a, b_, c in tr]

    if args.trace_export:
        # every rank runs the two extra steps (they contain collectives); rank 0 writes the trace
        from torch.profiler import ProfilerActivity, profile
        from rumus_b200.utils.metrics import enable_tracing
        enable_tracing(True)
        with profile(activities=[ProfilerActivity.CPU, ProfilerActivity.CUDA]) as prof:
            for _ in range(2):
                train_step_device(dev_tokens[args.warmup])
            torch.cuda.synchronize()
        if rank == 0:
            prof.export_chrome_trace(args.trace_export)
        enable_tracing(False)
    if args.kernel_profile:
        from rumus_b200.utils.metrics import kernel_breakdown
        kb = kernel_breakdown(lambda: train_step_device(dev_tokens[args.warmup]), steps=2)
        if rank == 0:
            print(f"[kernel profile] {kb['kernel_ms_per_step']:.2f} ms of kernels per step over "
                  f"{kb['launches_per_step']:.0f} launches; span {kb['span_ms_per_step']:.2f} ms; "
                  f"busy {kb['busy_fraction']:.3f}", file=sys.stderr)
            for k_name, k_ms, k_n in kb["kernels"]:
                print(f"[kernel profile] {k_ms:9.3f} ms {k_n:6.0f}x  {k_name}", file=sys.stderr)

    if rank == 0:
        flops = cfg.flops_per_token() * B * S
        out = {
            "metric": "train tokens/sec (whole job, device-timed, max over ranks)",
            "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic uniform-random tokens (seeded), random-init weights",
            "config": {"model": "GPT 1.3B (24L d2048 16h FFN8192 GELU vocab50304)" if not args.layers
                       else f"DEBUG {cfg.num_layers} layers",
                       "global_batch": world * B, "seq_len": S,
                       "parallelism": (f"fsdp{world}" + (" reshard-after-forward" if args.reshard else "")) if world > 1 else "fsdp1 (single GPU)",
                       "comm_mode": engine.mode, "optimizer": "Adam fp32 master + moments",
                       "l2": "per-step working set (tens of GB) exceeds the 126 MB L2; no explicit flush"},
            "clocks": clocks,
            "e2e": {"value": e2e_value, "unit": "tokens/s", "ms_per_step": ms_e2e / args.steps,
                    "h2d_bytes_per_step": B * (S + 1) * 8, "d2h_bytes_per_step": 4},
            "gpu_launches": launches,
            "model_tflops_per_gpu": flops / (ms / args.steps / 1e3) / 1e12,
            "final_loss": float(last_loss.item()) if last_loss is not None else None,
            "device_status": status,
            "param_bytes_per_rank": engine.param_bytes(),
        }
        if phases:
            out["phases"] = phases
        print(json.dumps(out))
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
