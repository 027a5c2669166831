#!/usr/bin/env python
"""ResNet-50 data-parallel training throughput: fp16 compute with dynamic loss scaling, SGD momentum 0.9,
256 images/GPU of 3x224x224 ~ N(0,1), labels uniform over 1000 classes; the gradient all-reduce is fused
with the loss-scale unscale and the non-finite check.

    python bench/bench_resnet.py --steps 5 --warmup 3 [--batch 256]
    torchrun --nproc-per-node N bench/bench_resnet.py ...
"""
import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=256)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--mode", default=None)
    ap.add_argument("--kernel-profile", action="store_true",
                    help="print a per-kernel breakdown of two extra steps to stderr")
    a = ap.parse_args()
    import torch
    import torch.distributed as dist
    from rumus_b200.models import ResNet50
    from rumus_b200.ops import _lib, functional as F, native
    from rumus_b200.optim import SGD, GradScaler
    from rumus_b200.parallel.dp import DataParallel
    world = int(os.environ.get("WORLD_SIZE", "1")); rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    native.lib().rb_init_device()
    torch.manual_seed(0)
    model = ResNet50(device=dev, dtype=torch.float16)
    dp = DataParallel(model, mode=a.mode)
    opt = SGD(model.parameters(), lr=0.1, momentum=0.9)
    scaler = GradScaler(init_scale=1024.0)
    g = torch.Generator(device=dev).manual_seed(100 + rank)
    x = torch.randn(a.batch, 3, 224, 224, device=dev, generator=g).half().contiguous(memory_format=torch.channels_last)
    y = torch.randint(0, 1000, (a.batch,), device=dev, generator=g)

    def step():
        dp.zero_grad()
        loss = F.cross_entropy_loss(model(x), y)
        scaler._ensure(dev)
        dp.begin_backward(scaler.inv_scale)      # buckets are reduced as backward fills them
        scaler.scale(loss).backward()
        found = dp.all_reduce_grads()
        opt.grad_scale, opt.skip_flag = None, found      # unscale already happened inside the all-reduce
        scaler.found_inf = found
        opt.step()
        scaler.update()
        return loss

    for _ in range(a.warmup):
        step()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    _lib.reset_launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(a.steps):
        loss = step()
    e1.record()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1)], device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    if rank == 0:
        ms = t.item() / a.steps
        print(json.dumps({"metric": "train images/sec (whole job, device-timed, max over ranks)",
                          "value": world * a.batch / (ms / 1e3), "unit": "images/s", "n_gpus": world,
                          "ms_per_step": ms, "dtype": "fp16", "loss_scale": scaler.scale_value,
                          "config": {"model": "ResNet-50", "images_per_gpu": a.batch, "comm_mode": dp.mode,
                                     "optimizer": "SGD momentum 0.9"},
                          "loss": float(loss.item()), "gpu_launches": _lib.launch_count(),
                          "device_status": native.read_status()}))
    if a.kernel_profile:
        from rumus_b200.utils.metrics import kernel_breakdown
        kb = kernel_breakdown(step, steps=2)
        if rank == 0:
            print(f"[kernel profile] {kb['kernel_ms_per_step']:.2f} ms of kernels per step over "
                  f"{kb['launches_per_step']:.0f} launches; span {kb['span_ms_per_step']:.2f} ms; "
                  f"busy {kb['busy_fraction']:.3f}", file=sys.stderr)
            for name, ms_k, n in kb["kernels"]:
                print(f"[kernel profile] {ms_k:9.3f} ms {n:6.0f}x  {name}", file=sys.stderr)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
