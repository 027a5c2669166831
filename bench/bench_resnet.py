#!/usr/bin/env python
"""ResNet-50 data-parallel training throughput: fp16 compute with dynamic loss scaling, SGD momentum 0.9,
256 images/GPU of 3x224x224 ~ N(0,1), labels uniform over 1000 classes; the gradient all-reduce is fused
with the loss-scale unscale and the non-finite check.

    python bench/bench_resnet.py --steps 5 --warmup 3 [--batch 256]
    torchrun --nproc-per-node N bench/bench_resnet.py ...
    python bench/bench_resnet.py --impl torch      # the same model in plain torch.nn (cuDNN convolutions,
                                                   # channels-last fp16, torch SGD + GradScaler, DDP): the
                                                   # library row to compare with on the same box
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
    ap.add_argument("--impl", default="ours", choices=["ours", "torch"])
    ap.add_argument("--host-scaler", action="store_true",
                    help="keep the loss scale on the host (one device-to-host read of the overflow flag per step)")
    ap.add_argument("--kernel-profile", action="store_true",
                    help="print a per-kernel breakdown of two extra steps to stderr")
    a = ap.parse_args()
    if a.impl == "torch":
        return torch_row(a)
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
    # the scale lives on the device: no host read of the overflow flag between steps
    scaler = GradScaler(init_scale=1024.0, device_side=not a.host_scaler)
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
                          "peak_mem_gb": torch.cuda.max_memory_allocated() / 2 ** 30,
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


def torch_row(a):
    """ResNet-50 written with torch.nn only, trained the same way (fp16 weights and activations,
    channels-last, SGD momentum 0.9, dynamic loss scaling, DistributedDataParallel over NCCL)."""
    import torch
    import torch.distributed as dist
    import torch.nn as nn
    world = int(os.environ.get("WORLD_SIZE", "1")); rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    torch.backends.cudnn.benchmark = True

    class Block(nn.Module):
        def __init__(self, cin, w, stride):
            super().__init__()
            cout = 4 * w
            self.c1, self.b1 = nn.Conv2d(cin, w, 1, bias=False), nn.BatchNorm2d(w)
            self.c2, self.b2 = nn.Conv2d(w, w, 3, stride, 1, bias=False), nn.BatchNorm2d(w)
            self.c3, self.b3 = nn.Conv2d(w, cout, 1, bias=False), nn.BatchNorm2d(cout)
            self.down = None
            if stride != 1 or cin != cout:
                self.down = nn.Sequential(nn.Conv2d(cin, cout, 1, stride, bias=False), nn.BatchNorm2d(cout))

        def forward(self, x):
            idt = x if self.down is None else self.down(x)
            y = torch.relu(self.b1(self.c1(x)))
            y = torch.relu(self.b2(self.c2(y)))
            return torch.relu(self.b3(self.c3(y)) + idt)

    layers, cin = [nn.Conv2d(3, 64, 7, 2, 3, bias=False), nn.BatchNorm2d(64), nn.ReLU(), nn.MaxPool2d(3, 2, 1)], 64
    for i, n in enumerate((3, 4, 6, 3)):
        for j in range(n):
            layers.append(Block(cin, 64 * 2 ** i, 2 if (j == 0 and i > 0) else 1))
            cin = 256 * 2 ** i
    layers += [nn.AdaptiveAvgPool2d(1), nn.Flatten(), nn.Linear(cin, 1000)]
    torch.manual_seed(0)
    model = nn.Sequential(*layers).to(dev).half().to(memory_format=torch.channels_last)
    if world > 1:
        model = nn.parallel.DistributedDataParallel(model, device_ids=[local])
    opt = torch.optim.SGD(model.parameters(), lr=0.1, momentum=0.9)
    scale = torch.full((), 1024.0, device=dev)
    g = torch.Generator(device=dev).manual_seed(100 + rank)
    x = torch.randn(a.batch, 3, 224, 224, device=dev, generator=g).half().contiguous(memory_format=torch.channels_last)
    y = torch.randint(0, 1000, (a.batch,), device=dev, generator=g)

    def step():
        opt.zero_grad(set_to_none=True)
        loss = nn.functional.cross_entropy(model(x).float(), y)
        (loss * scale).backward()
        grads = [p.grad for p in model.parameters() if p.grad is not None]
        torch._foreach_div_(grads, scale)                 # unscale on the device; fp16 weights, as in our arm
        opt.step()
        return loss

    for _ in range(a.warmup):
        step()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
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
        print(json.dumps({"impl": "torch.nn + cuDNN (channels-last fp16) + DDP",
                          "metric": "train images/sec (whole job, device-timed, max over ranks)",
                          "value": world * a.batch / (ms / 1e3), "unit": "images/s", "n_gpus": world,
                          "ms_per_step": ms, "dtype": "fp16", "loss": float(loss.item()),
                          "peak_mem_gb": torch.cuda.max_memory_allocated() / 2 ** 30}))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
