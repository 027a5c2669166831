#!/usr/bin/env python
"""Llama-style 7B, tensor x pipeline parallel training throughput (TP=4 x PP=2, 1F1B, 8 micro-batches,
seq 4096, global batch 64, bf16 + fp32 master weights) on one 8-GPU box.

    torchrun --nproc-per-node 8 bench/bench_llama3d.py --tp 4 --pp 2 --steps 3 --warmup 2 [--mode fused|nccl]
    torchrun --nproc-per-node 4 bench/bench_llama3d.py --tp 2 --pp 2 --layers 4 --d-model 1024 ...   (scaled-down check)
"""
import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tp", type=int, default=4)
    ap.add_argument("--pp", type=int, default=2)
    ap.add_argument("--micro-batches", type=int, default=8)
    ap.add_argument("--global-batch", type=int, default=64)
    ap.add_argument("--seq", type=int, default=4096)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=2)
    ap.add_argument("--mode", default=None)
    ap.add_argument("--layers", type=int, default=32)
    ap.add_argument("--d-model", type=int, default=4096)
    ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--ffn", type=int, default=11008)
    ap.add_argument("--vocab", type=int, default=32000)
    a = ap.parse_args()
    import torch
    import torch.distributed as dist
    from rumus_b200.models.llama import LlamaConfig
    from rumus_b200.models.llama_parallel import ParallelLlamaStage
    from rumus_b200.ops import _lib, native
    from rumus_b200.parallel import FSDP
    from rumus_b200.parallel.pp import PipelineStage
    from rumus_b200.parallel.topology import build_topology
    from rumus_b200.parallel.tp import TPContext

    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    dist.init_process_group("nccl", device_id=dev)
    native.lib().rb_init_device()
    topo = build_topology(tp=a.tp, pp=a.pp)
    cfg = LlamaConfig(vocab_size=a.vocab, seq_len=a.seq, d_model=a.d_model, num_heads=a.heads,
                      num_kv_heads=a.heads, num_layers=a.layers, ffn_dim=a.ffn)
    mb_seqs = a.global_batch // (topo.dp * a.micro_batches)
    mb_tokens = mb_seqs * a.seq
    tp = TPContext(group=topo.tp_group, mode=a.mode, max_tokens=mb_tokens, max_features=a.d_model)
    stage = ParallelLlamaStage(cfg, tp, topo.pp_idx, a.pp, device=dev, dtype=torch.bfloat16)
    stage.init_weights(0.02, seed=0)
    stage.set_microbatch_shape(mb_seqs, a.seq)
    units = [(f"blocks.{i}", [b]) for i, b in enumerate(stage.blocks)]
    rest = [p for n, p in stage.named_parameters() if not n.startswith("blocks.")]
    if rest:
        units.append(("edge", rest))
    opt = FSDP(stage, lr=1e-4, beta2=0.95, unit_roots=units, local_only=True, defer_update=True)
    ps = PipelineStage(stage, topo.pp_idx, a.pp, topo.prev_stage_rank, topo.next_stage_rank,
                       (mb_tokens // a.tp, a.d_model), torch.bfloat16, dev)
    g = torch.Generator(device="cpu").manual_seed(1234 + topo.dp_idx)
    first, last = topo.pp_idx == 0, topo.pp_idx == a.pp - 1

    def make_batch():
        toks = [torch.randint(0, a.vocab, (mb_seqs, a.seq + 1), generator=g) for _ in range(a.micro_batches)]
        if first and last:
            raise SystemExit("pp must be >= 2")
        if first:
            return [t[:, :-1].to(dev) for t in toks]
        if last:
            return [t[:, 1:].to(dev) for t in toks]
        return [None] * a.micro_batches

    def step():
        opt.zero_grad()
        loss = ps.run(make_batch())
        opt.reduce_grads(replicated_group=topo.tp_group, dp_group=topo.dp_group)
        opt.step()
        return loss

    for _ in range(max(a.warmup, 1)):
        step()
    dist.barrier(); torch.cuda.synchronize()
    _lib.reset_launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    loss = None
    for _ in range(a.steps):
        loss = step()
    e1.record()
    dist.barrier(); torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1)], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    # Pipeline bubble as measured: one micro-batch's forward + backward on every stage without its
    # neighbours (every stage at once, so the tensor-parallel collectives inside still pair up);
    # a step of M micro-batches that never waited would take M times the slowest stage.
    act_shape = (mb_tokens // a.tp, a.d_model)
    tok = torch.randint(0, a.vocab, (mb_seqs, a.seq + 1), generator=g)
    mb_ms = []
    for it in range(3):
        opt.zero_grad()
        s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        dist.barrier(); torch.cuda.synchronize()
        s0.record()
        if first:
            out = stage(tok[:, :-1].to(dev))
            out.backward(torch.ones_like(out))
        else:
            xin = torch.randn(act_shape, device=dev, dtype=torch.bfloat16).mul_(0.02).requires_grad_(True)
            if last:
                stage((xin, tok[:, 1:].to(dev))).backward()
            else:
                out = stage(xin)
                out.backward(torch.ones_like(out))
        s1.record()
        torch.cuda.synchronize()
        if it > 0:
            mb_ms.append(s0.elapsed_time(s1))
    mb = torch.tensor([sum(mb_ms) / len(mb_ms)], device=dev)
    dist.all_reduce(mb, op=dist.ReduceOp.MAX)
    st = torch.tensor([native.read_status()], device=dev)
    dist.all_reduce(st, op=dist.ReduceOp.MAX)
    lt = torch.tensor([float(loss) if loss is not None else 0.0], device=dev)
    dist.all_reduce(lt, op=dist.ReduceOp.MAX)
    if rank == 0:
        ms = t.item() / a.steps
        tokens = a.global_batch * a.seq
        print(json.dumps({"metric": "train tokens/sec (whole job, device-timed, max over ranks)",
                          "value": tokens / (ms / 1e3), "unit": "tokens/s", "n_gpus": world,
                          "ms_per_step": ms, "steps": a.steps, "warmup": a.warmup, "dtype": "bf16",
                          "config": {"model": f"Llama {a.layers}L d{a.d_model} h{a.heads} ffn{a.ffn} vocab{a.vocab}",
                                     "global_batch": a.global_batch, "seq_len": a.seq,
                                     "parallelism": f"tp{a.tp}xpp{a.pp}xdp{topo.dp}", "micro_batches": a.micro_batches,
                                     "schedule": "1F1B", "comm_mode": tp.mode,
                                     "bubble_fraction_ideal": (a.pp - 1) / (a.micro_batches + a.pp - 1),
                                     "bubble_fraction_measured": 1.0 - a.micro_batches * mb.item() / ms,
                                     "micro_batch_fwd_bwd_ms_slowest_stage": mb.item()},
                          "model_tflops_per_gpu": cfg.flops_per_token() * tokens / (ms / 1e3) / 1e12 / world,
                          "loss": lt.item(), "gpu_launches": _lib.launch_count(), "device_status": int(st.item())}))
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
