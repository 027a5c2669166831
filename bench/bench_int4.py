#!/usr/bin/env python
"""Weight-only quantised matmul paths on the Llama-7B layer shapes, per batch size: INT4 streaming
GEMV, INT4 dequantise + tcgen05 GEMM, the fused W4A16 tcgen05 kernel, and (``--q8``) the INT8 block
format through dequantise + GEMM and through the fused W8A16 kernel.

Kernel time, not launch time: every path is captured into a CUDA graph that runs it once on each of
eight distinct copies of the weight (200+ MB in total, so no copy is still in the 126 MB L2 when its
turn comes again), and the graph is replayed; CUDA events around the replay, 3 warm-ups.

    python bench/bench_int4.py [--shapes qkv,out,gate_up,down] [--rows 1,8,16,32,48,64,128] [--q8]

Prints, per shape and batch, microseconds per call of each path, the fraction of the measured copy
bandwidth the quantised weights' traffic reaches, and the fused kernels' relative error against the
dequantised fp32 product.
"""
import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402

SHAPES = {"qkv": (4096, 12288), "out": (4096, 4096), "gate_up": (4096, 22016), "down": (11008, 4096)}
COPIES = 8


def graph_time_us(fn_of_copy, reps=10, warm=3):
    """``fn_of_copy(i)`` runs the path on weight copy i.  Returns microseconds per call."""
    for i in range(COPIES):
        fn_of_copy(i)                      # eager warm-up (allocates cached workspaces)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for i in range(COPIES):
            fn_of_copy(i)
    for _ in range(warm):
        g.replay()
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(reps):
        g.replay()
    e.record()
    torch.cuda.synchronize()
    return s.elapsed_time(e) * 1e3 / (reps * COPIES)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--shapes", default="qkv,out,gate_up,down")
    ap.add_argument("--rows", default="1,8,16,32,48,64,128")
    ap.add_argument("--q8", action="store_true", help="also time the INT8 block format (block size 32)")
    a = ap.parse_args()
    from rumus_b200.nn.quant import Q8Tensor, QuantizedTensor, quantize_q8
    from rumus_b200.ops import native
    from rumus_b200.ops import quant_cuda as Q
    peaks = {}
    pk = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    if os.path.exists(pk):
        peaks = json.load(open(pk))
    hbm = float(peaks.get("hbm_gbs", 6650.0))
    for name in a.shapes.split(","):
        K, N = SHAPES[name]
        torch.manual_seed(0)
        qs = [QuantizedTensor.from_f32(torch.randn(K, N, device="cuda") * 0.02, 128, torch.float16) for _ in range(COPIES)]
        dense32 = qs[0].dequantize(torch.float32)
        packed_bytes = K * N / 2 + 2 * (K // 128) * N * 2
        q8s = None
        if a.q8:
            q8s = [quantize_q8(torch.randn(K, N, device="cuda") * 0.02, 32) for _ in range(COPIES)]
            q8_dense32 = native_dequant_q8(q8s[0])
            q8_bytes = K * N * 36 / 32
        for M in (int(r) for r in a.rows.split(",")):
            x = (torch.randn(M, K, device="cuda") * 0.5).bfloat16()
            row = {"shape": name, "K": K, "N": N, "M": M}
            if M <= Q.GEMV_MAX_M:
                old = Q.GEMV_CHUNKED_MAX_M
                Q.GEMV_CHUNKED_MAX_M = Q.GEMV_MAX_M      # force the GEMV for this batch size
                row["gemv_us"] = round(graph_time_us(lambda i: Q.int4_matmul(x, qs[i])), 1)
                Q.GEMV_CHUNKED_MAX_M = old
            row["dequant_gemm_us"] = round(graph_time_us(lambda i: native.gemm(x, Q.int4_dequant(qs[i], x.dtype))), 1)
            y = Q.int4_matmul_fused(x, qs[0])
            if y is not None:
                ref = x.float() @ dense32
                row["fused_rel_err"] = round(((y.float() - ref).norm() / ref.norm()).item(), 5)
                row["fused_us"] = round(graph_time_us(lambda i: Q.int4_matmul_fused(x, qs[i])), 1)
                row["fused_frac_of_measured_hbm"] = round(packed_bytes / (row["fused_us"] * 1e-6) / (hbm * 1e9), 3)
            if q8s is not None:
                row["q8_dequant_gemm_us"] = round(graph_time_us(
                    lambda i: native.gemm(x, Q.dequantize_q8_cuda(q8s[i], x.dtype))), 1)
                y8 = Q.q8_matmul_fused(x, q8s[0])
                if y8 is not None:
                    ref8 = x.float() @ q8_dense32
                    row["q8_fused_rel_err"] = round(((y8.float() - ref8).norm() / ref8.norm()).item(), 5)
                    row["q8_fused_us"] = round(graph_time_us(lambda i: Q.q8_matmul_fused(x, q8s[i])), 1)
                    row["q8_fused_frac_of_measured_hbm"] = round(q8_bytes / (row["q8_fused_us"] * 1e-6) / (hbm * 1e9), 3)
            row["status"] = native.read_status()
            print(json.dumps(row), flush=True)


def native_dequant_q8(q):
    from rumus_b200.ops import quant_cuda as Q
    return Q.dequantize_q8_cuda(q, torch.float32)


if __name__ == "__main__":
    main()
