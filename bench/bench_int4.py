#!/usr/bin/env python
"""INT4 weight-only matmul paths on the Llama-7B layer shapes, per batch size: streaming GEMV,
dequantise + tcgen05 GEMM, and the fused W4A16 tcgen05 kernel.  CUDA-event timing, 3 warm-ups, L2
flushed between iterations (the weights of one layer fit in L2, a decode step's do not).

    python bench/bench_int4.py [--shapes qkv,out,gate_up,down] [--rows 1,8,16,32,48,64,128]

Prints, per shape and batch, the time of each path in microseconds, the fraction of the measured
copy bandwidth the packed weights' traffic reaches, and the relative error of the fused kernel
against the dequantised fp32 product.
"""
import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402

SHAPES = {"qkv": (4096, 12288), "out": (4096, 4096), "gate_up": (4096, 22016), "down": (11008, 4096)}


def timeit(fn, flush, n=10, warm=3):
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(n):
        flush.zero_()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record(); fn(); e.record()
        torch.cuda.synchronize()
        ts.append(s.elapsed_time(e))
    ts.sort()
    return ts[len(ts) // 2] * 1e3


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--shapes", default="qkv,out,gate_up,down")
    ap.add_argument("--rows", default="1,8,16,32,48,64,128")
    a = ap.parse_args()
    from rumus_b200.nn.quant import QuantizedTensor
    from rumus_b200.ops import native
    from rumus_b200.ops import quant_cuda as Q
    peaks = {}
    pk = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    if os.path.exists(pk):
        peaks = json.load(open(pk))
    hbm = float(peaks.get("hbm_gbs", 6650.0))
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    for name in a.shapes.split(","):
        K, N = SHAPES[name]
        torch.manual_seed(0)
        q = QuantizedTensor.from_f32(torch.randn(K, N) * 0.02, 128, torch.float16).to("cuda")
        dense32 = q.dequantize(torch.float32)
        packed_bytes = K * N / 2 + 2 * (K // 128) * N * 2
        for M in (int(r) for r in a.rows.split(",")):
            x = (torch.randn(M, K, device="cuda") * 0.5).bfloat16()
            row = {"shape": name, "K": K, "N": N, "M": M}
            if M <= Q.GEMV_MAX_M:
                old = Q.GEMV_CHUNKED_MAX_M
                Q.GEMV_CHUNKED_MAX_M = Q.GEMV_MAX_M
                os.environ["RB_W4A16"] = "0"
                row["gemv_us"] = timeit(lambda: Q.int4_matmul(x, q), flush)
                Q.GEMV_CHUNKED_MAX_M = old
            row["dequant_gemm_us"] = timeit(lambda: native.gemm(x, Q.int4_dequant(q, x.dtype)), flush)
            y = Q.int4_matmul_fused(x, q)
            if y is not None:
                ref = x.float() @ dense32
                row["fused_rel_err"] = ((y.float() - ref).norm() / ref.norm()).item()
                row["fused_us"] = timeit(lambda: Q.int4_matmul_fused(x, q), flush)
                row["fused_frac_of_measured_hbm"] = packed_bytes / (row["fused_us"] * 1e-6) / (hbm * 1e9)
            row["status"] = native.read_status()
            print(json.dumps(row), flush=True)


if __name__ == "__main__":
    main()
