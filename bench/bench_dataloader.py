#!/usr/bin/env python
"""Data-loader throughput on the CPU: records per second and GB/s of batch assembly from a `.rrec`
file, native C++ loader (worker threads filling a batch ring) against the Python ``DataLoader``
(threads + ``collate``) over the same file and in the same shuffled order.

    python bench/bench_dataloader.py [--records 4096] [--record-floats 8192] [--batch 32] [--workers 4]

Prints one JSON line.  Record size defaults to 32 KiB (an fp32 window of 8192 values) plus a
target of the same size — the shape of a token-window corpus.
"""
import argparse
import json
import os
import sys
import tempfile
import time

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--records", type=int, default=4096)
    ap.add_argument("--record-floats", type=int, default=8192)
    ap.add_argument("--batch", type=int, default=32)
    ap.add_argument("--workers", type=int, default=4)
    ap.add_argument("--epochs", type=int, default=3)
    a = ap.parse_args()
    from rumus_b200.data import DataLoader, NativeBatchLoader, RecordDataset, RecordWriter
    with tempfile.TemporaryDirectory() as d:
        path = os.path.join(d, "corpus.rrec")
        w = RecordWriter.create(path)
        g = torch.Generator().manual_seed(0)
        for i in range(a.records):
            x = torch.randn(a.record_floats, generator=g)
            w.append(x, x + 1)
        w.finish()
        bytes_per_epoch = a.records * a.record_floats * 4 * 2

        def run(make):
            loader = make()
            best, checksum = None, 0.0
            for _ in range(a.epochs):
                t0 = time.perf_counter()
                n = 0
                for item in loader:
                    n += item.input.shape[0]
                    checksum += float(item.input[0, 0])
                dt = time.perf_counter() - t0
                best = dt if best is None else min(best, dt)
            return best, n, checksum

        t_native, n1, c1 = run(lambda: NativeBatchLoader(path, a.batch, shuffle=True, num_workers=a.workers,
                                                         prefetch_batches=8))
        t_python, n2, c2 = run(lambda: DataLoader(RecordDataset.open(path), a.batch, shuffle=True,
                                                  num_workers=a.workers))
        print(json.dumps({
            "metric": "data loader throughput (CPU)", "records": a.records,
            "record_bytes": a.record_floats * 4 * 2, "batch": a.batch, "workers": a.workers,
            "native_records_per_s": n1 / t_native, "native_gb_per_s": bytes_per_epoch / t_native / 1e9,
            "python_records_per_s": n2 / t_python, "python_gb_per_s": bytes_per_epoch / t_python / 1e9,
            "speedup": t_python / t_native, "same_order": abs(c1 - c2) < 1e-3}))


if __name__ == "__main__":
    main()
