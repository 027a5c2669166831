#!/usr/bin/env python
"""CPU fp32 functional baseline: 2-layer pre-LN decoder (d 128, 4 heads, FFN 512 ReLU, learned
position embedding, vocab 1024, seq 64, batch 8), Adam 1e-3, 50 steps on a fixed synthetic batch,
then a safetensors round trip that must be bit exact.

    python bench/bench_cpu_decoder.py [--steps 50] [--threads N]

Prints one JSON line: seconds per step (wall clock, CPU), first/last loss, round-trip check.
Comparison arms: the same model through plain ``torch.nn`` modules (``--impl torch``), and the
same step as a chain of single-threaded scalar C++ kernels (``--impl oracle``) — one kernel per op,
naive loops, the way the reference's CPU backend executes it (rumus/src/backend/cpu.rs).
"""
import argparse
import json
import os
import sys
import tempfile
import time

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402


def build_ours(cfg):
    from rumus_b200.models import GPT
    m = GPT(cfg, device="cpu", dtype=torch.float32)
    m.init_weights(0.02, seed=0)
    return m


class TorchDecoder(torch.nn.Module):
    def __init__(self, cfg):
        super().__init__()
        d = cfg.d_model
        self.tok = torch.nn.Embedding(cfg.vocab_size, d)
        self.pos = torch.nn.Embedding(cfg.seq_len, d)
        layer = torch.nn.TransformerEncoderLayer(d, cfg.num_heads, cfg.ffn_dim, 0.0, activation="relu",
                                                 batch_first=True, norm_first=True)
        self.enc = torch.nn.TransformerEncoder(layer, cfg.num_layers, enable_nested_tensor=False)
        self.ln = torch.nn.LayerNorm(d)
        self.head = torch.nn.Linear(d, cfg.vocab_size, bias=False)

    def forward(self, x, y):
        S = x.shape[1]
        h = self.tok(x) + self.pos(torch.arange(S))
        mask = torch.nn.Transformer.generate_square_subsequent_mask(S)
        h = self.ln(self.enc(h, mask=mask, is_causal=True))
        return torch.nn.functional.cross_entropy(self.head(h).flatten(0, 1), y.flatten())


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--threads", type=int, default=0)
    ap.add_argument("--impl", default="ours", choices=["ours", "torch", "oracle"])
    a = ap.parse_args()
    if a.threads:
        torch.set_num_threads(a.threads)
    from rumus_b200.models import GPTConfig
    cfg = GPTConfig.tiny_cpu()
    torch.manual_seed(0)
    tok = torch.randint(0, cfg.vocab_size, (8, cfg.seq_len + 1))
    x, y = tok[:, :-1], tok[:, 1:]
    if a.impl == "oracle":
        from rumus_b200.oracle import OracleDecoder
        dec = OracleDecoder(cfg, 8)
        dec.load_state_dict(build_ours(cfg).state_dict())
        for _ in range(3):
            dec.forward_backward(x, y); dec.adam_step(1e-3)
        losses = []
        t0 = time.perf_counter()
        for _ in range(a.steps):
            losses.append(dec.forward_backward(x, y))
            dec.adam_step(1e-3)
        dt = time.perf_counter() - t0
        print(json.dumps({"metric": "CPU seconds per training step", "impl": "oracle",
                          "value": dt / a.steps, "unit": "s/step", "steps": a.steps, "threads": 1,
                          "dtype": "f32", "first_loss": losses[0], "last_loss": losses[-1],
                          "safetensors_round_trip_exact": None,
                          "config": "2L d128 4h ffn512 relu vocab1024 seq64 batch8, Adam 1e-3"}))
        return
    if a.impl == "ours":
        from rumus_b200.optim import Adam
        model = build_ours(cfg)
        opt = Adam(model.parameters(), lr=1e-3)
    else:
        model = TorchDecoder(cfg)
        opt = torch.optim.Adam(model.parameters(), lr=1e-3)
    losses = []
    for _ in range(3):   # warm-up (allocator, thread pool); state is reset afterwards for neither arm
        loss = model(x, y); opt.zero_grad(); loss.backward(); opt.step()
    t0 = time.perf_counter()
    for _ in range(a.steps):
        loss = model(x, y)
        opt.zero_grad()
        loss.backward()
        opt.step()
        losses.append(float(loss.detach()))
    dt = time.perf_counter() - t0
    exact = None
    if a.impl == "ours":
        from rumus_b200.io.safetensors import load_safetensors, save_safetensors
        sd = {k: v.detach() for k, v in model.state_dict().items()}
        with tempfile.TemporaryDirectory() as d:
            path = os.path.join(d, "m.safetensors")
            save_safetensors(sd, path)
            back = load_safetensors(path)
        exact = all(torch.equal(sd[k].float(), back[k].float()) for k in sd) and set(sd) == set(back)
    print(json.dumps({"metric": "CPU seconds per training step", "impl": a.impl,
                      "value": dt / a.steps, "unit": "s/step", "steps": a.steps,
                      "threads": torch.get_num_threads(), "dtype": "f32",
                      "first_loss": losses[0], "last_loss": losses[-1],
                      "safetensors_round_trip_exact": exact,
                      "config": "2L d128 4h ffn512 relu vocab1024 seq64 batch8, Adam 1e-3"}))


if __name__ == "__main__":
    main()
