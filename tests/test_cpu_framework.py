"""CPU tests of the framework layer: replicas of the reference's five integration tests
(rumus/tests/*.rs — same shapes and thresholds), checkpoint byte compatibility, optimizers,
schedulers, quantisation formats."""
import json
import math
import os
import struct

import pytest
import torch
import torch.nn as nn

import rumus_b200.nn as rnn
from rumus_b200.io import load_into, load_safetensors, save_safetensors, serialize
from rumus_b200.models import GPT, GPTConfig, Llama, LlamaConfig
from rumus_b200.ops import functional as F
from rumus_b200.optim import (SGD, Adam, AdamW, CosineAnnealingLR, GradScaler, StepLR,
                              clip_grad_norm_)
from rumus_b200.train import Trainer


class XorMlp(rnn.Module):
    def __init__(self):
        super().__init__()
        self.hidden = rnn.Linear(2, 8)
        self.output = rnn.Linear(8, 1)

    def forward(self, x):
        return self.output(F.relu(self.hidden(x)))


def test_xor_training_and_save_load(tmp_path):
    """rumus/tests/mlp_test.rs:43-122"""
    torch.manual_seed(0)
    x = torch.tensor([[0., 0.], [0., 1.], [1., 0.], [1., 1.]])
    y = torch.tensor([[0.], [1.], [1.], [0.]])
    m = XorMlp()
    opt = Adam(m.parameters(), lr=0.01)
    loss = None
    for _ in range(200):
        opt.zero_grad()
        loss = F.mse_loss(m(x), y)
        loss.backward()
        opt.step()
        if loss.item() < 0.01:
            break
    for _ in range(800):   # the reference seed converges in 200; allow a different init more room
        if loss.item() < 0.01:
            break
        opt.zero_grad(); loss = F.mse_loss(m(x), y); loss.backward(); opt.step()
    assert loss.item() < 0.01
    sd = m.state_dict()
    assert set(sd.keys()) == {"hidden.weight", "hidden.bias", "output.weight", "output.bias"}
    assert tuple(sd["hidden.weight"].shape) == (2, 8)   # [in, out]
    p = str(tmp_path / "xor.safetensors")
    save_safetensors(sd, p)
    m2 = XorMlp()
    load_into(m2, p)
    assert torch.equal(m(x), m2(x))


def test_cross_entropy_training_and_trainer_api():
    """rumus/tests/train_loop_test.rs:72-196"""
    torch.manual_seed(1)
    xs = torch.randn(12, 4)
    ys = torch.arange(12) % 3
    xs = xs + torch.nn.functional.one_hot(ys, 4)[:, :4].float() * 3
    model = nn.Sequential(rnn.Linear(4, 16), nn.ReLU(), rnn.Linear(16, 3))
    tr = Trainer(AdamW(model.parameters(), lr=0.01, weight_decay=0.01))
    for epoch in range(200):
        tr.reset_epoch()
        tr.train_step(lambda: F.cross_entropy_loss(model(xs), ys))
    assert tr.epoch_avg_loss() < 0.15
    assert tr.optimizer_mut().get_lr() == 0.01


def test_cnn_spatial_classification():
    """rumus/tests/cnn_test.rs:82-116"""
    torch.manual_seed(2)
    imgs = torch.zeros(4, 1, 8, 8)
    imgs[0, 0, :4, :4] = 1; imgs[1, 0, :4, 4:] = 1; imgs[2, 0, 4:, :4] = 1; imgs[3, 0, 4:, 4:] = 1
    tgt = torch.eye(4)
    model = nn.Sequential(rnn.Conv2d(1, 4, 3, 1, 1), nn.ReLU(), rnn.MaxPool2d(2), rnn.Flatten(),
                          rnn.Linear(4 * 4 * 4, 4))
    opt = Adam(model.parameters(), lr=0.01)
    for _ in range(100):
        opt.zero_grad(); loss = F.mse_loss(model(imgs), tgt); loss.backward(); opt.step()
    assert loss.item() < 0.05
    assert tuple(model[0].weight.shape) == (4, 9)   # reference layout [C_out, C_in*K*K]


class TinyGPT(rnn.Module):
    """rumus/tests/transformer_test.rs:21-73"""

    def __init__(self, vocab, seq, d, heads):
        super().__init__()
        self.token_emb = rnn.Embedding(vocab, d)
        self.pos_emb = rnn.Embedding(seq, d)
        self.block = rnn.TransformerBlock(d, heads)
        self.ln_final = rnn.LayerNorm(d)
        self.head = rnn.Linear(d, vocab, bias=False)

    def forward(self, ids, mask=None):
        x = self.token_emb(ids, self.pos_emb.weight)
        x = self.block(x, mask)
        return self.head(self.ln_final(x))


def test_tiny_gpt_cpu():
    torch.manual_seed(3)
    vocab, seq, d, batch = 4, 6, 32, 8
    ids = torch.tensor([[(b + s) % vocab for s in range(seq)] for b in range(batch)])
    tgt = torch.tensor([[(b + s + 1) % vocab for s in range(seq)] for b in range(batch)])
    mask = torch.triu(torch.full((seq, seq), -1e9), diagonal=1)
    m = TinyGPT(vocab, seq, d, 1)
    opt = AdamW(m.parameters(), lr=1e-3)
    for _ in range(200):
        opt.zero_grad()
        loss = F.cross_entropy_loss(m(ids, mask).reshape(-1, vocab), tgt.reshape(-1))
        loss.backward(); opt.step()
    assert loss.item() < 1.0
    # the fused (flash) path and the additive-mask path agree
    with torch.no_grad():
        assert torch.allclose(m(ids, mask), m(ids, None), atol=1e-4)


def test_config1_decoder_50_adam_steps_and_exact_roundtrip(tmp_path):
    """CPU f32 2-layer pre-LN decoder: d128, 4 heads, FFN 512 ReLU, learned pos-emb, vocab 1024,
    seq 64, batch 8, tokens uniform from seed 0, Adam 1e-3, 50 steps, safetensors round trip."""
    cfg = GPTConfig.tiny_cpu()
    torch.manual_seed(0)
    m = GPT(cfg)
    g = torch.Generator().manual_seed(0)
    tr = Trainer(Adam(m.parameters(), lr=1e-3))
    tok = torch.randint(0, cfg.vocab_size, (8, cfg.seq_len + 1), generator=g)
    first = last = None
    for step in range(50):
        l = tr.train_step(lambda: m(tok[:, :-1], tok[:, 1:]))
        first = first if first is not None else l.item()
        last = l.item()
    assert last < first
    p = str(tmp_path / "dec.safetensors")
    save_safetensors(m.state_dict(), p)
    m2 = GPT(cfg)
    load_into(m2, p)
    x = torch.randint(0, cfg.vocab_size, (2, cfg.seq_len))
    assert torch.equal(m(x), m2(x))
    keys = set(load_safetensors(p).keys())
    assert "blocks.0.attn.q_proj.weight" in keys and "blocks.1.mlp_fc2.bias" in keys
    assert "token_emb.weight" in keys and "ln_final.weight" in keys and "head.weight" in keys


def test_safetensors_bytes_match_reference_serializer(tmp_path):
    """Same byte stream as the safetensors crate the reference uses (python package = same core)."""
    st = pytest.importorskip("safetensors.torch")
    torch.manual_seed(4)
    sd = {"b.weight": torch.randn(3, 5), "a.bias": torch.randn(7), "zeta": torch.randn(2, 2, 2),
          "a.weight": torch.randn(4, 4).t()}   # non-contiguous input is stored contiguous
    ours = serialize(sd)
    ref = st.save({k: v.contiguous() for k, v in sd.items()})
    assert ours == ref
    n = struct.unpack("<Q", ours[:8])[0]
    assert n % 8 == 0
    hdr = json.loads(ours[8:8 + n])
    assert all(v["dtype"] == "F32" for v in hdr.values())
    p = str(tmp_path / "x.safetensors")
    save_safetensors(sd, p)
    back = load_safetensors(p)
    assert all(torch.equal(back[k], sd[k]) for k in sd)
    # loader refuses non-F32 like the reference (rumus/src/nn/io.rs:102-107)
    st.save_file({"h": torch.zeros(2, dtype=torch.float16)}, p)
    with pytest.raises(ValueError):
        load_safetensors(p)


def test_state_dict_names_and_layouts():
    blk = rnn.TransformerBlock(16, 2)
    keys = list(blk.state_dict().keys())
    for n in ("ln1.weight", "attn.q_proj.weight", "attn.k_proj.bias", "attn.v_proj.weight",
              "attn.out_proj.bias", "ln2.bias", "mlp_fc1.weight", "mlp_fc2.bias"):
        assert n in keys
    assert tuple(blk.state_dict()["mlp_fc1.weight"].shape) == (16, 64)
    sd = blk.state_dict()
    blk2 = rnn.TransformerBlock(16, 2)
    blk2.load_state_dict(sd)
    x = torch.randn(2, 5, 16)
    assert torch.equal(blk(x), blk2(x))
    bn = rnn.BatchNorm2d(3)
    assert set(bn.state_dict().keys()) == {"weight", "bias", "running_mean", "running_var"}
    ct = rnn.ConvTranspose2d(2, 3, 4)
    assert tuple(ct.weight.shape) == (2, 3 * 16)
    lm = Llama(LlamaConfig.tiny())
    k = lm.state_dict().keys()
    assert "blocks.0.mlp.gate_proj.weight" in k and "blocks.0.mlp.up_proj.weight" in k


def test_reference_lcg_init_stream():
    """Linear init follows the reference LCG (seed 42, rumus/src/nn/linear.rs:15-31)."""
    rnn.use_reference_init(True)
    try:
        lin = rnn.Linear(3, 2)
        s = 42
        vals = []
        for _ in range(6):
            s = (s * 6364136223846793005 + 1442695040888963407) & (2 ** 64 - 1)
            vals.append((2.0 * ((s >> 33) / 2 ** 31) - 1.0) * math.sqrt(1 / 3))
        assert torch.allclose(lin.weight.detach().view(-1), torch.tensor(vals, dtype=torch.float32))
    finally:
        rnn.use_reference_init(False)


def test_optimizers_match_torch():
    torch.manual_seed(5)
    w0 = torch.randn(10, 3)
    g = [torch.randn(10, 3) for _ in range(5)]
    for ours_cls, torch_cls, kw, tkw in [
        (Adam, torch.optim.Adam, dict(lr=1e-2), dict(lr=1e-2, eps=1e-8)),
        (AdamW, torch.optim.AdamW, dict(lr=1e-2, weight_decay=0.1), dict(lr=1e-2, weight_decay=0.1, eps=1e-8)),
        (SGD, torch.optim.SGD, dict(lr=0.1, momentum=0.9), dict(lr=0.1, momentum=0.9)),
    ]:
        p = nn.Parameter(w0.clone()); q = nn.Parameter(w0.clone())
        o, t = ours_cls([p], **kw), torch_cls([q], **tkw)
        for gi in g:
            p.grad = gi.clone(); q.grad = gi.clone()
            o.step(); t.step()
        assert torch.allclose(p, q, atol=1e-5), ours_cls


def test_clip_and_schedulers_and_scaler():
    p = nn.Parameter(torch.zeros(4)); p.grad = torch.tensor([3., 4., 0., 0.])
    n = clip_grad_norm_([p], 1.0)
    assert abs(float(n) - 5.0) < 1e-5 and abs(p.grad.norm().item() - 1.0) < 1e-4
    s = StepLR(0.1, 2, 0.5)
    lrs = []
    for _ in range(4):
        s.step(); lrs.append(s.get_lr())
    assert lrs == [0.1, 0.05, 0.05, 0.025]
    c = CosineAnnealingLR(1.0, 4, 0.0)
    c.step(); assert abs(c.get_lr() - 0.5 * (1 + math.cos(math.pi / 4))) < 1e-6
    for _ in range(5):
        c.step()
    assert c.get_lr() == 0.0
    # GradScaler: overflow -> skip + halve; clean steps grow the scale
    q = nn.Parameter(torch.ones(3))
    opt = SGD([q], lr=1.0)
    sc = GradScaler(init_scale=8.0, growth_interval=2)
    q.grad = torch.tensor([float("inf"), 1., 1.])
    sc._ensure(q.device); sc.unscale_and_check(opt); opt.step()
    assert sc.update() is True and sc.scale_value == 4.0 and torch.equal(q.data, torch.ones(3))
    for _ in range(2):
        q.grad = torch.full((3,), 4.0)      # scaled by 4 -> true grad 1
        sc.unscale_and_check(opt); opt.step(); assert sc.update() is False
    assert sc.scale_value == 8.0 and torch.allclose(q.data, torch.full((3,), -1.0))
    # the same sequence with the scale kept next to the gradients (no host read of the flag in update())
    q2 = nn.Parameter(torch.ones(3))
    opt2 = SGD([q2], lr=1.0)
    sd = GradScaler(init_scale=8.0, growth_interval=2, device_side=True)
    q2.grad = torch.tensor([float("inf"), 1., 1.])
    sd._ensure(q2.device); sd.unscale_and_check(opt2); opt2.step()
    assert sd.update() is None and sd.scale_value == 4.0 and torch.equal(q2.data, torch.ones(3))
    assert float(sd.inv_scale) == 0.25
    for _ in range(2):
        q2.grad = torch.full((3,), 4.0)
        sd.unscale_and_check(opt2); opt2.step(); sd.update()
    assert sd.scale_value == 8.0 and torch.allclose(q2.data, torch.full((3,), -1.0))
    assert sd.state_dict() == {"scale": 8.0, "good_steps": 2}
    assert float((torch.ones(()) * 1.0 * sd._scale_dev)) == float(sd.scale(torch.ones(())))


def test_int4_and_q8_formats():
    from rumus_b200.nn.quant import (QLinear, QuantizedTensor, dequantize_q8, matmul_q8,
                                     quantize_q8)
    torch.manual_seed(6)
    w = torch.randn(200, 24)   # K not a multiple of the group: padded to 256
    q = QuantizedTensor.from_f32(w, 128)
    assert q.padded_k == 256 and tuple(q.packed.shape) == (32, 24) and tuple(q.scales.shape) == (2, 24)
    # word/nibble order of the reference: word (row//8)*N + col, nibble row%8
    row, col = 13, 5
    grp = row // 128
    sc, zp = q.scales[grp, col].item(), q.zero_points[grp, col].item()
    expect = int(min(15, max(0, round(w[row, col].item() / sc + zp))))
    word = int(q.packed[row // 8, col].item()) & 0xFFFFFFFF
    assert (word >> (4 * (row % 8))) & 0xF == expect
    deq = q.dequantize()
    assert (deq - w).abs().max() <= q.scales.max() * 0.51
    lin = rnn.Linear(200, 24)
    ql = QLinear.from_linear(lin, 128)
    x = torch.randn(5, 200)
    assert torch.allclose(ql(x), x @ ql.qweight.dequantize() + lin.bias, atol=1e-4)
    # Q8: [f16 scale | 2 pad bytes | int8 x block] per block, blocks run down each column
    w8 = torch.randn(64, 6)
    q8 = quantize_q8(w8, 32)
    assert q8.data.numel() == (64 * 6 // 32) * 36
    blk0 = w8[:32, 0]
    scale = torch.tensor(blk0.abs().max().item() / 127).half()
    raw = q8.data[:2].view(torch.float16)
    assert raw.item() == scale.item()
    assert (dequantize_q8(q8) - w8).abs().max() < 0.02 * w8.abs().max()
    assert matmul_q8(torch.randn(3, 64), q8).shape == torch.Size([3, 6])


def test_reference_op_names_are_all_present():
    """Every public op of the reference's tensor surface (rumus/src/tensor/ops.rs) has a function of
    the same name; the plain tensor-layer ones behave like their PyTorch counterparts."""
    import torch
    from rumus_b200.ops import functional as F
    names = ("transpose reshape contiguous add sub mul matmul relu mse_loss cross_entropy_loss add_bias "
             "slice_batch im2col add_channel_bias max_pool2d flatten dropout sigmoid tanh_act gelu leaky_relu "
             "bmm batched_transpose softmax layer_norm batch_norm_2d adaptive_avg_pool2d embedding "
             "broadcast_add broadcast_sub broadcast_mul to_dtype quantize dequantize slice_range cat stack "
             "flash_attention").split()
    missing = [n for n in names if not callable(getattr(F, n, None))]
    assert not missing, missing
    torch.manual_seed(0)
    x = torch.randn(2, 3, 8, 8, requires_grad=True)
    assert F.im2col(x, 3, 1, 1).shape == (2, 27, 64) and F.im2col(x[0], 3).shape == (27, 36)
    assert torch.equal(F.add_channel_bias(x, torch.arange(3.0)), x + torch.arange(3.0).view(3, 1, 1))
    assert torch.equal(F.slice_range(x, 1, 1, 3), x[:, 1:3]) and torch.equal(F.slice_batch(x, 1, 2), x[1:2])
    assert F.stack([x, x]).shape == (2, 2, 3, 8, 8) and F.cat([x, x], 1).shape == (2, 6, 8, 8)
    assert torch.equal(F.broadcast_mul(x, torch.ones(8)), x) and torch.equal(F.sub(x, x), torch.zeros_like(x))
    assert F.batched_transpose(x).shape == (2, 3, 8, 8) and F.flatten(x).shape == (2, 192)
    w = torch.randn(64, 16)
    assert (F.dequantize(F.quantize(w)) - w).abs().max() < 0.05
    F.to_dtype(F.tanh_act(x), torch.float64).sum().backward()
    assert x.grad is not None and x.grad.shape == x.shape


def test_stem_weight_matrix_order_matches_the_patch_rows():
    """The direct stem kernels order K as kh*24 + 1 + kw*3 + ci: a patch matrix built that way times the
    permuted weight is the convolution, and the inverse map turns a [192, 64] gradient back into
    [64, 3, 7, 7]."""
    import torch.nn.functional as TF
    from rumus_b200.ops.vision_cuda import STEM_K, _stem_weight_matrix
    torch.manual_seed(0)
    B, H, W = 2, 12, 16
    x = torch.randn(B, 3, H, W, dtype=torch.float64)
    w = torch.randn(64, 3, 7, 7, dtype=torch.float64, requires_grad=True)
    y = TF.conv2d(x, w, None, 2, 3, 1)
    Ho, Wo = y.shape[2], y.shape[3]
    xp = TF.pad(x.permute(0, 2, 3, 1), (0, 0, 3, 3 + 8, 3, 3))                  # NHWC, zero border
    cols = torch.zeros(B, Ho, Wo, STEM_K, dtype=torch.float64)
    for kh in range(7):
        for oh in range(Ho):
            for ow in range(Wo):
                run = xp[:, 2 * oh + kh, 2 * ow:2 * ow + 7].reshape(B, 21)        # 7 taps x 3 channels
                cols[:, oh, ow, kh * 24 + 1:kh * 24 + 22] = run
    wk = _stem_weight_matrix(w.detach())
    assert wk.shape == (64, STEM_K)
    torch.testing.assert_close((cols.view(-1, STEM_K) @ wk.t()).view(B, Ho, Wo, 64).permute(0, 3, 1, 2), y.detach())
    g = torch.randn_like(y)
    y.backward(g)
    dwk = cols.view(-1, STEM_K).t() @ g.permute(0, 2, 3, 1).reshape(-1, 64)      # [192, 64]
    dw = dwk[:168].view(7, 24, 64)[:, 1:22].reshape(7, 7, 3, 64).permute(3, 2, 0, 1)
    torch.testing.assert_close(dw, w.grad)


def test_strided_conv_data_gradient_decomposes_into_stride1_phases():
    """The strided data gradient of the implicit-GEMM convolution runs one stride-1 gather per phase
    ((ih + pad) % s, (iw + pad) % s) with the taps kh = phase + s*a.  The same index arithmetic in plain
    PyTorch reproduces autograd's data gradient, including 1x1 kernels (phases without taps stay zero)
    and ragged sizes."""
    import torch.nn.functional as TF
    torch.manual_seed(0)
    for (H, W, K, s, pad) in ((15, 13, 3, 2, 1), (14, 14, 1, 2, 0), (9, 12, 5, 3, 2), (8, 8, 3, 2, 0)):
        B, Cin, Cout = 2, 3, 4
        x = torch.randn(B, Cin, H, W, dtype=torch.float64, requires_grad=True)
        w = torch.randn(Cout, Cin, K, K, dtype=torch.float64)
        y = TF.conv2d(x, w, None, s, pad, 1)
        g = torch.randn_like(y)
        y.backward(g)
        Ho, Wo = y.shape[2], y.shape[3]
        dy = g.permute(0, 2, 3, 1)                                          # NHWC
        dx = torch.zeros(B, H, W, Cin, dtype=torch.float64)
        for rh in range(min(s, K)):
            for rw in range(min(s, K)):
                e_h, e_w = (rh - pad) % s, (rw - pad) % s
                if e_h >= H or e_w >= W:
                    continue
                c_h, c_w = (e_h + pad - rh) // s, (e_w + pad - rw) // s
                taps = w[:, :, rh::s, rw::s]                                # [Cout, Cin, KHp, KWp]
                Hu, Wu = -(-(H - e_h) // s), -(-(W - e_w) // s)
                for u in range(Hu):
                    for v in range(Wu):
                        acc = torch.zeros(B, Cin, dtype=torch.float64)
                        for a in range(taps.shape[2]):
                            for b in range(taps.shape[3]):
                                oh, ow = u + c_h - a, v + c_w - b
                                if 0 <= oh < Ho and 0 <= ow < Wo:
                                    acc += dy[:, oh, ow, :] @ taps[:, :, a, b]
                        dx[:, s * u + e_h, s * v + e_w, :] = acc
        torch.testing.assert_close(dx.permute(0, 3, 1, 2), x.grad)
