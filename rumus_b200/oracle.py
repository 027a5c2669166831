"""ctypes face of the C++ scalar CPU oracle (``csrc/cpu_oracle/cpu_oracle.cpp``): an independent
fp32 restatement of the reference's CPU backend and shader math, used as a second opinion next to
the PyTorch references and as the timed CPU baseline."""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_longlong, c_uint, c_void_p

import numpy as np
import torch

from .ops import _lib


def _p(t):
    return c_void_p(t.data_ptr()) if t is not None else c_void_p(0)


def _f(t):
    return t.detach().float().contiguous()


def _L():
    L = _lib.host_lib()
    L.orc_cross_entropy.restype = c_float
    return L


def matmul(a, b):
    a, b = _f(a), _f(b)
    out = torch.empty(a.shape[0], b.shape[1])
    _L().orc_matmul(_p(a), _p(b), _p(out), c_int(a.shape[0]), c_int(a.shape[1]), c_int(b.shape[1]))
    return out


def unary(name, x, arg=None):
    x = _f(x)
    out = torch.empty_like(x)
    fn = getattr(_L(), f"orc_{name}")
    if arg is None:
        fn(_p(x), _p(out), c_longlong(x.numel()))
    else:
        fn(_p(x), c_float(arg), _p(out), c_longlong(x.numel()))
    return out


def softmax(x):
    x = _f(x)
    out = torch.empty_like(x)
    _L().orc_softmax(_p(x), _p(out), c_int(x.numel() // x.shape[-1]), c_int(x.shape[-1]))
    return out


def layer_norm(x, w, b, eps=1e-5):
    x, w, b = _f(x), _f(w), _f(b)
    rows, d = x.numel() // x.shape[-1], x.shape[-1]
    out, save = torch.empty_like(x), torch.empty(rows, 2)
    _L().orc_layer_norm(_p(x), _p(w), _p(b), _p(out), _p(save), c_int(rows), c_int(d), c_float(eps))
    return out, save


def layer_norm_backward(x, w, dy, save):
    x, w, dy = _f(x), _f(w), _f(dy)
    rows, d = x.numel() // x.shape[-1], x.shape[-1]
    dx, dw, db = torch.empty_like(x), torch.empty(d), torch.empty(d)
    _L().orc_layer_norm_backward(_p(x), _p(w), _p(dy), _p(save), _p(dx), _p(dw), _p(db), c_int(rows), c_int(d))
    return dx, dw, db


def cross_entropy(logits, targets):
    x = _f(logits)
    t = targets.to(torch.int64).contiguous()
    g = torch.empty_like(x)
    loss = _L().orc_cross_entropy(_p(x), _p(t), _p(g), c_int(x.shape[0]), c_int(x.shape[1]))
    return float(loss), g


def conv2d(x, w, bias=None, stride=1, pad=0, dil=1):
    x, w = _f(x), _f(w)
    B, Ci, H, W = x.shape
    Co, _, Kh, Kw = w.shape
    Ho = (H + 2 * pad - dil * (Kh - 1) - 1) // stride + 1
    Wo = (W + 2 * pad - dil * (Kw - 1) - 1) // stride + 1
    y = torch.empty(B, Co, Ho, Wo)
    b = _f(bias) if bias is not None else None
    _L().orc_conv2d(_p(x), _p(w), _p(b), _p(y), *[c_int(v) for v in (B, Ci, H, W, Co, Kh, Kw, stride, pad, dil)])
    return y


def flash_attention(q, k, v, causal=True):
    """q/k/v [BH, N, d]"""
    q, k, v = _f(q), _f(k), _f(v)
    o = torch.empty_like(q)
    _L().orc_flash_attention(_p(q), _p(k), _p(v), _p(o), c_int(q.shape[0]), c_int(q.shape[1]), c_int(q.shape[2]),
                             c_int(1 if causal else 0))
    return o


def qmatmul_int4(x, qw):
    x = _f(x)
    y = torch.empty(x.shape[0], qw.n)
    sc, zp = _f(qw.scales), _f(qw.zero_points)
    packed = qw.packed.cpu().contiguous()
    _L().orc_qmatmul_int4(_p(x), _p(packed), _p(sc), _p(zp), _p(y), c_int(x.shape[0]), c_int(qw.k), c_int(qw.n),
                          c_int(qw.group_size))
    return y


def spmm(a, x):
    x = _f(x)
    y = torch.empty(a.rows, x.shape[1])
    val = _f(a.val) if a.val is not None else None
    _L().orc_spmm(_p(a.rowptr.cpu().contiguous()), _p(a.col.cpu().contiguous()), _p(val), _p(x), _p(y),
                  c_int(a.rows), c_int(x.shape[1]))
    return y


def dropout(x, p, seed):
    x = _f(x)
    y = torch.empty_like(x)
    _L().orc_dropout(_p(x), _p(y), c_longlong(x.numel()), c_uint(seed & 0xFFFFFFFF), c_float(p))
    return y


class OracleDecoder:
    """The small pre-LN decoder as one chain of oracle kernels (``csrc/cpu_oracle/decoder_baseline.cpp``):
    forward, backward and Adam, single-threaded scalar fp32 like the reference's CPU backend
    (rumus/src/backend/cpu.rs, rumus/src/nn/transformer.rs).  Parameters live in the native object
    in the order of ``GPT.state_dict()``; ``load_state_dict`` copies them in, ``grads`` / ``params``
    hand back tensors under the state-dict names."""

    def __init__(self, cfg, batch: int):
        if getattr(cfg, "activation", "relu") != "relu":
            raise ValueError("the oracle decoder implements the ReLU feed-forward of the functional configuration")
        L = _L()
        L.orc_decoder_create.restype = c_void_p
        L.orc_decoder_tensor.restype = ctypes.POINTER(c_float)
        L.orc_decoder_forward_backward.restype = c_float
        self._L, self.cfg, self.batch = L, cfg, batch
        self._h = c_void_p(L.orc_decoder_create(c_int(cfg.vocab_size), c_int(cfg.seq_len), c_int(cfg.d_model),
                                                c_int(cfg.num_heads), c_int(cfg.num_layers), c_int(cfg.ffn_dim),
                                                c_int(batch)))
        if not self._h:
            raise ValueError("invalid decoder configuration")
        names = ["token_emb.weight", "pos_emb.weight"]
        for l in range(cfg.num_layers):
            b = f"blocks.{l}."
            names += [b + n for n in ("ln1.weight", "ln1.bias", "attn.q_proj.weight", "attn.q_proj.bias",
                                      "attn.k_proj.weight", "attn.k_proj.bias", "attn.v_proj.weight",
                                      "attn.v_proj.bias", "attn.out_proj.weight", "attn.out_proj.bias",
                                      "ln2.weight", "ln2.bias", "mlp_fc1.weight", "mlp_fc1.bias",
                                      "mlp_fc2.weight", "mlp_fc2.bias")]
        names += ["ln_final.weight", "ln_final.bias", "head.weight"]
        assert len(names) == L.orc_decoder_num_tensors(self._h)
        self.names = names

    def _view(self, i, which):
        n = c_longlong(0)
        ptr = self._L.orc_decoder_tensor(self._h, c_int(i), c_int(which), ctypes.byref(n))
        return torch.from_numpy(np.ctypeslib.as_array(ptr, shape=(n.value,)))      # aliases native memory

    def load_state_dict(self, sd):
        for i, name in enumerate(self.names):
            dst = self._view(i, 0)
            src = _f(sd[name]).reshape(-1)
            if src.numel() != dst.numel():
                raise ValueError(f"{name}: {src.numel()} elements, expected {dst.numel()}")
            dst.copy_(src)

    def params(self):
        return {n: self._view(i, 0).clone() for i, n in enumerate(self.names)}

    def grads(self):
        return {n: self._view(i, 1).clone() for i, n in enumerate(self.names)}

    def forward_backward(self, x, y, backward: bool = True) -> float:
        x = x.to(torch.int64).contiguous().reshape(-1)
        y = y.to(torch.int64).contiguous().reshape(-1)
        if x.numel() != self.batch * self.cfg.seq_len or y.numel() != x.numel():
            raise ValueError("token tensors must be [batch, seq_len]")
        return float(self._L.orc_decoder_forward_backward(self._h, _p(x), _p(y), c_int(1 if backward else 0)))

    def adam_step(self, lr=1e-3, betas=(0.9, 0.999), eps=1e-8):
        self._L.orc_decoder_adam(self._h, c_float(lr), c_float(betas[0]), c_float(betas[1]), c_float(eps))

    def close(self):
        if self._h:
            self._L.orc_decoder_destroy(self._h)
            self._h = c_void_p(0)

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
