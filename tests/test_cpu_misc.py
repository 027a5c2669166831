"""CPU tests: C++ oracle vs PyTorch, data engine, graph, ONNX export, JIT, custom ops, checkpoints."""
import os

import pytest
import torch
import torch.nn as nn
import torch.nn.functional as TF

import rumus_b200.nn as rnn
from rumus_b200 import oracle
from rumus_b200.ops import functional as F


def test_cpu_oracle_agrees_with_pytorch():
    torch.manual_seed(0)
    a, b = torch.randn(7, 5), torch.randn(5, 9)
    assert torch.allclose(oracle.matmul(a, b), a @ b, atol=1e-5)
    x = torch.randn(6, 11)
    assert torch.allclose(oracle.unary("gelu", x), TF.gelu(x, approximate="tanh"), atol=1e-6)
    assert torch.allclose(oracle.unary("leaky_relu", x, 0.1), TF.leaky_relu(x, 0.1))
    assert torch.allclose(oracle.softmax(x), torch.softmax(x, -1), atol=1e-6)
    w, bb = torch.randn(11), torch.randn(11)
    y, save = oracle.layer_norm(x, w, bb)
    assert torch.allclose(y, TF.layer_norm(x, (11,), w, bb), atol=1e-5)
    xr = x.clone().requires_grad_(True); wr = w.clone().requires_grad_(True); br = bb.clone().requires_grad_(True)
    g = torch.randn(6, 11)
    TF.layer_norm(xr, (11,), wr, br).backward(g)
    dx, dw, db = oracle.layer_norm_backward(x, w, g, save)
    assert torch.allclose(dx, xr.grad, atol=1e-5) and torch.allclose(dw, wr.grad, atol=1e-5)
    t = torch.randint(0, 11, (6,))
    loss, grad = oracle.cross_entropy(x, t)
    xr = x.clone().requires_grad_(True)
    lr = TF.cross_entropy(xr, t); lr.backward()
    assert abs(loss - lr.item()) < 1e-5 and torch.allclose(grad, xr.grad, atol=1e-6)
    img, k = torch.randn(2, 3, 9, 8), torch.randn(4, 3, 3, 3)
    assert torch.allclose(oracle.conv2d(img, k, None, 2, 1, 1), TF.conv2d(img, k, None, 2, 1), atol=1e-4)
    q, kk, v = torch.randn(3, 10, 8), torch.randn(3, 10, 8), torch.randn(3, 10, 8)
    ref = F.sdpa_reference(q[:, :, None], kk[:, :, None], v[:, :, None], True)[:, :, 0]
    assert torch.allclose(oracle.flash_attention(q, kk, v, True), ref, atol=1e-5)
    from rumus_b200.nn.quant import QuantizedTensor
    qw = QuantizedTensor.from_f32(torch.randn(64, 6), 32)
    xm = torch.randn(3, 64)
    assert torch.allclose(oracle.qmatmul_int4(xm, qw), xm @ qw.dequantize(), atol=1e-4)


def test_oracle_decoder_step_matches_framework_decoder():
    """End-to-end second opinion: loss, every gradient and two Adam steps of the scalar C++ decoder
    chain against the framework's GPT on the same weights."""
    from rumus_b200.models import GPT, GPTConfig
    from rumus_b200.optim import Adam
    cfg = GPTConfig(vocab_size=96, seq_len=12, d_model=32, num_heads=4, num_layers=2, ffn_dim=48, activation="relu")
    m = GPT(cfg, device="cpu", dtype=torch.float32)
    m.init_weights(0.05, seed=3)
    torch.manual_seed(4)
    with torch.no_grad():
        for p in m.parameters():
            if p.dim() == 1:
                p.add_(0.1 * torch.randn_like(p))
    tok = torch.randint(0, cfg.vocab_size, (3, cfg.seq_len + 1))
    x, y = tok[:, :-1], tok[:, 1:]
    dec = oracle.OracleDecoder(cfg, 3)
    dec.load_state_dict(m.state_dict())
    loss = m(x, y)
    loss.backward()
    assert abs(dec.forward_backward(x, y) - loss.item()) < 1e-5
    g, d = dec.grads(), cfg.d_model
    for n, p in m.named_parameters():
        if n.endswith("qkv_weight"):
            ref = torch.cat([g[n.replace("qkv_weight", f"{c}_proj.weight")].view(d, d) for c in "qkv"], 1)
        elif n.endswith("qkv_bias"):
            ref = torch.cat([g[n.replace("qkv_bias", f"{c}_proj.bias")] for c in "qkv"])
        else:
            ref = g[n]
        assert torch.allclose(p.grad.reshape(-1), ref.reshape(-1), atol=1e-6, rtol=1e-4), n
    opt = Adam(m.parameters(), lr=1e-3)
    for _ in range(2):
        l = m(x, y); opt.zero_grad(); l.backward(); opt.step()
        lo = dec.forward_backward(x, y); dec.adam_step(1e-3)
        assert abs(lo - l.item()) < 1e-4
    with pytest.raises(ValueError):
        dec.forward_backward(x[:, :-1], y[:, :-1])
    dec.close()


def test_dropout_matches_reference_hash_on_cpu_oracle():
    x = torch.ones(4096)
    y = oracle.dropout(x, 0.25, 99)
    keep = (y != 0).float().mean().item()
    assert abs(keep - 0.75) < 0.03 and torch.allclose(y[y != 0], torch.tensor(1 / 0.75))


def test_data_engine(tmp_path):
    from rumus_b200.data import DataLoader, RecordDataset, RecordWriter, SyntheticTokens, TensorDataset
    p = str(tmp_path / "d.rrec")
    w = RecordWriter.create(p)
    xs = [torch.randn(3, 5) for _ in range(7)]
    ys = [torch.randn(2).half() for _ in range(7)]
    for x, y in zip(xs, ys):
        w.append(x, y)
    w.finish()
    raw = open(p, "rb").read()
    assert raw[:4] == b"RREC" and len(raw) % 4 == 0
    for force_py in (False, True):
        ds = RecordDataset(p, force_python=force_py)
        assert len(ds) == 7
        for i in range(7):
            it = ds.get(i)
            assert torch.equal(it.input, xs[i]) and torch.equal(it.target, ys[i]) and it.target.dtype == torch.float16
    ds = TensorDataset(torch.arange(10).float()[:, None], torch.arange(10).float())
    for workers in (0, 3):
        dl = DataLoader(ds, 4, shuffle=False, drop_last=False, num_workers=workers)
        got = torch.cat([b.input[:, 0] for b in dl])
        assert torch.equal(got, torch.arange(10).float()) and len(dl) == 3
    dl = DataLoader(ds, 4, shuffle=True, drop_last=True, num_workers=2)
    seen = torch.cat([b.target for b in dl])
    assert seen.numel() == 8 and len(set(seen.tolist())) == 8
    # early teardown of a threaded iterator must not hang
    it = iter(DataLoader(ds, 1, num_workers=2, prefetch_factor=1))
    next(it); del it
    st = SyntheticTokens(4, 16, 100, seed=0)
    a = st.get(1)
    assert torch.equal(a.input[1:], a.target[:-1])


def test_native_batch_loader_matches_python_loader(tmp_path):
    """C++ worker threads + pinned ring vs the Python DataLoader over the same .rrec file: same
    batches in the same order, with and without shuffling, short last batch, several epochs."""
    from rumus_b200.data import DataLoader, NativeBatchLoader, RecordDataset, RecordWriter
    from rumus_b200.data import dataloader as dl_mod
    p = str(tmp_path / "tok.rrec")
    w = RecordWriter.create(p)
    g = torch.Generator().manual_seed(0)
    for i in range(37):
        w.append(torch.randn(6, 4, generator=g), torch.full((3,), float(i)).half())
    w.finish()
    ds = RecordDataset(p)
    for shuffle, drop_last in ((False, False), (True, False), (True, True)):
        nat = NativeBatchLoader(p, 8, shuffle=shuffle, drop_last=drop_last, num_workers=3,
                                prefetch_batches=2, pin_memory=False)
        dl_mod._shuffle_rng = dl_mod._Lcg()       # both shuffles start from the reference seed
        py = DataLoader(ds, 8, shuffle=shuffle, drop_last=drop_last)
        assert len(nat) == len(py)
        for epoch in range(3):
            a = [(b.input.clone(), b.target.clone()) for b in nat]
            b = [(it.input, it.target) for it in py]
            assert len(a) == len(b) == len(py)
            for (xa, ya), (xb, yb) in zip(a, b):
                assert torch.equal(xa, xb) and torch.equal(ya, yb) and ya.dtype == torch.float16
        nat.close()
    # stopping in the middle of an epoch and starting the next one must not hang or mix epochs
    nat = NativeBatchLoader(p, 4, shuffle=False, num_workers=2, prefetch_batches=3, pin_memory=False)
    it = iter(nat)
    first = next(it).target[:, 0].clone()
    del it
    again = torch.cat([b.target[:, 0].clone() for b in nat])
    assert torch.equal(first, torch.arange(4).half()) and torch.equal(again, torch.arange(37).half())
    nat.close()


def test_graph_spmm_and_oracle():
    from rumus_b200.graph import Graph
    g = Graph.new(5, [0, 1, 2, 3, 0], [1, 2, 3, 4, 4], [1., 2., 3., 4., 5.])
    x = torch.randn(5, 3, requires_grad=True)
    y = g.spmm(x)
    y.sum().backward()
    A = g.adj.dense()
    assert torch.allclose(y, A @ x) and torch.allclose(x.grad, A.t() @ torch.ones(5, 3))
    assert torch.allclose(oracle.spmm(g.adj, x.detach()), A @ x.detach(), atol=1e-6)


def test_onnx_export_structure(tmp_path):
    from rumus_b200.io.onnx_export import export_onnx, parse_model

    class M(rnn.Module):
        def __init__(self):
            super().__init__()
            self.hidden, self.output = rnn.Linear(2, 8), rnn.Linear(8, 1)

        def forward(self, x):
            return self.output(F.relu(self.hidden(x)))

    m = M()
    p = str(tmp_path / "m.onnx")
    pm = parse_model(export_onnx(m, [torch.randn(4, 2)], p))
    assert os.path.getsize(p) > 0
    assert (pm["ir_version"], pm["producer_name"], pm["opset"]) == (9, "rumus", 17)
    assert [n["op_type"] for n in pm["nodes"]] == ["Gemm", "Relu", "Gemm"]
    assert pm["initializers"]["hidden.weight"].shape == (2, 8)
    assert torch.allclose(torch.from_numpy(pm["initializers"]["hidden.weight"].copy()), m.hidden.weight.detach())
    cnn = nn.Sequential(rnn.Conv2d(1, 4, 3, 1, 1), nn.ReLU(), rnn.MaxPool2d(2), rnn.Flatten(), rnn.Linear(64, 4))
    pm = parse_model(export_onnx(cnn, [torch.randn(2, 1, 8, 8)]))
    assert [n["op_type"] for n in pm["nodes"]] == ["Conv", "Relu", "MaxPool", "Flatten", "Gemm"]
    assert pm["initializers"]["0.weight"].shape == (4, 1, 3, 3)


def test_jit_fused_chain_cpu_and_codegen():
    from rumus_b200 import jit
    a, b = torch.randn(100), torch.randn(100)
    y = jit.compile(lambda x, z: ((x + z) * x).relu() * 0.5 + z.gelu(), a, b)
    assert torch.allclose(y, torch.relu((a + b) * a) * 0.5 + TF.gelu(b, approximate="tanh"), atol=1e-6)
    src, entry = jit.generate_cuda(2, [("add", 0, 1), ("relu", 2), ("scale", 3, 2.0)], torch.bfloat16, 4)
    assert entry == "fused_kernel" and "fmaxf(v2, 0.0f)" in src and "float s0" in src


def test_custom_op_cpu_path_and_backward():
    from rumus_b200.ext import CustomOp, custom_forward
    op = CustomOp("square_plus", "", "k", 2, lambda shapes: shapes[0], cpu_fn=lambda a, b: a * a + b,
                  backward=lambda g, ins, out: (2 * ins[0] * g, g))
    a = torch.randn(5, requires_grad=True); b = torch.randn(5, requires_grad=True)
    y = custom_forward(op, a, b)
    y.sum().backward()
    assert torch.allclose(y, a * a + b) and torch.allclose(a.grad, 2 * a.detach()) and torch.allclose(b.grad, torch.ones(5))


def test_custom_op_registered_with_the_dispatcher():
    """A CustomOp as torch.ops.<ns>.<name>: schema, CPU kernel, shape-only kernel, autograd formula."""
    from torch._subclasses.fake_tensor import FakeTensorMode
    from rumus_b200.ext import CustomOp, register_torch_op
    src = ("extern \"C\" __global__ void k(const float* a, const float* b, float* o, int n) {"
           " int i = blockIdx.x * blockDim.x + threadIdx.x; if (i < n) o[i] = a[i] + 2.f * b[i]; }")
    op = CustomOp("scaled_add_for_test", src, "k", 2, output_shape=lambda shapes: shapes[0],
                  backward=lambda g, ins, out: (g, 2 * g), cpu_fn=lambda a, b: a + 2 * b)
    f = register_torch_op(op)
    assert register_torch_op(op) is f
    a = torch.randn(5, requires_grad=True)
    b = torch.randn(5, requires_grad=True)
    y = torch.ops.rumus_b200_ext.scaled_add_for_test(a, b)
    assert torch.allclose(y, a + 2 * b)
    y.sum().backward()
    assert torch.equal(a.grad, torch.ones(5)) and torch.equal(b.grad, 2 * torch.ones(5))
    res = torch.library.opcheck(f, (a.detach().requires_grad_(), b.detach().requires_grad_()),
                                test_utils=("test_schema", "test_autograd_registration", "test_faketensor"))
    assert set(res.values()) == {"SUCCESS"}
    with FakeTensorMode():
        assert f(torch.empty(3, 4), torch.empty(3, 4)).shape == (3, 4)


def _fd_exchange_child(rank, world, d, q, late):
    import ctypes
    import time
    from rumus_b200.ops import _lib
    if late and rank == 0:
        time.sleep(0.3)                       # peers must retry until this rank listens
    fd = os.memfd_create(f"rank{rank}")
    os.write(fd, f"payload-of-rank-{rank}".encode())
    fds = (ctypes.c_int * world)()
    rc = _lib.host_lib().rb_fd_exchange(d.encode(), ctypes.c_int(rank), ctypes.c_int(world), ctypes.c_int(fd),
                                        fds, ctypes.c_int(10000))
    seen = []
    if rc == 0:
        for r in range(world):
            seen.append(os.pread(fds[r], 64, 0).decode())
    q.put((rank, rc, seen))


def test_fd_exchange_between_processes(tmp_path):
    """Every rank hands one descriptor (here: a memfd with a rank-specific payload) to every other
    process over Unix sockets, including a rank that starts listening late; a missing rank makes
    the others time out with a status code instead of blocking."""
    import ctypes
    import multiprocessing as mp
    from rumus_b200.ops import _lib
    ctx = mp.get_context("spawn")
    world = 3
    q = ctx.Queue()
    procs = [ctx.Process(target=_fd_exchange_child, args=(r, world, str(tmp_path), q, True)) for r in range(world)]
    for p in procs:
        p.start()
    got = sorted(q.get(timeout=60) for _ in range(world))
    for p in procs:
        p.join(timeout=30)
    for rank, rc, seen in got:
        assert rc == 0 and seen == [f"payload-of-rank-{r}" for r in range(world)]
    # a peer that never shows up: bounded wait, status 3
    fds = (ctypes.c_int * 2)()
    fd = os.memfd_create("alone")
    rc = _lib.host_lib().rb_fd_exchange(str(tmp_path).encode(), ctypes.c_int(0), ctypes.c_int(2), ctypes.c_int(fd),
                                        fds, ctypes.c_int(300))
    os.close(fd)
    assert rc == 3 and fds[1] == -1


def test_canary_guard_detects_out_of_bounds_writes():
    """Bounds-guard mode on CPU tensors: clean runs pass, an overrun on either side is reported with
    the allocation site; tensors allocated without an explicit device are left alone."""
    from rumus_b200.utils.canary import CanaryError, canary_guard
    with canary_guard(devices=("cpu",)) as g:
        a = torch.empty((3, 5), dtype=torch.float32, device="cpu")
        b = torch.zeros(7, dtype=torch.int64, device="cpu")
        c = torch.empty_like(a)
        d = torch.empty_strided((2, 3), (3, 1), dtype=torch.float16, device="cpu")
        torch.empty(4)
        a.fill_(1); c.copy_(a); d.fill_(2)
        assert b.sum().item() == 0 and a.is_contiguous() and g.check() == 4
    with pytest.raises(CanaryError, match=r"\(3, 5\).*after the tensor.*\+0 from its end"):
        with canary_guard(devices=("cpu",)):
            a = torch.empty((3, 5), dtype=torch.float32, device="cpu")
            torch.as_strided(a, (17,), (1,)).fill_(3.0)
    with pytest.raises(CanaryError, match="before the tensor"):
        with canary_guard(devices=("cpu",)):
            a = torch.empty((8,), dtype=torch.float32, device="cpu")
            torch.as_strided(a, (1,), (1,), storage_offset=a.storage_offset() - 1).fill_(3.0)


def test_split_k_workspaces_are_dropped_after_a_bad_device_status():
    """A kernel that gave up on a bounded wait may leave the shared split-K workspace and tile counters
    non-zero; reading a non-zero status word runs the registered hooks, which drop the cached buffers so
    that the next call starts from fresh zeros."""
    import torch
    from rumus_b200.ops import native, quant_cuda
    assert quant_cuda._W4_WS.clear in native._BAD_STATUS_HOOKS
    quant_cuda._W4_WS[("cpu", None, 0)] = (torch.ones(4), torch.ones(4, dtype=torch.int32))
    for fn in native._BAD_STATUS_HOOKS:
        fn()
    assert not quant_cuda._W4_WS
