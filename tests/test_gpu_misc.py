"""GPU tests: SpMM kernel, NVRTC custom ops, fused JIT kernels, bounded device-side waits."""
import ctypes

import pytest
import torch
import torch.nn.functional as TF

pytestmark = pytest.mark.gpu


def test_spmm_cuda_matches_dense():
    from rumus_b200.graph import Graph
    torch.manual_seed(0)
    n, e = 300, 2000
    src, dst = torch.randint(0, n, (e,)), torch.randint(0, n, (e,))
    w = torch.rand(e)
    g = Graph.new(n, src, dst, w).to("cuda")
    A = g.adj.dense()
    for feat, dt, tol in ((64, torch.float32, 1e-5), (24, torch.bfloat16, 2e-2), (7, torch.float32, 1e-5)):
        x = torch.randn(n, feat, device="cuda").to(dt).requires_grad_(True)
        y = g.spmm(x)
        y.float().sum().backward()
        ref = A @ x.detach().float()
        assert ((y.float() - ref).norm() / ref.norm()).item() < tol
        gref = A.t() @ torch.ones(n, feat, device="cuda")
        assert ((x.grad.float() - gref).norm() / gref.norm()).item() < tol


def test_custom_op_nvrtc():
    from rumus_b200.ext import CustomOp, cache_size, custom_forward
    src = r'''
extern "C" __global__ void saxpy_sq(const float* a, const float* b, float* out, int n, float alpha) {
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) out[i] = alpha * a[i] * a[i] + b[i];
}'''
    op = CustomOp("saxpy_sq", src, "saxpy_sq", 2, lambda shapes: shapes[0],
                  uniform_data=lambda ins: (ins[0].numel(), 3.0),
                  backward=lambda g, ins, out: (6.0 * ins[0] * g, g),
                  cpu_fn=lambda a, b: 3.0 * a * a + b)
    a = torch.randn(1000, device="cuda", requires_grad=True)
    b = torch.randn(1000, device="cuda", requires_grad=True)
    y = custom_forward(op, a, b)
    y.sum().backward()
    assert torch.allclose(y, 3.0 * a * a + b, atol=1e-5)
    assert torch.allclose(a.grad, 6.0 * a.detach(), atol=1e-5) and torch.allclose(b.grad, torch.ones_like(b))
    n0 = cache_size()
    custom_forward(op, a.detach(), b.detach())
    assert cache_size() == n0          # second use hits the compile cache


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_jit_fused_kernel(dtype):
    from rumus_b200 import jit
    a = torch.randn(100003, device="cuda").to(dtype)
    b = torch.randn(100003, device="cuda").to(dtype)
    y = jit.compile(lambda x, z: ((x + z) * x).relu() * 0.5 + z.gelu(), a, b)
    af, bf = a.float(), b.float()
    ref = torch.relu((af + bf) * af) * 0.5 + TF.gelu(bf, approximate="tanh")
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    assert ((y.float() - ref).norm() / ref.norm()).item() < tol
    n0 = jit.cache_len()
    jit.compile(lambda x, z: ((x + z) * x).relu() * 0.25 + z.gelu(), a, b)   # same program, new scalar
    assert jit.cache_len() == n0


def test_bounded_wait_times_out_and_context_survives():
    """A device-side wait on a flag that nothing sets gives up after its budget, reports through the
    status word, and the kernel returns: the context stays usable."""
    from rumus_b200.ops import native
    from rumus_b200.ops._lib import ptr, stream_ptr
    L = native.lib()
    L.rb_wait_flag_probe.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_void_p,
                                     ctypes.c_void_p]
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    res = torch.full((1,), -1, dtype=torch.int32, device="cuda")
    assert native.read_status() == 0
    assert L.rb_wait_flag_probe(ptr(flag), 1, 200, ptr(res), stream_ptr()) == 0
    torch.cuda.synchronize()
    assert res.item() == 0
    with pytest.raises(native.DeviceWaitTimeout):
        native.raise_on_status("probe")
    assert native.read_status() == 0            # cleared by the read
    flag.fill_(5)                               # a satisfied wait returns at once
    assert L.rb_wait_flag_probe(ptr(flag), 5, 200, ptr(res), stream_ptr()) == 0
    torch.cuda.synchronize()
    assert res.item() == 1 and native.read_status() == 0
    assert torch.allclose(native.gemm(torch.ones(128, 64, device="cuda").bfloat16(),
                                      torch.ones(64, 128, device="cuda").bfloat16(), path=1).float(),
                          torch.full((128, 128), 64.0, device="cuda"))


def test_grad_scaler_device_side_update_kernel():
    """The loss-scale update kernel: halve after an overflow, double after `growth_interval` clean steps,
    reciprocal kept in step — all without a host read of the flag."""
    import torch
    from rumus_b200.optim import GradScaler
    sc = GradScaler(init_scale=64.0, growth_interval=3, device_side=True)
    sc._ensure(torch.device("cuda"))
    seen = []
    for bad in (1, 0, 0, 0, 0, 1, 0):
        sc.found_inf.fill_(bad)
        assert sc.update() is None
        seen.append((sc.scale_value, float(sc.inv_scale), int(sc._good_dev)))
    assert [s for s, _, _ in seen] == [32.0, 32.0, 32.0, 64.0, 64.0, 32.0, 32.0]
    assert all(abs(i * s - 1.0) < 1e-6 for s, i, _ in seen)
    assert [g for _, _, g in seen] == [0, 1, 2, 3, 4, 0, 1]
    assert float(sc.scale(torch.ones((), device="cuda"))) == 32.0
