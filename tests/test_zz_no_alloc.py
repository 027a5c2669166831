"""The allocation-free norm-backward entry point, called through its exported C symbol.

Some users of the library cannot allocate device memory when they need this kernel (fixed memory
budgets, code running inside someone else's pool or under a lock where cudaMalloc is off limits),
so ``rb_norm_bwd_noalloc`` keeps its scratch in an array built into the library.  The test drives
the raw symbol with ctypes — no helper from the package in between — and checks it against the
regular entry point and against a plain fp32 PyTorch backward on two back-to-back calls (the second
reuses the array with different sizes, so leftovers of the first call must not matter; one of them
passes a gradient to add to dx), plus the size refusal.

Collected last on purpose: a ``-x`` run has already exercised everything else when it gets here.
"""
import ctypes
from ctypes import c_int, c_longlong, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu


def _rel(a, b):
    a, b = a.float(), b.float()
    return ((a - b).norm() / (b.norm() + 1e-12)).item()


def _call_noalloc(lib, x, dy, gamma, stats, rms, dres=None):
    rows, D = x.shape
    dx = torch.empty_like(x)
    dgamma = torch.empty_like(gamma)
    dbeta = torch.empty_like(gamma)
    code = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}[x.dtype]
    rc = lib.rb_norm_bwd_noalloc(code, 1 if rms else 0, c_void_p(x.data_ptr()),
                                 c_void_p(dy.data_ptr()), c_void_p(gamma.data_ptr()),
                                 c_void_p(stats.data_ptr()),
                                 c_void_p(dres.data_ptr() if dres is not None else 0), c_void_p(dx.data_ptr()),
                                 c_void_p(dgamma.data_ptr()), c_void_p(dbeta.data_ptr()),
                                 c_longlong(rows), c_int(D),
                                 c_void_p(torch.cuda.current_stream().cuda_stream))
    return rc, dx, dgamma, dbeta


def test_norm_bwd_noalloc_matches_regular_entry_point_twice():
    from rumus_b200.ops import _lib, native
    lib = ctypes.CDLL(_lib.cuda_lib_path())
    lib.rb_norm_bwd_noalloc.restype = c_int
    lib.rb_norm_bwd_noalloc.argtypes = [c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                                        c_void_p, c_void_p, c_void_p, c_void_p, c_longlong, c_int,
                                        c_void_p]
    lib.rb_norm_bwd_noalloc_max_dim.restype = c_int
    max_dim = lib.rb_norm_bwd_noalloc_max_dim()
    assert max_dim == 4096
    torch.manual_seed(7)
    cases = [(torch.bfloat16, 3000, 2048, False, True), (torch.float32, 517, 264, True, False)]
    for dtype, rows, D, rms, with_dres in cases:      # two calls in a row on the shared array
        x = torch.randn(rows, D, device="cuda").to(dtype)
        dy = torch.randn(rows, D, device="cuda").to(dtype)
        gamma = (1 + 0.1 * torch.randn(D, device="cuda")).to(dtype)
        beta = torch.zeros(D, device="cuda").to(dtype)
        dres = torch.randn(rows, D, device="cuda").to(dtype) if with_dres else None
        _, _, stats = native.norm_fwd(x, gamma, None if rms else beta, 1e-5, rms)
        ref_dx, ref_dg, ref_db = native.norm_bwd(x, dy, gamma, stats, rms, dres=dres)
        rc, dx, dg, db = _call_noalloc(lib, x, dy, gamma, stats, rms, dres)
        assert rc == 0
        torch.cuda.synchronize()
        tol = 2e-2 if dtype == torch.bfloat16 else 1e-4
        assert _rel(dx, ref_dx) < tol
        assert _rel(dg, ref_dg) < tol
        if not rms:
            assert _rel(db, ref_db) < tol
        # the same gradients from plain fp32 PyTorch math
        xf = x.float().requires_grad_(True)
        gf = gamma.float().requires_grad_(True)
        bf = beta.float().requires_grad_(True)
        if rms:
            yf = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-5) * gf
        else:
            yf = torch.nn.functional.layer_norm(xf, (D,), gf, bf, 1e-5)
        yf.backward(dy.float())
        want_dx = xf.grad + (dres.float() if dres is not None else 0)
        assert _rel(dx, want_dx) < tol
        assert _rel(dg, gf.grad) < tol
        if not rms:
            assert _rel(db, bf.grad) < tol
    # a row longer than the built-in array is refused, nothing runs
    D = max_dim + 8
    x = torch.randn(4, D, device="cuda")
    stats = torch.zeros(4, 2, device="cuda")
    rc, *_ = _call_noalloc(lib, x, x, torch.ones(D, device="cuda"), stats, False)
    assert rc == 40
    assert native.read_status() == 0
