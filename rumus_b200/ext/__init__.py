"""Custom-op plug-in API.

Reference: ``trait CustomOp`` (name, shader source, entry point, number of inputs, output shape,
workgroup size, dispatch size, uniform data, optional backward handler) and ``custom_forward``
(compile-cache -> allocate output -> bind N inputs + 1 output + uniforms -> dispatch -> record a
custom backward node), rumus/src/ext/mod.rs:52-272.

Here the kernel source is CUDA C++, compiled at first use with NVRTC for sm_100a and cached by
source hash (the counterpart of the reference's ``CustomOpCache``); launches go through the
driver API on the caller's current stream.  Kernel signature convention:

    extern "C" __global__ void entry(const T* in0, ..., const T* inN-1, T* out, <uniforms...>)

Uniforms are passed as a tuple of Python ints / floats (int32 / float32 kernel parameters).
CPU tensors use the op's ``cpu_fn`` (plain PyTorch), which is also the test oracle.
"""
from __future__ import annotations

import ctypes
import hashlib
import threading
from typing import Callable, Optional, Sequence, Tuple

import numpy as np
import torch

_cache = {}
_lock = threading.Lock()


class CustomOpError(RuntimeError):
    pass


def compile_cuda(source: str, entry: str, arch: str = "sm_100a"):
    """NVRTC-compile ``source`` and return a ``CUfunction`` (cached per (source, entry))."""
    key = hashlib.sha1((arch + entry + source).encode()).hexdigest()
    with _lock:
        if key in _cache:
            return _cache[key][1]
    from cuda.bindings import driver, nvrtc

    def chk(res):
        err = res[0]
        if int(err) != 0:
            raise CustomOpError(f"CUDA/NVRTC error {err}")
        return res[1:] if len(res) > 1 else None

    (prog,) = chk(nvrtc.nvrtcCreateProgram(source.encode(), b"custom_op.cu", 0, [], []))
    import os
    inc = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "include")
    opts = [f"--gpu-architecture={arch}".encode(), b"--std=c++17", b"-default-device",
            f"--include-path={inc}".encode()]
    res = nvrtc.nvrtcCompileProgram(prog, len(opts), opts)
    if int(res[0]) != 0:
        (n,) = chk(nvrtc.nvrtcGetProgramLogSize(prog))
        log = b" " * n
        nvrtc.nvrtcGetProgramLog(prog, log)
        raise CustomOpError("NVRTC compilation failed:\n" + log.decode(errors="replace"))
    (n,) = chk(nvrtc.nvrtcGetCUBINSize(prog))
    cubin = b" " * n
    chk(nvrtc.nvrtcGetCUBIN(prog, cubin))
    torch.cuda.init()
    torch.zeros(1, device="cuda")   # make sure the primary context is current on this thread
    (module,) = chk(driver.cuModuleLoadData(np.char.array(cubin).ctypes.data))
    (fn,) = chk(driver.cuModuleGetFunction(module, entry.encode()))
    with _lock:
        _cache[key] = (module, fn)
    return fn


def cache_size() -> int:
    return len(_cache)


def launch(fn, grid: Tuple[int, int, int], block: Tuple[int, int, int], tensors: Sequence[torch.Tensor],
           scalars: Sequence = (), shared_bytes: int = 0) -> None:
    from cuda.bindings import driver
    vals, types = [], []
    for t in tensors:
        vals.append(t.data_ptr()); types.append(ctypes.c_void_p)
    for s in scalars:
        if isinstance(s, float):
            vals.append(s); types.append(ctypes.c_float)
        else:
            vals.append(int(s)); types.append(ctypes.c_int)
    stream = torch.cuda.current_stream().cuda_stream
    err = driver.cuLaunchKernel(fn, *grid, *block, shared_bytes, stream, (tuple(vals), tuple(types)), 0)
    if int(err[0]) != 0:
        raise CustomOpError(f"cuLaunchKernel failed: {err[0]}")
    from ..ops._lib import count_launch
    count_launch()


class CustomOp:
    """Subclass or instantiate with the pieces the reference trait asks for."""

    def __init__(self, name: str, cuda_source: str, entry: str, num_inputs: int,
                 output_shape: Callable[[Sequence[torch.Size]], Sequence[int]],
                 block_size: int = 256,
                 grid: Optional[Callable[[int], int]] = None,
                 uniform_data: Optional[Callable[[Sequence[torch.Tensor]], Sequence]] = None,
                 backward: Optional[Callable] = None,
                 cpu_fn: Optional[Callable] = None,
                 save_for_backward: bool = True):
        self.name, self.cuda_source, self.entry, self.num_inputs = name, cuda_source, entry, num_inputs
        self.output_shape, self.block_size = output_shape, block_size
        self.grid = grid or (lambda numel: (numel + block_size - 1) // block_size)
        self.uniform_data = uniform_data or (lambda inputs: (int(np.prod(output_shape([i.shape for i in inputs]))),))
        self.backward, self.cpu_fn, self.save = backward, cpu_fn, save_for_backward


class _CustomFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, op: CustomOp, *inputs):
        out_shape = tuple(op.output_shape([i.shape for i in inputs]))
        if inputs[0].is_cuda:
            ins = [i.contiguous() for i in inputs]
            out = torch.empty(out_shape, dtype=ins[0].dtype, device=ins[0].device)
            fn = compile_cuda(op.cuda_source, op.entry)
            numel = out.numel()
            launch(fn, (op.grid(numel), 1, 1), (op.block_size, 1, 1), ins + [out], op.uniform_data(ins))
        else:
            if op.cpu_fn is None:
                raise CustomOpError(f"custom op {op.name!r} has no cpu_fn")
            out = op.cpu_fn(*inputs)
        ctx.op = op
        if op.save:
            ctx.save_for_backward(*inputs, out)
        return out

    @staticmethod
    def backward(ctx, grad_out):
        op = ctx.op
        if op.backward is None:
            raise CustomOpError(f"custom op {op.name!r} has no backward handler")
        saved = ctx.saved_tensors
        inputs, out = saved[:-1], saved[-1]
        grads = op.backward(grad_out, inputs, out)
        if isinstance(grads, torch.Tensor):
            grads = (grads,)
        return (None, *grads)


def custom_forward(op: CustomOp, *inputs: torch.Tensor) -> torch.Tensor:
    """Run ``op`` on ``inputs`` (reference: ext/mod.rs:122)."""
    assert len(inputs) == op.num_inputs, f"{op.name}: expected {op.num_inputs} inputs"
    return _CustomFn.apply(op, *inputs)


# ------------------------------------------------------------------ dispatcher registration
_registered = {}


def register_torch_op(op: CustomOp, namespace: str = "rumus_b200_ext"):
    """Registers ``op`` with PyTorch's dispatcher as ``torch.ops.<namespace>.<op.name>`` and returns
    the callable.

    The reference's plug-in point is the ``CustomOp`` trait + ``BackwardOp::Custom`` tape entry
    (rumus/src/ext/mod.rs:52-110, rumus/src/autograd/backward_ops.rs:502-528); with PyTorch as the
    tensor layer the native counterpart is a dispatcher operator, which — unlike a bare
    ``autograd.Function`` — carries a schema, has separate CPU and CUDA kernels, a shape-only
    ("fake") kernel so that the op can be traced and exported, and an autograd formula:

    * CPU kernel   = ``op.cpu_fn``;
    * CUDA kernel  = the NVRTC-compiled source launched on the current stream;
    * fake kernel  = ``op.output_shape`` (no data);
    * autograd     = ``op.backward(grad_out, inputs, out)`` when the op has a backward handler.

    Registering the same op name twice returns the first registration.
    """
    qual = f"{namespace}::{op.name}"
    with _lock:
        if qual in _registered:
            return _registered[qual]
    args = ", ".join(f"Tensor in{i}" for i in range(op.num_inputs))
    torch.library.define(qual, f"({args}) -> Tensor")

    def cuda_impl(*inputs):
        ins = [i.contiguous() for i in inputs]
        out = torch.empty(tuple(op.output_shape([i.shape for i in ins])), dtype=ins[0].dtype, device=ins[0].device)
        fn = compile_cuda(op.cuda_source, op.entry)
        launch(fn, (op.grid(out.numel()), 1, 1), (op.block_size, 1, 1), ins + [out], op.uniform_data(ins))
        return out

    def cpu_impl(*inputs):
        if op.cpu_fn is None:
            raise CustomOpError(f"custom op {op.name!r} has no cpu_fn")
        out = op.cpu_fn(*inputs)
        # a dispatcher kernel must not return one of its inputs
        return out.clone() if any(out is i for i in inputs) else out

    def fake_impl(*inputs):
        return inputs[0].new_empty(tuple(op.output_shape([i.shape for i in inputs])))

    torch.library.impl(qual, "CUDA")(cuda_impl)
    torch.library.impl(qual, "CPU")(cpu_impl)
    torch.library.register_fake(qual)(fake_impl)

    if op.backward is not None:
        def setup_context(ctx, inputs, output):
            if op.save:
                ctx.save_for_backward(*inputs, output)

        def backward(ctx, grad_out):
            saved = ctx.saved_tensors
            grads = op.backward(grad_out, saved[:-1], saved[-1])
            return grads if isinstance(grads, (tuple, list)) and len(grads) > 1 else (
                grads[0] if isinstance(grads, (tuple, list)) else grads)

        torch.library.register_autograd(qual, backward, setup_context=setup_context)

    fn = getattr(getattr(torch.ops, namespace), op.name)
    with _lock:
        _registered[qual] = fn
    return fn
