"""Element-wise fusion JIT.

Reference (rumus/src/jit/): inside ``jit::compile(|| ...)`` the element-wise ops add / mul / relu
do not execute; they record a ``FusedOp`` IR and hand back deferred tensors; at the end of the
block one straight-line kernel is generated, compiled, cached (keyed on the op tags, element count
and dtype) and dispatched (tracer.rs:241-264, codegen.rs:13-121, cache.rs:24-176, mod.rs:41-134).

Here the traced values are ``Lazy`` handles; the generated kernel is CUDA C++ compiled by NVRTC
for sm_100a (through ``rumus_b200.ext``), one thread per 4 elements, cached on
(op program, dtype).  The op set is wider than the reference's three (add, sub, mul, relu,
sigmoid, tanh, gelu, scale).  CPU tensors are evaluated with PyTorch, one op at a time (the fp32
oracle for the generated kernel).
"""
from __future__ import annotations

from typing import Callable, List, Tuple, Union

import torch
import torch.nn.functional as TF

from .. import ext

_CTYPE = {torch.float32: "float", torch.float16: "__half", torch.bfloat16: "__nv_bfloat16"}
_UNARY_SRC = {
    "relu": "fmaxf({0}, 0.0f)",
    "sigmoid": "1.0f / (1.0f + __expf(-{0}))",
    "tanh": "tanhf({0})",
    "gelu": "0.5f * {0} * (1.0f + tanhf(0.7978845608028654f * ({0} + 0.044715f * {0} * {0} * {0})))",
}
_BINARY_SRC = {"add": "{0} + {1}", "sub": "{0} - {1}", "mul": "{0} * {1}"}
_UNARY_TORCH = {"relu": torch.relu, "sigmoid": torch.sigmoid, "tanh": torch.tanh,
                "gelu": lambda t: TF.gelu(t, approximate="tanh")}
_BINARY_TORCH = {"add": torch.add, "sub": torch.sub, "mul": torch.mul}


class Lazy:
    """A value inside a traced block: either an input tensor or the result of a fused op."""

    def __init__(self, tracer: "Tracer", idx: int):
        self.tracer, self.idx = tracer, idx

    def _bin(self, other, op):
        o = other if isinstance(other, Lazy) else self.tracer.input(other) if isinstance(other, torch.Tensor) \
            else None
        if o is None:
            assert op == "mul", "only multiplication by a Python scalar is fused"
            return self.tracer.emit(("scale", self.idx, float(other)))
        return self.tracer.emit((op, self.idx, o.idx))

    def __add__(self, o): return self._bin(o, "add")
    def __sub__(self, o): return self._bin(o, "sub")
    def __mul__(self, o): return self._bin(o, "mul")
    __radd__ = __add__
    __rmul__ = __mul__

    def relu(self): return self.tracer.emit(("relu", self.idx))
    def sigmoid(self): return self.tracer.emit(("sigmoid", self.idx))
    def tanh(self): return self.tracer.emit(("tanh", self.idx))
    def gelu(self): return self.tracer.emit(("gelu", self.idx))


class Tracer:
    def __init__(self):
        self.inputs: List[torch.Tensor] = []
        self.ops: List[tuple] = []          # (tag, operand ids..., [scalar])
        self.nvals = 0

    def input(self, t: torch.Tensor) -> Lazy:
        for i, u in enumerate(self.inputs):
            if u is t:
                return Lazy(self, i)
        assert not self.ops or True
        self.inputs.append(t)
        # inputs occupy value slots [0, n_inputs); ops are renumbered at flush time
        return Lazy(self, -len(self.inputs))   # negative ids mark inputs until flush

    def emit(self, op: tuple) -> Lazy:
        self.ops.append(op)
        return Lazy(self, len(self.ops) - 1)


def _resolve(tr: Tracer):
    """Value numbering: inputs first (0..n-1), then op results."""
    n = len(tr.inputs)
    def vid(i):
        return (-i - 1) if i < 0 else n + i
    prog = []
    for op in tr.ops:
        tag = op[0]
        if tag == "scale":
            prog.append((tag, vid(op[1]), op[2]))
        elif tag in _BINARY_SRC:
            prog.append((tag, vid(op[1]), vid(op[2])))
        else:
            prog.append((tag, vid(op[1])))
    return n, prog


def generate_cuda(n_inputs: int, prog: List[tuple], dtype: torch.dtype, out_val: int) -> Tuple[str, str]:
    """Straight-line fused kernel (reference: codegen.rs:51-119 generates the WGSL twin)."""
    ct = _CTYPE[dtype]
    hdr = "#include <cuda_fp16.h>\n#include <cuda_bf16.h>\n"
    ld = {"float": "{0}", "__half": "__half2float({0})", "__nv_bfloat16": "__bfloat162float({0})"}[ct]
    st = {"float": "{0}", "__half": "__float2half_rn({0})", "__nv_bfloat16": "__float2bfloat16_rn({0})"}[ct]
    params = ", ".join(f"const {ct}* __restrict__ in{i}" for i in range(n_inputs))
    body = [f"  float v{i} = {ld.format(f'in{i}[i]')};" for i in range(n_inputs)]
    scalars = []
    for k, op in enumerate(prog):
        dst = n_inputs + k
        tag = op[0]
        if tag == "scale":
            scalars.append(op[2])
            body.append(f"  float v{dst} = v{op[1]} * s{len(scalars) - 1};")
        elif tag in _BINARY_SRC:
            body.append(f"  float v{dst} = {_BINARY_SRC[tag].format(f'v{op[1]}', f'v{op[2]}')};")
        else:
            body.append(f"  float v{dst} = {_UNARY_SRC[tag].format(f'v{op[1]}')};")
    sparams = "".join(f", float s{i}" for i in range(len(scalars)))
    src = (hdr + f'extern "C" __global__ void fused_kernel({params}, {ct}* __restrict__ out, int n{sparams}) {{\n'
           "  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {\n"
           + "\n".join("  " + b for b in body) + f"\n    out[i] = {st.format(f'v{out_val}')};\n  }}\n}}\n")
    return src, "fused_kernel"


_kernel_cache = {}


def cache_len() -> int:
    return len(_kernel_cache)


def _flush(tr: Tracer, result: Lazy) -> torch.Tensor:
    n, prog = _resolve(tr)
    out_val = (-result.idx - 1) if result.idx < 0 else n + result.idx
    x0 = tr.inputs[0]
    assert all(t.shape == x0.shape and t.dtype == x0.dtype and t.device == x0.device for t in tr.inputs), \
        "fused block needs same-shape, same-dtype inputs"
    if not x0.is_cuda:
        vals = list(tr.inputs)
        for op in prog:
            tag = op[0]
            if tag == "scale":
                vals.append(vals[op[1]] * op[2])
            elif tag in _BINARY_TORCH:
                vals.append(_BINARY_TORCH[tag](vals[op[1]], vals[op[2]]))
            else:
                vals.append(_UNARY_TORCH[tag](vals[op[1]]))
        return vals[out_val]
    key = (tuple((o[0],) + tuple(o[1:3] if o[0] != "scale" else (o[1],)) for o in prog), n, out_val, x0.dtype)
    if key not in _kernel_cache:
        src, entry = generate_cuda(n, prog, x0.dtype, out_val)
        _kernel_cache[key] = ext.compile_cuda(src, entry)
    fn = _kernel_cache[key]
    ins = [t.contiguous() for t in tr.inputs]
    out = torch.empty_like(ins[0])
    numel = out.numel()
    scalars = [numel] + [float(o[2]) for o in prog if o[0] == "scale"]
    grid = min((numel + 255) // 256, 148 * 16)
    ext.launch(fn, (max(grid, 1), 1, 1), (256, 1, 1), ins + [out], scalars)
    return out


def compile(fn: Callable[..., Lazy], *tensors: torch.Tensor) -> torch.Tensor:
    """Trace ``fn`` over lazy handles of ``tensors`` and run the whole chain as ONE kernel
    (reference entry point: ``jit::compile``, tracer.rs:241)."""
    tr = Tracer()
    handles = [tr.input(t) for t in tensors]
    result = fn(*handles)
    assert isinstance(result, Lazy), "the traced function must return a traced value"
    return _flush(tr, result)
