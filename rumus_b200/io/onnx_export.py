"""ONNX export (reference: rumus/src/onnx/{tracer,export}.rs + rumus/proto/onnx.proto).

The reference traces a forward closure — primitive hooks in add / mul / matmul / relu, and
``Linear`` / ``Conv2d`` fused into single ``Gemm`` / ``Conv`` nodes — and writes a ModelProto
(IR version 9, opset 17 by default, producer "rumus") with prost.

Here the trace comes from forward hooks on the leaf modules of a model built from this package's
layers (each module becomes one ONNX node, so ``Linear`` -> ``Gemm`` and ``Conv2d`` -> ``Conv`` are
fused by construction) plus hooks on the functional add / mul / matmul / relu ops used between
modules.  The protobuf wire format is emitted by a small encoder in this file (no ``onnx``
package needed); ``parse_model`` decodes it again for tests and inspection.

Weights are exported in ONNX conventions: ``Gemm`` gets ``B = weight`` with ``transB = 0`` because
this framework already stores ``[in, out]``; ``Conv`` gets the 2-D ``[C_out, C_in*K*K]`` weight
reshaped to 4-D.
"""
from __future__ import annotations

import struct
from typing import Callable, Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch
import torch.nn as nn

from .. import nn as rnn
from ..ops import functional as F

# ----------------------------------------------------------------------------- protobuf writer
def _varint(n: int) -> bytes:
    n &= (1 << 64) - 1
    out = bytearray()
    while True:
        b = n & 0x7F
        n >>= 7
        if n:
            out.append(b | 0x80)
        else:
            out.append(b)
            return bytes(out)


def _key(field: int, wire: int) -> bytes:
    return _varint((field << 3) | wire)


def f_varint(field: int, v: int) -> bytes:
    return _key(field, 0) + _varint(v)


def f_bytes(field: int, b: bytes) -> bytes:
    return _key(field, 2) + _varint(len(b)) + b


def f_str(field: int, s: str) -> bytes:
    return f_bytes(field, s.encode())


def f_float(field: int, v: float) -> bytes:
    return _key(field, 5) + struct.pack("<f", v)


FLOAT, FLOAT16, INT64 = 1, 10, 7


def tensor_proto(name: str, t: torch.Tensor) -> bytes:
    """TensorProto: dims=1, data_type=2, name=8, raw_data=9.  F16 raw bytes are preserved."""
    if t.dtype == torch.float16:
        dt, arr = FLOAT16, t.detach().cpu().contiguous().numpy()
    elif t.dtype == torch.int64:
        dt, arr = INT64, t.detach().cpu().contiguous().numpy()
    else:
        dt, arr = FLOAT, t.detach().cpu().float().contiguous().numpy()
    msg = b"".join(f_varint(1, int(d)) for d in arr.shape)
    msg += f_varint(2, dt) + f_str(8, name) + f_bytes(9, arr.tobytes())
    return msg


def attr_int(name: str, v: int) -> bytes:
    return f_str(1, name) + f_varint(3, v) + f_varint(20, 2)


def attr_float(name: str, v: float) -> bytes:
    return f_str(1, name) + f_float(2, v) + f_varint(20, 1)


def attr_ints(name: str, vs: Sequence[int]) -> bytes:
    return f_str(1, name) + b"".join(f_varint(8, int(v)) for v in vs) + f_varint(20, 7)


def node_proto(op_type: str, inputs: Sequence[str], outputs: Sequence[str], name: str,
               attrs: Sequence[bytes] = ()) -> bytes:
    msg = b"".join(f_str(1, i) for i in inputs) + b"".join(f_str(2, o) for o in outputs)
    msg += f_str(3, name) + f_str(4, op_type) + b"".join(f_bytes(5, a) for a in attrs)
    return msg


def value_info(name: str, shape: Sequence[int], elem_type: int = FLOAT) -> bytes:
    dims = b"".join(f_bytes(1, f_varint(1, int(d))) for d in shape)        # TensorShapeProto.dim
    ttype = f_varint(1, elem_type) + f_bytes(2, dims)                      # TypeProto.Tensor
    return f_str(1, name) + f_bytes(2, f_bytes(1, ttype))                  # ValueInfoProto


def model_proto(graph: bytes, opset: int = 17, producer_version: str = "0.1.0") -> bytes:
    opset_id = f_str(1, "") + f_varint(2, opset)
    return (f_varint(1, 9) + f_str(2, "rumus") + f_str(3, producer_version) + f_bytes(7, graph)
            + f_bytes(8, opset_id))


# ----------------------------------------------------------------------------- tracer
class _Tracer:
    def __init__(self):
        self.nodes: List[bytes] = []
        self.inits: List[bytes] = []
        self.names: Dict[int, str] = {}
        self.shapes: Dict[str, Tuple[int, ...]] = {}
        self.n = 0

    def name_of(self, t: torch.Tensor) -> str:
        k = id(t)
        if k not in self.names:
            raise KeyError("tensor reached a traced op without a producer; wrap the computation in "
                           "modules or the traced functional ops")
        return self.names[k]

    def new_value(self, t: torch.Tensor, hint: str) -> str:
        self.n += 1
        nm = f"{hint}_{self.n}"
        self.names[id(t)] = nm
        self.shapes[nm] = tuple(t.shape)
        self._keep.append(t)
        return nm

    _keep: List[torch.Tensor] = []

    def add_init(self, name: str, t: torch.Tensor):
        self.inits.append(tensor_proto(name, t))

    def add_node(self, op, ins, out_t, name, attrs=()):
        out = self.new_value(out_t, op.lower())
        self.nodes.append(node_proto(op, ins, [out], name, attrs))
        return out


def _module_node(tr: _Tracer, name: str, m: nn.Module, x: torch.Tensor, y: torch.Tensor):
    xin = tr.name_of(x)
    if isinstance(m, rnn.Linear):
        ins = [xin, name + ".weight"]
        tr.add_init(name + ".weight", m.weight)
        if m.bias is not None:
            ins.append(name + ".bias")
            tr.add_init(name + ".bias", m.bias)
        if x.dim() == 2:
            out = tr.add_node("Gemm", ins, y, name, [attr_float("alpha", 1.0), attr_float("beta", 1.0),
                                                    attr_int("transB", 0)])
        else:
            mm = torch.empty(0)
            out = tr.add_node("MatMul", ins[:2], y if m.bias is None else mm, name + "_matmul")
            if m.bias is not None:
                tr.shapes[out] = tuple(y.shape)
                out = tr.add_node("Add", [out, ins[2]], y, name + "_bias")
        if m.act:
            act = {"relu": "Relu", "gelu": "Gelu", "silu": "Swish"}[m.act]
            out = tr.add_node(act, [out], y, name + "_act")
        return
    if isinstance(m, rnn.Conv2d):
        k = m.kernel_size
        tr.add_init(name + ".weight", m.weight.view(m.out_channels, m.in_channels, k, k))
        ins = [xin, name + ".weight"]
        if m.bias is not None:
            ins.append(name + ".bias")
            tr.add_init(name + ".bias", m.bias)
        tr.add_node("Conv", ins, y, name, [attr_ints("kernel_shape", [k, k]), attr_ints("strides", [m.stride] * 2),
                                           attr_ints("pads", [m.padding] * 4),
                                           attr_ints("dilations", [m.dilation] * 2)])
        return
    if isinstance(m, rnn.BatchNorm2d):
        for suffix, t in (("weight", m.weight), ("bias", m.bias), ("running_mean", m.running_mean),
                          ("running_var", m.running_var)):
            tr.add_init(f"{name}.{suffix}", t)
        tr.add_node("BatchNormalization", [xin] + [f"{name}.{s}" for s in
                                                   ("weight", "bias", "running_mean", "running_var")],
                    y, name, [attr_float("epsilon", m.eps), attr_float("momentum", 1.0 - m.momentum)])
        return
    if isinstance(m, rnn.LayerNorm):
        tr.add_init(name + ".weight", m.weight)
        tr.add_init(name + ".bias", m.bias)
        tr.add_node("LayerNormalization", [xin, name + ".weight", name + ".bias"], y, name,
                    [attr_int("axis", -1), attr_float("epsilon", m.eps)])
        return
    if isinstance(m, rnn.MaxPool2d):
        tr.add_node("MaxPool", [xin], y, name, [attr_ints("kernel_shape", [m.kernel_size] * 2),
                                                attr_ints("strides", [m.stride] * 2),
                                                attr_ints("pads", [m.padding] * 4)])
        return
    if isinstance(m, rnn.AdaptiveAvgPool2d) and tuple(m.output_size) == (1, 1):
        tr.add_node("GlobalAveragePool", [xin], y, name)
        return
    if isinstance(m, rnn.Flatten):
        tr.add_node("Flatten", [xin], y, name, [attr_int("axis", 1)])
        return
    if isinstance(m, (nn.ReLU,)):
        tr.add_node("Relu", [xin], y, name)
        return
    if isinstance(m, (rnn.Dropout, nn.Identity)):
        tr.add_node("Identity", [xin], y, name)
        return
    if isinstance(m, rnn.Embedding):
        tr.add_init(name + ".weight", m.weight)
        tr.add_node("Gather", [name + ".weight", xin], y, name, [attr_int("axis", 0)])
        return
    raise NotImplementedError(f"ONNX export: no mapping for module {type(m).__name__} ({name})")


_LEAVES = (rnn.Linear, rnn.Conv2d, rnn.BatchNorm2d, rnn.LayerNorm, rnn.MaxPool2d, rnn.AdaptiveAvgPool2d,
           rnn.Flatten, rnn.Dropout, rnn.Embedding, nn.ReLU, nn.Identity)


def export_onnx(model: nn.Module, example_inputs: Sequence[torch.Tensor], path: Optional[str] = None,
                forward_fn: Optional[Callable] = None, opset: int = 17,
                input_names: Optional[Sequence[str]] = None) -> bytes:
    """Trace ``forward_fn(model, *example_inputs)`` (default ``model(*inputs)``) and serialise the
    graph.  Returns the ModelProto bytes and writes them to ``path`` if given
    (reference: ``export_onnx`` / ``export_onnx_with_opset``, onnx/export.rs:282-334)."""
    tr = _Tracer()
    tr._keep = []
    graph_inputs = []
    for i, t in enumerate(example_inputs):
        nm = (input_names[i] if input_names else f"input_{i}")
        tr.names[id(t)] = nm
        tr.shapes[nm] = tuple(t.shape)
        graph_inputs.append(value_info(nm, t.shape, INT64 if t.dtype == torch.int64 else FLOAT))
    hooks = []
    for name, m in model.named_modules():
        if isinstance(m, _LEAVES):
            hooks.append(m.register_forward_hook(
                lambda mod, args, out, _n=name: _module_node(tr, _n or type(mod).__name__, mod, args[0], out)))
    # primitive hooks between modules (the reference hooks exactly these four ops)
    saved = {}

    def wrap(fn_name, onnx_op, binary):
        orig = getattr(F, fn_name)
        saved[fn_name] = orig

        def traced(*a):
            out = orig(*a)
            ins = [tr.name_of(a[0])] + ([tr.name_of(a[1])] if binary else [])
            tr.add_node(onnx_op, ins, out, f"{fn_name}_{tr.n}")
            return out

        setattr(F, fn_name, traced)

    wrap("relu", "Relu", False)
    wrap("matmul", "MatMul", True)
    was_training = model.training
    model.eval()
    try:
        with torch.no_grad():
            out = forward_fn(model, *example_inputs) if forward_fn else model(*example_inputs)
    finally:
        for h in hooks:
            h.remove()
        for k, v in saved.items():
            setattr(F, k, v)
        model.train(was_training)
    outs = out if isinstance(out, (tuple, list)) else [out]
    graph_outputs = [value_info(tr.name_of(o), o.shape) for o in outs]
    graph = (b"".join(f_bytes(1, n) for n in tr.nodes) + f_str(2, "rumus_graph")
             + b"".join(f_bytes(5, i) for i in tr.inits) + b"".join(f_bytes(11, i) for i in graph_inputs)
             + b"".join(f_bytes(12, o) for o in graph_outputs))
    data = model_proto(graph, opset)
    if path:
        with open(path, "wb") as f:
            f.write(data)
    return data


# ----------------------------------------------------------------------------- minimal reader
def _read_varint(b: bytes, p: int) -> Tuple[int, int]:
    v = s = 0
    while True:
        c = b[p]
        p += 1
        v |= (c & 0x7F) << s
        s += 7
        if not c & 0x80:
            return v, p


def _fields(b: bytes):
    p = 0
    while p < len(b):
        k, p = _read_varint(b, p)
        field, wire = k >> 3, k & 7
        if wire == 0:
            v, p = _read_varint(b, p)
        elif wire == 2:
            n, p = _read_varint(b, p)
            v = b[p:p + n]
            p += n
        elif wire == 5:
            v = struct.unpack("<f", b[p:p + 4])[0]
            p += 4
        elif wire == 1:
            v = b[p:p + 8]
            p += 8
        else:
            raise ValueError(f"unsupported wire type {wire}")
        yield field, v


def parse_model(data: bytes) -> dict:
    """Decode the subset this exporter writes: ir_version, producer, opset, nodes, initializers."""
    m = {"nodes": [], "initializers": {}, "inputs": [], "outputs": []}
    for f, v in _fields(data):
        if f == 1:
            m["ir_version"] = v
        elif f == 2:
            m["producer_name"] = v.decode()
        elif f == 8:
            m["opset"] = dict(_fields(v)).get(2)
        elif f == 7:
            for gf, gv in _fields(v):
                if gf == 1:
                    node = {"inputs": [], "outputs": [], "attrs": []}
                    for nf, nv in _fields(gv):
                        if nf == 1:
                            node["inputs"].append(nv.decode())
                        elif nf == 2:
                            node["outputs"].append(nv.decode())
                        elif nf == 3:
                            node["name"] = nv.decode()
                        elif nf == 4:
                            node["op_type"] = nv.decode()
                        elif nf == 5:
                            node["attrs"].append(dict(_fields(nv)).get(1, b"").decode())
                    m["nodes"].append(node)
                elif gf == 5:
                    dims, name, raw, dt = [], "", b"", FLOAT
                    for tf, tv in _fields(gv):
                        if tf == 1:
                            dims.append(tv)
                        elif tf == 2:
                            dt = tv
                        elif tf == 8:
                            name = tv.decode()
                        elif tf == 9:
                            raw = tv
                    npdt = {FLOAT: "<f4", FLOAT16: "<f2", INT64: "<i8"}[dt]
                    m["initializers"][name] = np.frombuffer(raw, dtype=npdt).reshape(dims)
                elif gf in (11, 12):
                    nm = dict(_fields(gv)).get(1, b"").decode()
                    m["inputs" if gf == 11 else "outputs"].append(nm)
    return m
