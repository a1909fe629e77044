"""`import ttnn` for the Python side of the reference: the subset of the TTNN Python API that py/engine.py, py/nn.py,
py/optim.py, py/experiment.py and tests/*.py of csirak/tt-perf call, implemented over the B200 C ABI (libb200ttperf.so)
so that those files run unchanged:

    PYTHONPATH=<this repo>/tt-perf_b200/ttnn_py:<tt-perf>  python <tt-perf>/tests/tensor_add_mul_matmul_tanh.py

Every op allocates its result from the context's pool and launches one library kernel on the context stream
(ttnn.matmul -> b200_gemm, element-wise ops -> b200_binary / b200_unary with numpy-style broadcasting, ttnn.sum ->
b200_reduce, ttnn.softmax -> b200_softmax, ttnn.permute -> b200_permute, ttnn.embedding -> b200_embedding_forward).
torch is touched only by from_torch / to_torch, as a container of host data. Device tensors are bfloat16 (or uint32 for
indices); float32 device tensors are not offered (the reference's default is bfloat16, py/engine.py:6).

Call sites followed: py/engine.py:63-67 (from_torch / to_torch), :156-393 (add, mul, matmul, permute, sum, tanh, reshape,
softmax, log, exp, relu, gtz, sub, ones_like), py/nn.py:98-249 (embedding, full_like, triu), py/optim.py:19-86 (div,
sqrt), tests/*.py (open_device / close_device)."""
from __future__ import annotations

import builtins
import importlib.util
import math
import sys
from pathlib import Path

import numpy as np

_REPO = Path(__file__).resolve().parents[3]


def _package():
    if "ttperf_b200" in sys.modules:
        return sys.modules["ttperf_b200"]
    spec = importlib.util.spec_from_file_location("__graft_entry__", _REPO / "__graft_entry__.py")
    entry = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(entry)
    return entry.load_package()


# ---- enums and configuration objects ----------------------------------------------------------------------------------
class DataType:
    def __init__(self, name):
        self.name = name

    def __repr__(self):
        return f"DataType.{self.name}"


bfloat16, float32, uint32 = DataType("BFLOAT16"), DataType("FLOAT32"), DataType("UINT32")


class Layout:
    def __init__(self, name):
        self.name = name

    def __repr__(self):
        return f"Layout.{self.name}"


TILE_LAYOUT, ROW_MAJOR_LAYOUT = Layout("TILE"), Layout("ROW_MAJOR")


class MathFidelity:
    LoFi, HiFi2, HiFi3, HiFi4 = "LoFi", "HiFi2", "HiFi3", "HiFi4"


class WormholeComputeKernelConfig:
    """Accepted and carried around; math_fidelity selects the GEMM fidelity knob (LoFi / HiFi2 round K-slice sums to bf16)."""

    def __init__(self, math_fidelity=MathFidelity.HiFi4, math_approx_mode=False, fp32_dest_acc_en=True, packer_l1_acc=False,
                 **_):
        self.math_fidelity = math_fidelity
        self.math_approx_mode = math_approx_mode
        self.fp32_dest_acc_en = fp32_dest_acc_en
        self.packer_l1_acc = packer_l1_acc


DeviceComputeKernelConfig = WormholeComputeKernelConfig


# ---- device ----------------------------------------------------------------------------------------------------------
class Device:
    def __init__(self, device_id: int):
        self.pkg = _package()
        self.ctx = self.pkg.Context(device_id)
        self.device_id = device_id

    def id(self):
        return self.device_id

    def __repr__(self):
        return f"ttnn.Device(B200 #{self.device_id})"


def open_device(device_id: int = 0, **_) -> Device:
    return Device(device_id)


def close_device(device: Device) -> None:
    if device.ctx is not None:
        device.ctx.synchronize()
        device.ctx.close()
        device.ctx = None


def synchronize_device(device: Device) -> None:
    device.ctx.synchronize()


def ReadDeviceProfiler(device: Device) -> None:   # profiler hook of the vendor runtime: nothing to read here
    return None


# ---- tensor ----------------------------------------------------------------------------------------------------------
class Shape(tuple):
    """A tuple that also answers `.rank`."""

    @property
    def rank(self):
        return len(self)


class Tensor:
    def __init__(self, storage, shape, dtype, layout, device: Device):
        self._t = storage            # DeviceTensor, contiguous row-major
        self.shape = Shape(int(d) for d in shape)
        self.dtype = dtype
        self.layout = layout
        self._device = device

    def device(self):
        return self._device

    def get_layout(self):
        return self.layout

    def get_dtype(self):
        return self.dtype

    def volume(self):
        return int(math.prod(self.shape)) if self.shape else 1

    def __repr__(self):
        return f"ttnn.Tensor(shape={tuple(self.shape)}, dtype={self.dtype}, layout={self.layout})"


def _new(device: Device, shape, dtype=bfloat16, layout=TILE_LAYOUT) -> Tensor:
    pkg = device.pkg
    abi = pkg.BF16 if dtype is bfloat16 else pkg.U32
    return Tensor(pkg.DeviceTensor(device.ctx, tuple(shape) if len(shape) else (1,), abi), shape, dtype, layout, device)


def _check_bf16(*ts):
    for t in ts:
        if t.dtype is not bfloat16:
            raise TypeError(f"this op needs bfloat16 tensors, got {t.dtype}")


def from_torch(tensor, dtype=None, layout=None, device=None, **_) -> Tensor:
    """Host torch tensor -> device tensor (py/engine.py:63, py/nn.py:100-105)."""
    import torch
    if device is None:
        raise RuntimeError("ttnn.from_torch: the B200 stand-in keeps tensors on a device; pass device=")
    if dtype is None:
        dtype = uint32 if tensor.dtype in (torch.int32, torch.int64, torch.uint8) else bfloat16
    if dtype is float32:
        raise NotImplementedError("ttnn.from_torch: device tensors are bfloat16 (or uint32) on B200; pass dtype=ttnn.bfloat16")
    host = tensor.detach().cpu()
    out = _new(device, tuple(host.shape), dtype, layout or TILE_LAYOUT)
    if dtype is uint32:
        out._t.copy_from_numpy(host.to(torch.int64).numpy().astype(np.uint32))
    else:
        out._t.copy_from_numpy(host.to(torch.float32).numpy())
    return out


def to_torch(tensor: Tensor, **_):
    """Device tensor -> host torch tensor of the matching dtype (py/engine.py:67)."""
    import torch
    tensor._device.ctx.synchronize()
    host = tensor._t.numpy().reshape(tuple(tensor.shape))
    if tensor.dtype is uint32:
        return torch.from_numpy(host.astype(np.int64)).to(torch.int32)
    return torch.from_numpy(np.ascontiguousarray(host, dtype=np.float32)).to(torch.bfloat16)


def to_device(tensor: Tensor, device: Device, **_) -> Tensor:
    return tensor


def to_layout(tensor: Tensor, layout, **_) -> Tensor:
    return Tensor(tensor._t, tensor.shape, tensor.dtype, layout, tensor._device)


def deallocate(tensor: Tensor, **_) -> None:
    tensor._t.free()


# ---- element-wise ------------------------------------------------------------------------------------------------------
def _broadcast(a, b):
    r = builtins.max(len(a), len(b))   # this module defines ttnn.max / ttnn.sum, which shadow the built-ins here
    a4, b4 = (1,) * (r - len(a)) + tuple(a), (1,) * (r - len(b)) + tuple(b)
    out = []
    for x, y in zip(a4, b4):
        if x != y and x != 1 and y != 1:
            raise ValueError(f"shapes {tuple(a)} and {tuple(b)} do not broadcast")
        out.append(builtins.max(x, y))
    return tuple(out), a4, b4


def _fold4(out, a4, b4):
    """Ranks above 4 are folded from the left while both operands agree there (no broadcasting inside the fold)."""
    while len(out) > 4:
        if a4[0] == out[0] and b4[0] == out[0] and a4[1] == out[1] and b4[1] == out[1]:
            out = (out[0] * out[1],) + tuple(out[2:])
            a4 = (a4[0] * a4[1],) + tuple(a4[2:])
            b4 = (b4[0] * b4[1],) + tuple(b4[2:])
        else:
            raise ValueError("broadcasting over more than four dimensions is not supported")
    return out, a4, b4


def _binary(op_name, a, b):
    if isinstance(a, (int, float)):
        if op_name in ("ADD", "MUL"):
            a, b = b, a
        else:
            a = full_like(b, a)
    pkg = a._device.pkg
    c = pkg.capi
    if isinstance(b, (int, float)):
        _check_bf16(a)
        out = _new(a._device, a.shape, bfloat16, a.layout)
        if op_name == "ADD":
            a._device.ctx.unary(c.U_ADD_SCALAR, a._t, out._t, a.volume(), scalar=float(b))
        elif op_name == "SUB":
            a._device.ctx.unary(c.U_ADD_SCALAR, a._t, out._t, a.volume(), scalar=-float(b))
        elif op_name == "MUL":
            a._device.ctx.unary(c.U_MUL_SCALAR, a._t, out._t, a.volume(), scalar=float(b))
        else:
            a._device.ctx.unary(c.U_MUL_SCALAR, a._t, out._t, a.volume(), scalar=1.0 / float(b))
        return out
    _check_bf16(a, b)
    shape, a4, b4 = _broadcast(a.shape, b.shape)
    f_out, f_a, f_b = _fold4(shape, a4, b4)
    out = _new(a._device, shape, bfloat16, a.layout)
    a._device.ctx.binary(getattr(c, "B_" + op_name), a._t, f_a, b._t, f_b, out._t)
    return out


def add(a, b, **_):
    return _binary("ADD", a, b)


def sub(a, b, **_):
    return _binary("SUB", a, b)


def mul(a, b, **_):
    return _binary("MUL", a, b)


def div(a, b, **_):
    return _binary("DIV", a, b)


subtract, multiply, divide = sub, mul, div


def _unary(name, x):
    _check_bf16(x)
    c = x._device.pkg.capi
    out = _new(x._device, x.shape, bfloat16, x.layout)
    x._device.ctx.unary(getattr(c, "U_" + name), x._t, out._t, x.volume())
    return out


def relu(x, **_):
    return _unary("RELU", x)


def gtz(x, **_):
    return _unary("GTZ", x)


def gelu(x, **_):
    return _unary("GELU", x)


def tanh(x, **_):
    return _unary("TANH", x)


def exp(x, **_):
    return _unary("EXP", x)


def log(x, **_):
    return _unary("LOG", x)


def sqrt(x, **_):
    return _unary("SQRT", x)


def rsqrt(x, **_):
    return _unary("RSQRT", x)


def neg(x, **_):
    return _unary("NEG", x)


def full_like(x: Tensor, fill_value, **_) -> Tensor:
    out = _new(x._device, x.shape, x.dtype, x.layout)
    pkg = x._device.pkg
    x._device.ctx.fill(out._t, out.volume(), pkg.BF16 if x.dtype is bfloat16 else pkg.U32, float(fill_value))
    return out


def ones_like(x, **_):
    return full_like(x, 1.0)


def zeros_like(x, **_):
    return full_like(x, 0.0)


def full(shape, fill_value, dtype=bfloat16, layout=TILE_LAYOUT, device=None, **_):
    out = _new(device, tuple(shape), dtype, layout)
    pkg = device.pkg
    device.ctx.fill(out._t, out.volume(), pkg.BF16 if dtype is bfloat16 else pkg.U32, float(fill_value))
    return out


# ---- matmul ------------------------------------------------------------------------------------------------------------
_FIDELITY = {MathFidelity.LoFi: "LOFI", MathFidelity.HiFi2: "HIFI2", MathFidelity.HiFi3: "HIFI3", MathFidelity.HiFi4: "HIFI4"}


def matmul(a: Tensor, b: Tensor, transpose_a: bool = False, transpose_b: bool = False, compute_kernel_config=None, **_) -> Tensor:
    """Leading dimensions are batches; a rank-2 operand broadcasts over the other's batches (py/engine.py:237-244)."""
    _check_bf16(a, b)
    pkg, ctx = a._device.pkg, a._device.ctx
    if len(a.shape) < 2 or len(b.shape) < 2:
        raise ValueError("ttnn.matmul needs operands of rank >= 2")
    kw = {}
    if compute_kernel_config is not None:
        kw["fidelity"] = getattr(pkg.capi, _FIDELITY.get(compute_kernel_config.math_fidelity, "HIFI4"))
    am, ak = (a.shape[-1], a.shape[-2]) if transpose_a else (a.shape[-2], a.shape[-1])
    bk, bn = (b.shape[-1], b.shape[-2]) if transpose_b else (b.shape[-2], b.shape[-1])
    if ak != bk:
        raise ValueError(f"ttnn.matmul: inner dimensions differ ({tuple(a.shape)} x {tuple(b.shape)})")
    lead_a, lead_b = tuple(a.shape[:-2]), tuple(b.shape[:-2])
    na, nb = int(math.prod(lead_a)) if lead_a else 1, int(math.prod(lead_b)) if lead_b else 1
    if nb == 1 and not transpose_a:
        # [.., M, K] x [K, N]: one GEMM with the batches folded into M
        out = _new(a._device, lead_a + (am, bn), bfloat16, a.layout)
        d = ctx.gemm_desc(a._t, b._t, out._t, na * am, bn, ak, transpose_b=transpose_b, **kw)
    else:
        if na != 1 and nb != 1 and lead_a != lead_b:
            if int(math.prod(lead_a)) != int(math.prod(lead_b)):
                raise ValueError(f"ttnn.matmul: batch dimensions differ ({tuple(a.shape)} x {tuple(b.shape)})")
        lead = lead_a if na >= nb else lead_b
        batch = builtins.max(na, nb)
        out = _new(a._device, lead + (am, bn), bfloat16, a.layout)
        d = ctx.gemm_desc(a._t, b._t, out._t, am, bn, ak, transpose_a=transpose_a, transpose_b=transpose_b, batch=batch,
                          stride_a=0 if na == 1 and batch > 1 else None, stride_b=0 if nb == 1 and batch > 1 else None, **kw)
    ctx.gemm(d)
    return out


def linear(a, w, bias=None, transpose_a=False, transpose_b=False, **kw):
    out = matmul(a, w, transpose_a, transpose_b, **kw)
    return add(out, bias) if bias is not None else out


# ---- reductions, softmax ----------------------------------------------------------------------------------------------
def _reduce(op_name, x, dim, keepdim):
    _check_bf16(x)
    c = x._device.pkg.capi
    shape = tuple(x.shape)
    if dim is None:
        out = _new(x._device, (1,) * len(shape) if keepdim else (), bfloat16, x.layout)
        x._device.ctx.reduce(getattr(c, "R_" + op_name), x._t, 1, x.volume(), 1, out._t)
        return out
    dim = dim + len(shape) if dim < 0 else dim
    outer = int(math.prod(shape[:dim])) if dim else 1
    inner = int(math.prod(shape[dim + 1:])) if dim + 1 < len(shape) else 1
    out_shape = shape[:dim] + ((1,) if keepdim else ()) + shape[dim + 1:]
    out = _new(x._device, out_shape, bfloat16, x.layout)
    x._device.ctx.reduce(getattr(c, "R_" + op_name), x._t, outer, shape[dim], inner, out._t)
    return out


def sum(x, dim=None, keepdim=False, **_):   # noqa: A001 - the TTNN name
    return _reduce("SUM", x, dim, keepdim)


def mean(x, dim=None, keepdim=False, **_):
    return _reduce("MEAN", x, dim, keepdim)


def max(x, dim=None, keepdim=False, **_):   # noqa: A001
    return _reduce("MAX", x, dim, keepdim)


def softmax(x, dim=-1, **_):
    _check_bf16(x)
    shape = tuple(x.shape)
    dim = dim + len(shape) if dim < 0 else dim
    if dim != len(shape) - 1:
        order = list(range(len(shape)))
        order[dim], order[-1] = order[-1], order[dim]
        return permute(softmax(permute(x, order), -1), order)
    cols = shape[-1]
    out = _new(x._device, shape, bfloat16, x.layout)
    x._device.ctx.softmax(x._t, out._t, x.volume() // cols, cols)
    return out


# ---- layout ------------------------------------------------------------------------------------------------------------
def reshape(x: Tensor, shape, **_) -> Tensor:
    shape = tuple(int(d) for d in (shape if not isinstance(shape, int) else (shape,)))
    if -1 in shape:
        known = -int(math.prod(shape))
        shape = tuple(x.volume() // known if d == -1 else d for d in shape)
    if int(math.prod(shape)) != x.volume():
        raise ValueError(f"ttnn.reshape: cannot view {tuple(x.shape)} as {shape}")
    return Tensor(x._t, shape, x.dtype, x.layout, x._device)


def permute(x: Tensor, dims, **_) -> Tensor:
    _check_bf16(x)
    dims = [d + len(x.shape) if d < 0 else d for d in dims]
    r = len(x.shape)
    if sorted(dims) != list(range(r)):
        raise ValueError(f"ttnn.permute: {dims} is not a permutation of {r} dimensions")
    if r > 4:
        raise ValueError("ttnn.permute supports up to four dimensions")
    pad = 4 - r
    in4 = (1,) * pad + tuple(x.shape)
    perm4 = list(range(pad)) + [d + pad for d in dims]
    out = _new(x._device, tuple(x.shape[d] for d in dims), bfloat16, x.layout)
    x._device.ctx.permute(x._t, in4, perm4, out._t)
    return out


def transpose(x: Tensor, dim0: int, dim1: int, **_) -> Tensor:
    order = list(range(len(x.shape)))
    order[dim0], order[dim1] = order[dim1], order[dim0]
    return permute(x, order)


def triu(x: Tensor, diagonal: int = 0, **_) -> Tensor:
    _check_bf16(x)
    rows, cols = x.shape[-2], x.shape[-1]
    out = _new(x._device, x.shape, bfloat16, x.layout)
    x._device.ctx.triu(x._t, out._t, x.volume() // (rows * cols), rows, cols, diagonal)
    return out


def embedding(indices: Tensor, weight: Tensor, layout=None, **_) -> Tensor:
    """Row gather (py/nn.py:106-111): indices uint32 of any shape, weight [vocab, dim] -> indices.shape + (dim,)."""
    if indices.dtype is not uint32:
        raise TypeError("ttnn.embedding: indices must be uint32")
    _check_bf16(weight)
    vocab, dim = weight.shape
    out = _new(weight._device, tuple(indices.shape) + (dim,), bfloat16, layout or TILE_LAYOUT)
    weight._device.ctx.embedding_forward(indices._t, indices.volume(), weight._t, vocab, dim, out._t)
    return out
