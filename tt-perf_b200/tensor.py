"""Device tensors for the Python host side: a shape + dtype + device pointer owned through the C ABI
(the pooled allocator b200_pool_alloc / b200_pool_free, so that allocation is cheap and legal while a trace is
being recorded), with host <-> device copies through b200_memcpy_*. No torch, no CPU math:
numpy is used only to hold host bytes and to convert fp32 <-> bf16 bit patterns at the boundary, the way
`Tensor::from_vector` / `.cpu().to_vector<bfloat16>()` do in the reference (autograd/common.hpp:53,
traced/nn.hpp:40-52)."""
from __future__ import annotations

import ctypes as C
import math

import numpy as np

from . import capi
from .capi import BF16, F32, FP8_E4M3, U32

_ITEMSIZE = {BF16: 2, F32: 4, U32: 4, FP8_E4M3: 1}


def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even fp32 -> bf16 bit patterns (uint16)."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    return (((u + 0x7FFF + ((u >> 16) & 1)) >> 16) & 0xFFFF).astype(np.uint16)


def bf16_bits_to_f32(b: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(b, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


class DeviceTensor:
    """Contiguous row-major device buffer. Freed when the object dies (or on `free()`)."""

    def __init__(self, ctx: capi.Context, shape, dtype: int = BF16, ptr: int | None = None, owner=None):
        self.ctx = ctx
        self.shape = tuple(int(d) for d in shape)
        self.dtype = dtype
        self.numel = int(math.prod(self.shape)) if self.shape else 1
        self.nbytes = self.numel * _ITEMSIZE[dtype]
        self._owner = owner          # keeps the storage of a view alive
        self._owns = ptr is None
        self.ptr = ctx.pool_alloc(max(self.nbytes, 16)) if ptr is None else ptr

    # -- construction -------------------------------------------------------------------------------------------
    @classmethod
    def from_numpy(cls, ctx, array: np.ndarray, dtype: int = BF16, stream=None) -> "DeviceTensor":
        t = cls(ctx, array.shape, dtype)
        t.copy_from_numpy(array, stream)
        return t

    @classmethod
    def zeros(cls, ctx, shape, dtype: int = BF16, stream=None) -> "DeviceTensor":
        t = cls(ctx, shape, dtype)
        ctx.memset(t.ptr, 0, t.nbytes, stream)
        return t

    @classmethod
    def full(cls, ctx, shape, value: float, dtype: int = BF16, stream=None) -> "DeviceTensor":
        t = cls(ctx, shape, dtype)
        ctx.fill(t.ptr, t.numel, dtype, value, stream=stream)
        return t

    # -- host transfer ------------------------------------------------------------------------------------------
    def copy_from_numpy(self, array: np.ndarray, stream=None) -> None:
        if self.dtype == BF16:
            host = f32_to_bf16_bits(np.asarray(array, dtype=np.float32))
        elif self.dtype == F32:
            host = np.ascontiguousarray(array, dtype=np.float32)
        elif self.dtype == FP8_E4M3:
            host = np.ascontiguousarray(array, dtype=np.uint8)  # e4m3 codes, one byte each
        else:
            host = np.ascontiguousarray(array, dtype=np.uint32)
        if host.size != self.numel:
            raise ValueError(f"size mismatch: tensor {self.shape}, array {array.shape}")
        self.ctx.h2d(self.ptr, host.ctypes.data, self.nbytes, stream)
        self.ctx.synchronize(stream)  # `host` may be a temporary

    def numpy(self, stream=None) -> np.ndarray:
        """Device -> host; bf16 is widened to fp32, e4m3 comes back as its one-byte codes."""
        if self.dtype == BF16:
            host = np.empty(self.numel, dtype=np.uint16)
        elif self.dtype == F32:
            host = np.empty(self.numel, dtype=np.float32)
        elif self.dtype == FP8_E4M3:
            host = np.empty(self.numel, dtype=np.uint8)
        else:
            host = np.empty(self.numel, dtype=np.uint32)
        if self.numel:
            self.ctx.d2h(host.ctypes.data, self.ptr, self.nbytes, stream)
        out = bf16_bits_to_f32(host) if self.dtype == BF16 else host
        return out.reshape(self.shape)

    # -- views --------------------------------------------------------------------------------------------------
    def reshape(self, *shape) -> "DeviceTensor":
        shape = shape[0] if len(shape) == 1 and isinstance(shape[0], (tuple, list)) else shape
        if int(math.prod(shape)) != self.numel:
            raise ValueError(f"cannot reshape {self.shape} to {tuple(shape)}")
        return DeviceTensor(self.ctx, shape, self.dtype, ptr=self.ptr, owner=self)

    def narrow0(self, start: int, length: int) -> "DeviceTensor":
        """View of rows [start, start + length) of the first dimension (shares storage)."""
        if not (0 <= start and start + length <= self.shape[0]):
            raise ValueError(f"rows [{start}, {start + length}) outside {self.shape}")
        row_bytes = self.nbytes // self.shape[0] if self.shape[0] else 0
        return DeviceTensor(self.ctx, (length,) + self.shape[1:], self.dtype, ptr=self.ptr + start * row_bytes, owner=self)

    def data_ptr(self) -> int:
        return self.ptr

    def free(self) -> None:
        if self._owns and self.ptr and getattr(self.ctx, "_h", None):
            self.ctx.pool_free(self.ptr)
        self.ptr = 0
        self._owns = False

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass

    def __repr__(self):
        return f"DeviceTensor(shape={self.shape}, dtype={('bf16', 'f32', 'u32', 'e4m3')[self.dtype]}, ptr=0x{self.ptr:x})"
