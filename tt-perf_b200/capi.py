"""ctypes declarations for every entry point of include/b200_ttperf.h, plus a thin `Context` wrapper.

Device buffers are passed as integer addresses (anything with a `data_ptr()` method, such as a
torch CUDA tensor, is also accepted); nothing here allocates through torch or copies through numpy.
"""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

BF16, F32, U32 = 0, 1, 2
ACT_NONE, ACT_RELU, ACT_GELU = 0, 1, 2
LOFI, HIFI2, HIFI3, HIFI4 = 0, 1, 2, 3
ALGO_AUTO, ALGO_TCGEN05, ALGO_SIMT = 0, 1, 2

OK, ERR_INVALID_ARG, ERR_CUDA, ERR_UNSUPPORTED, ERR_DEVICE_TIMEOUT, ERR_NOMEM, ERR_COMM = range(7)

_STATUS_NAMES = {
    0: "B200_OK", 1: "B200_ERR_INVALID_ARG", 2: "B200_ERR_CUDA", 3: "B200_ERR_UNSUPPORTED",
    4: "B200_ERR_DEVICE_TIMEOUT", 5: "B200_ERR_NOMEM", 6: "B200_ERR_COMM",
}


class B200Error(RuntimeError):
    def __init__(self, code: int, text: str):
        super().__init__(f"{_STATUS_NAMES.get(code, code)}: {text}")
        self.code = code
        self.text = text


class GemmDesc(C.Structure):
    """Mirror of `b200_gemm_desc`."""
    _fields_ = [
        ("transpose_a", C.c_int32), ("transpose_b", C.c_int32),
        ("M", C.c_int64), ("N", C.c_int64), ("K", C.c_int64), ("batch", C.c_int64),
        ("A", C.c_void_p), ("lda", C.c_int64), ("stride_a", C.c_int64),
        ("B", C.c_void_p), ("ldb", C.c_int64), ("stride_b", C.c_int64),
        ("C", C.c_void_p), ("ldc", C.c_int64), ("stride_c", C.c_int64),
        ("c_dtype", C.c_int32),
        ("bias", C.c_void_p), ("bias_dtype", C.c_int32),
        ("activation", C.c_int32), ("alpha", C.c_float),
        ("causal_mask", C.c_int32), ("mask_value", C.c_float),
        ("fidelity", C.c_int32), ("algo", C.c_int32), ("split_k", C.c_int32),
    ]


def lib_path() -> Path:
    return Path(__file__).resolve().parent / "lib" / "libb200ttperf.so"


# name -> (restype, argtypes); kept in one table so tests can check it against the header.
SIGNATURES = {
    "b200_ctx_create": (C.c_int, [C.c_int, C.POINTER(C.c_void_p)]),
    "b200_ctx_destroy": (C.c_int, [C.c_void_p]),
    "b200_ctx_device": (C.c_int, [C.c_void_p, C.POINTER(C.c_int)]),
    "b200_ctx_sm_count": (C.c_int, [C.c_void_p, C.POINTER(C.c_int)]),
    "b200_synchronize": (C.c_int, [C.c_void_p, C.c_void_p]),
    "b200_last_error": (C.c_char_p, []),
    "b200_abi_version": (C.c_int, []),
    "b200_malloc": (C.c_int, [C.c_void_p, C.c_size_t, C.POINTER(C.c_void_p)]),
    "b200_free": (C.c_int, [C.c_void_p, C.c_void_p]),
    "b200_memcpy_h2d": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p]),
    "b200_memcpy_d2h": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p]),
    "b200_memset": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_size_t, C.c_void_p]),
    "b200_gemm_desc_init": (None, [C.POINTER(GemmDesc)]),
    "b200_gemm": (C.c_int, [C.c_void_p, C.POINTER(GemmDesc), C.c_void_p]),
    "b200_gemm_scratch_bytes": (C.c_int, [C.c_void_p, C.POINTER(GemmDesc), C.POINTER(C.c_size_t)]),
    "b200_gemm_static_scratch": (C.c_int, [C.c_int, C.POINTER(GemmDesc), C.c_void_p]),
}

_lib = None


def lib() -> C.CDLL:
    """Loads the CUDA library; raises if it has not been built (there is no other backend)."""
    global _lib
    if _lib is None:
        p = lib_path()
        if not p.exists():
            raise B200Error(ERR_UNSUPPORTED, f"{p} is missing: build it with `python tt-perf_b200/build.py` "
                                             "(this package has no CPU or PyTorch fallback)")
        handle = C.CDLL(os.fspath(p))
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype = res
            fn.argtypes = args
        _lib = handle
    return _lib


def ptr(x) -> int:
    """Device address of `x`: an int, None, or any object with data_ptr()."""
    if x is None:
        return 0
    if isinstance(x, int):
        return x
    if hasattr(x, "data_ptr"):
        return int(x.data_ptr())
    raise TypeError(f"cannot take a device address from {type(x)!r}")


def check(code: int) -> None:
    if code != OK:
        raise B200Error(code, lib().b200_last_error().decode("utf-8", "replace"))


class Context:
    """One per (process, GPU). `stream` arguments are raw cudaStream_t values (0/None = the context's stream)."""

    def __init__(self, device: int = 0):
        self._h = C.c_void_p()
        check(lib().b200_ctx_create(int(device), C.byref(self._h)))
        self.device = int(device)

    def close(self) -> None:
        if getattr(self, "_h", None) is not None and self._h:
            lib().b200_ctx_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    @property
    def handle(self) -> C.c_void_p:
        return self._h

    @property
    def sm_count(self) -> int:
        n = C.c_int()
        check(lib().b200_ctx_sm_count(self._h, C.byref(n)))
        return n.value

    def synchronize(self, stream=None) -> None:
        check(lib().b200_synchronize(self._h, C.c_void_p(ptr(stream))))

    # ---- memory -------------------------------------------------------------------------------------
    def malloc(self, nbytes: int) -> int:
        out = C.c_void_p()
        check(lib().b200_malloc(self._h, nbytes, C.byref(out)))
        return out.value or 0

    def free(self, dptr: int) -> None:
        check(lib().b200_free(self._h, C.c_void_p(dptr)))

    def h2d(self, d_dst, h_src, nbytes: int, stream=None) -> None:
        check(lib().b200_memcpy_h2d(self._h, C.c_void_p(ptr(d_dst)), C.c_void_p(ptr(h_src)), nbytes,
                                    C.c_void_p(ptr(stream))))

    def d2h(self, h_dst, d_src, nbytes: int, stream=None) -> None:
        check(lib().b200_memcpy_d2h(self._h, C.c_void_p(ptr(h_dst)), C.c_void_p(ptr(d_src)), nbytes,
                                    C.c_void_p(ptr(stream))))

    def memset(self, d_dst, value: int, nbytes: int, stream=None) -> None:
        check(lib().b200_memset(self._h, C.c_void_p(ptr(d_dst)), value, nbytes, C.c_void_p(ptr(stream))))

    # ---- matmul -------------------------------------------------------------------------------------
    def gemm_desc(self, A, B, Cout, M, N, K, *, transpose_a=False, transpose_b=False, lda=None, ldb=None, ldc=None,
                  batch=1, stride_a=None, stride_b=None, stride_c=None, c_dtype=BF16, bias=None, bias_dtype=BF16,
                  activation=ACT_NONE, alpha=1.0, causal_mask=False, mask_value=-1e9, fidelity=HIFI4,
                  algo=ALGO_AUTO, split_k=0) -> GemmDesc:
        """Descriptor for C = act(mask(alpha * op(A) @ op(B) + bias)); dense row-major defaults for ld/strides."""
        d = GemmDesc()
        lib().b200_gemm_desc_init(C.byref(d))
        d.transpose_a, d.transpose_b = int(bool(transpose_a)), int(bool(transpose_b))
        d.M, d.N, d.K, d.batch = M, N, K, batch
        a_rows, a_cols = (K, M) if transpose_a else (M, K)
        b_rows, b_cols = (N, K) if transpose_b else (K, N)
        d.A, d.B, d.C = ptr(A) or None, ptr(B) or None, ptr(Cout) or None
        d.lda = a_cols if lda is None else lda
        d.ldb = b_cols if ldb is None else ldb
        d.ldc = N if ldc is None else ldc
        d.stride_a = a_rows * d.lda if stride_a is None else stride_a
        d.stride_b = b_rows * d.ldb if stride_b is None else stride_b
        d.stride_c = M * d.ldc if stride_c is None else stride_c
        d.c_dtype = c_dtype
        d.bias, d.bias_dtype = ptr(bias) or None, bias_dtype
        d.activation, d.alpha = activation, alpha
        d.causal_mask, d.mask_value = int(bool(causal_mask)), mask_value
        d.fidelity, d.algo, d.split_k = fidelity, algo, split_k
        return d

    def gemm(self, desc: GemmDesc, stream=None) -> None:
        check(lib().b200_gemm(self._h, C.byref(desc), C.c_void_p(ptr(stream))))

    def gemm_static_scratch(self, desc: GemmDesc, stream) -> None:
        """Split-K matmul whose partial sums use the library's fixed 32 MiB array: no device allocation at
        call time (see b200_gemm_static_scratch in the header). `stream` is required."""
        check(lib().b200_gemm_static_scratch(self.device, C.byref(desc), C.c_void_p(ptr(stream))))

    def gemm_scratch_bytes(self, desc: GemmDesc) -> int:
        n = C.c_size_t()
        check(lib().b200_gemm_scratch_bytes(self._h, C.byref(desc), C.byref(n)))
        return n.value
