"""ctypes declarations for every entry point of include/b200_ttperf.h, plus a thin `Context` wrapper.

Device buffers are passed as integer addresses (anything with a `data_ptr()` method, such as a
torch CUDA tensor, is also accepted); nothing here allocates through torch or copies through numpy.
"""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

BF16, F32, U32, FP8_E4M3 = 0, 1, 2, 3
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
        ("fidelity", C.c_int32), ("algo", C.c_int32), ("split_k", C.c_int32), ("ab_dtype", C.c_int32),
    ]


ATTN_DETERMINISTIC = 1
KERNEL_SIMT, KERNEL_TCGEN05, KERNEL_TCGEN05_PAIR = 0, 1, 2


class GemmPlan(C.Structure):
    """Mirror of `b200_gemm_plan`: kernel, tile width, K slices and tile order of one product."""
    _fields_ = [("kernel", C.c_int32), ("block_n", C.c_int32), ("k_slices", C.c_int32), ("group_m", C.c_int32)]


class AttnOperand(C.Structure):
    """Mirror of b200_attn_operand: element (b, h, s, d) at ptr[b*stride_b + h*stride_h + s*stride_s + d]."""
    _fields_ = [("ptr", C.c_void_p), ("stride_b", C.c_int64), ("stride_h", C.c_int64), ("stride_s", C.c_int64)]


def lib_path() -> Path:
    """The library this process binds."""
    return Path(__file__).resolve().parent / "lib" / "libb200ttperf.so"


# name -> (restype, argtypes); kept in one table so tests can check it against the header.
SIGNATURES = {
    "b200_ctx_create": (C.c_int, [C.c_int, C.POINTER(C.c_void_p)]),
    "b200_ctx_destroy": (C.c_int, [C.c_void_p]),
    "b200_ctx_device": (C.c_int, [C.c_void_p, C.POINTER(C.c_int)]),
    "b200_ctx_stream": (C.c_int, [C.c_void_p, C.POINTER(C.c_void_p)]),
    "b200_ctx_sm_count": (C.c_int, [C.c_void_p, C.POINTER(C.c_int)]),
    "b200_synchronize": (C.c_int, [C.c_void_p, C.c_void_p]),
    "b200_timer_start": (C.c_int, [C.c_void_p, C.c_void_p, C.POINTER(C.c_void_p)]),
    "b200_timer_stop": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.POINTER(C.c_float)]),
    "b200_last_error": (C.c_char_p, []),
    "b200_abi_version": (C.c_int, []),
    "b200_malloc": (C.c_int, [C.c_void_p, C.c_size_t, C.POINTER(C.c_void_p)]),
    "b200_free": (C.c_int, [C.c_void_p, C.c_void_p]),
    "b200_memcpy_h2d": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p]),
    "b200_memcpy_d2h": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p]),
    "b200_memcpy_d2d": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p]),
    "b200_memset": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_size_t, C.c_void_p]),
    "b200_pool_alloc": (C.c_int, [C.c_void_p, C.c_size_t, C.POINTER(C.c_void_p)]),
    "b200_pool_free": (C.c_int, [C.c_void_p, C.c_void_p]),
    "b200_pool_stats": (C.c_int, [C.c_void_p, C.POINTER(C.c_size_t), C.POINTER(C.c_size_t)]),
    "b200_trace_begin": (C.c_int, [C.c_void_p, C.POINTER(C.c_uint32)]),
    "b200_trace_end": (C.c_int, [C.c_void_p, C.c_uint32]),
    "b200_trace_execute": (C.c_int, [C.c_void_p, C.c_uint32, C.c_int]),
    "b200_trace_execute_on": (C.c_int, [C.c_void_p, C.c_uint32, C.c_void_p]),
    "b200_trace_release": (C.c_int, [C.c_void_p, C.c_uint32]),
    "b200_gemm_desc_init": (None, [C.POINTER(GemmDesc)]),
    "b200_gemm": (C.c_int, [C.c_void_p, C.POINTER(GemmDesc), C.c_void_p]),
    "b200_matmul_host": (C.c_int, [C.c_void_p, C.POINTER(GemmDesc), C.c_int]),
    "b200_gemm_scratch_bytes": (C.c_int, [C.c_void_p, C.POINTER(GemmDesc), C.POINTER(C.c_size_t)]),
    "b200_gemm_static_scratch": (C.c_int, [C.c_int, C.POINTER(GemmDesc), C.c_void_p]),
    "b200_static_scratch_status": (C.c_int, [C.c_int, C.c_void_p, C.POINTER(C.c_int)]),
    "b200_gemm_plan_query": (C.c_int, [C.c_void_p, C.POINTER(GemmDesc), C.POINTER(GemmPlan)]),
    "b200_gemm_plan_describe": (C.c_int, [C.POINTER(GemmDesc), C.POINTER(GemmPlan), C.c_char_p, C.c_size_t]),
    "b200_gemm_planned": (C.c_int, [C.c_void_p, C.POINTER(GemmDesc), C.POINTER(GemmPlan), C.c_void_p]),
    "b200_selftest_wait_timeout": (C.c_int, [C.c_void_p, C.c_uint64, C.c_void_p]),
    "b200_ipc_get_handle": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p]),
    "b200_ipc_open_handle": (C.c_int, [C.c_void_p, C.c_void_p, C.POINTER(C.c_void_p)]),
    "b200_ipc_close_handle": (C.c_int, [C.c_void_p, C.c_void_p]),
    "b200_enable_peer_access": (C.c_int, [C.c_void_p, C.c_void_p]),
    "b200_peer_copy_2d": (C.c_int, [C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p, C.c_void_p, C.c_size_t, C.c_size_t,
                                    C.c_size_t]),
    "b200_ctx_wait_ctx": (C.c_int, [C.c_void_p, C.c_void_p]),
    "b200_peer_barrier": (C.c_int, [C.c_void_p, C.POINTER(C.c_void_p), C.c_int, C.c_int, C.c_void_p, C.c_void_p]),
    "b200_mc_supported": (C.c_int, [C.c_void_p, C.POINTER(C.c_int)]),
    "b200_mc_alloc": (C.c_int, [C.c_void_p, C.c_size_t, C.POINTER(C.c_void_p), C.POINTER(C.c_void_p), C.POINTER(C.c_void_p)]),
    "b200_mc_free": (C.c_int, [C.c_void_p]),
    "b200_mc_broadcast": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p]),
    "b200_gemm_allgather_mc": (C.c_int, [C.c_void_p, C.POINTER(GemmDesc), C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p]),
    "b200_gemm_allgather": (C.c_int, [C.c_void_p, C.POINTER(GemmDesc), C.POINTER(C.c_void_p), C.c_int, C.c_int, C.c_void_p]),
    "b200_gemm_reduce_scatter_partials": (C.c_int, [C.c_void_p, C.POINTER(GemmDesc), C.POINTER(C.c_void_p), C.c_int, C.c_int,
                                                    C.c_void_p]),
    "b200_gemm_dist_plan_query": (C.c_int, [C.c_void_p, C.POINTER(GemmDesc), C.c_int, C.c_int, C.POINTER(GemmPlan)]),
    "b200_reduce_slices": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.POINTER(GemmDesc), C.c_void_p]),
    "b200_reduce_slices_typed": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.POINTER(GemmDesc), C.c_void_p]),
    "b200_comm_unique_id": (C.c_int, [C.c_void_p]),
    "b200_comm_create": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.POINTER(C.c_void_p)]),
    "b200_comm_destroy": (C.c_int, [C.c_void_p]),
    "b200_comm_size": (C.c_int, [C.c_void_p, C.POINTER(C.c_int), C.POINTER(C.c_int)]),
    "b200_comm_barrier": (C.c_int, [C.c_void_p, C.c_void_p]),
    "b200_comm_exchange_host": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t]),
    "b200_comm_allreduce": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int64, C.c_int, C.c_int, C.c_void_p]),
    "b200_comm_allgather": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p]),
    "b200_attention_forward": (C.c_int, [C.c_void_p] + [C.POINTER(AttnOperand)] * 4 + [C.c_void_p, C.c_int64, C.c_int64,
                                         C.c_int64, C.c_int, C.c_float, C.c_int, C.c_void_p]),
    "b200_attention_backward": (C.c_int, [C.c_void_p] + [C.POINTER(AttnOperand)] * 5 + [C.c_void_p] +
                                [C.POINTER(AttnOperand)] * 3 + [C.c_int64, C.c_int64, C.c_int64, C.c_int, C.c_float, C.c_int,
                                                                C.c_void_p]),
    "b200_attention_forward_hp": (C.c_int, [C.c_void_p] + [C.POINTER(AttnOperand)] * 5 + [C.c_void_p, C.c_int64, C.c_int64,
                                            C.c_int64, C.c_int, C.c_float, C.c_int, C.c_void_p]),
    "b200_attention_backward_hp": (C.c_int, [C.c_void_p] + [C.POINTER(AttnOperand)] * 6 + [C.c_void_p] +
                                   [C.POINTER(AttnOperand)] * 3 + [C.c_int64, C.c_int64, C.c_int64, C.c_int, C.c_float, C.c_int,
                                                                   C.c_void_p]),
    "b200_attention_backward_opts": (C.c_int, [C.c_void_p] + [C.POINTER(AttnOperand)] * 6 + [C.c_void_p] +
                                     [C.POINTER(AttnOperand)] * 3 + [C.c_int64, C.c_int64, C.c_int64, C.c_int, C.c_float,
                                                                     C.c_int, C.c_uint, C.c_void_p]),
    "b200_softmax": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p, C.c_int64, C.c_int64, C.c_int64, C.c_float,
                               C.c_int64, C.c_void_p]),
    "b200_softmax_backward": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p, C.c_int64, C.c_void_p, C.c_int64,
                                        C.c_int64, C.c_int64, C.c_float, C.c_void_p]),
    "b200_log_softmax": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p, C.c_int64, C.c_int64, C.c_int64,
                                   C.c_void_p]),
    "b200_log_softmax_backward": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p, C.c_int64, C.c_void_p,
                                            C.c_int64, C.c_int64, C.c_int64, C.c_void_p]),
    "b200_cross_entropy": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p, C.c_int64, C.c_int64, C.c_float,
                                     C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p]),
    "b200_layernorm_forward": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64,
                                         C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_float, C.c_void_p]),
    "b200_layernorm_backward": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p,
                                          C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64,
                                          C.c_void_p]),
    "b200_add_layernorm_forward": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p, C.c_int64, C.c_void_p, C.c_int64,
                                             C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p,
                                             C.c_int64, C.c_int64, C.c_float, C.c_void_p]),
    "b200_layernorm_backward_add": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p, C.c_int64, C.c_void_p,
                                              C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p, C.c_int64,
                                              C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_void_p]),
    "b200_layernorm_backward_full": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p, C.c_int64, C.c_void_p,
                                               C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p, C.c_int64,
                                               C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_void_p]),
    "b200_unary": (C.c_int, [C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.c_int64, C.c_float, C.c_void_p]),
    "b200_binary": (C.c_int, [C.c_void_p, C.c_int, C.c_void_p, C.POINTER(C.c_int64), C.c_void_p, C.POINTER(C.c_int64),
                              C.c_void_p, C.c_void_p]),
    "b200_reduce": (C.c_int, [C.c_void_p, C.c_int, C.c_void_p, C.c_int64, C.c_int64, C.c_int64, C.c_void_p, C.c_void_p]),
    "b200_gelu_backward": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_void_p]),
    "b200_absmax": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p]),
    "b200_quantize_fp8": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int64, C.c_float, C.c_void_p, C.c_void_p]),
    "b200_quantize_fp8_transposed": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_int64, C.c_float, C.c_void_p,
                                               C.c_int64, C.c_void_p]),
    "b200_fill": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int64, C.c_int, C.c_float, C.c_void_p]),
    "b200_cast": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.c_int64, C.c_void_p]),
    "b200_permute": (C.c_int, [C.c_void_p, C.c_void_p, C.POINTER(C.c_int64), C.POINTER(C.c_int32), C.c_void_p, C.c_void_p]),
    "b200_triu": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_int64, C.c_int, C.c_void_p]),
    "b200_embedding_forward": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p, C.c_int64, C.c_int64, C.c_void_p,
                                         C.c_void_p]),
    "b200_embedding_backward": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p, C.c_int64, C.c_int64, C.c_void_p,
                                          C.c_void_p]),
    "b200_sgd_step": (C.c_int, [C.c_void_p, C.c_int64, C.POINTER(C.c_void_p), C.POINTER(C.c_void_p), C.POINTER(C.c_void_p),
                                C.POINTER(C.c_int64), C.c_int, C.c_int, C.c_float, C.c_void_p]),
    "b200_adam_step": (C.c_int, [C.c_void_p, C.c_int64, C.POINTER(C.c_void_p), C.POINTER(C.c_void_p), C.POINTER(C.c_void_p),
                                 C.POINTER(C.c_void_p), C.POINTER(C.c_void_p), C.POINTER(C.c_int64), C.c_int, C.c_int, C.c_float, C.c_float,
                                 C.c_float, C.c_float, C.c_int64, C.c_void_p]),
    "b200_adam_step_device": (C.c_int, [C.c_void_p, C.c_int64, C.POINTER(C.c_void_p), C.POINTER(C.c_void_p), C.POINTER(C.c_void_p),
                                        C.POINTER(C.c_void_p), C.POINTER(C.c_void_p), C.POINTER(C.c_int64), C.c_int, C.c_int,
                                        C.c_float, C.c_float, C.c_float, C.c_float, C.c_void_p, C.c_int, C.c_void_p]),
}

COMM_SUM, COMM_AVG, COMM_MAX = 0, 1, 2
U_NEG, U_RELU, U_GTZ, U_GELU, U_RSQRT, U_EXP, U_LOG, U_TANH, U_SQRT, U_ADD_SCALAR, U_MUL_SCALAR, U_RSUB_SCALAR, U_COPY, \
    U_RECIP, U_SQUARE = range(15)
B_ADD, B_SUB, B_MUL, B_DIV, B_RELU_BW, B_GELU_BW, B_MAX = range(7)
R_SUM, R_MEAN, R_MAX = range(3)

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
    def stream(self) -> int:
        """The context's own cudaStream_t (the stream of every call made with stream=None)."""
        out = C.c_void_p()
        check(lib().b200_ctx_stream(self._h, C.byref(out)))
        return out.value or 0

    @property
    def sm_count(self) -> int:
        n = C.c_int()
        check(lib().b200_ctx_sm_count(self._h, C.byref(n)))
        return n.value

    def synchronize(self, stream=None) -> None:
        check(lib().b200_synchronize(self._h, C.c_void_p(ptr(stream))))

    def timer_start(self, stream=None):
        t = C.c_void_p()
        check(lib().b200_timer_start(self._h, C.c_void_p(ptr(stream)), C.byref(t)))
        return t

    def timer_stop(self, timer, stream=None) -> float:
        ms = C.c_float()
        check(lib().b200_timer_stop(self._h, C.c_void_p(ptr(stream)), timer, C.byref(ms)))
        return ms.value

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

    def memcpy_d2d(self, d_dst, d_src, nbytes: int, stream=None) -> None:
        check(lib().b200_memcpy_d2d(self._h, C.c_void_p(ptr(d_dst)), C.c_void_p(ptr(d_src)), nbytes,
                                    C.c_void_p(ptr(stream))))

    def memset(self, d_dst, value: int, nbytes: int, stream=None) -> None:
        check(lib().b200_memset(self._h, C.c_void_p(ptr(d_dst)), value, nbytes, C.c_void_p(ptr(stream))))

    # ---- matmul -------------------------------------------------------------------------------------
    def gemm_desc(self, A, B, Cout, M, N, K, *, transpose_a=False, transpose_b=False, lda=None, ldb=None, ldc=None,
                  batch=1, stride_a=None, stride_b=None, stride_c=None, c_dtype=BF16, bias=None, bias_dtype=BF16,
                  activation=ACT_NONE, alpha=1.0, causal_mask=False, mask_value=-1e9, fidelity=HIFI4,
                  algo=ALGO_AUTO, split_k=0, ab_dtype=BF16) -> GemmDesc:
        """Descriptor for C = act(mask(alpha * op(A) @ op(B) + bias)); dense row-major defaults for ld/strides.
        ab_dtype=FP8_E4M3: A and B hold one-byte e4m3 values (A [M,K], B [N,K] with transpose_b=True)."""
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
        d.fidelity, d.algo, d.split_k, d.ab_dtype = fidelity, algo, split_k, ab_dtype
        return d

    def gemm(self, desc: GemmDesc, stream=None) -> None:
        check(lib().b200_gemm(self._h, C.byref(desc), C.c_void_p(ptr(stream))))

    def gemm_plan(self, desc: GemmDesc) -> GemmPlan:
        """The plan b200_gemm follows for this product."""
        plan = GemmPlan()
        check(lib().b200_gemm_plan_query(self._h, C.byref(desc), C.byref(plan)))
        return plan

    @staticmethod
    def gemm_plan_text(desc: GemmDesc, plan: GemmPlan) -> str:
        buf = C.create_string_buffer(256)
        check(lib().b200_gemm_plan_describe(C.byref(desc), C.byref(plan), buf, 256))
        return buf.value.decode()

    def gemm_planned(self, desc: GemmDesc, plan: GemmPlan, stream=None) -> None:
        """The product with an explicit plan (kernel, tile width, K slices, tile order) instead of the library's own."""
        check(lib().b200_gemm_planned(self._h, C.byref(desc), C.byref(plan), C.c_void_p(ptr(stream))))

    def selftest_wait_timeout(self, limit_ns: int = 1_000_000, stream=None) -> None:
        """Queues the one-CTA kernel whose bounded wait runs out after `limit_ns`; the next synchronize() reports it."""
        check(lib().b200_selftest_wait_timeout(self._h, limit_ns, C.c_void_p(ptr(stream))))

    def static_scratch_status(self, stream) -> int:
        """Waits for `stream`, then reads and clears the status word of the static-scratch kernels (raises on a time-out)."""
        out = C.c_int()
        check(lib().b200_static_scratch_status(self.device, C.c_void_p(ptr(stream)), C.byref(out)))
        return out.value

    def gemm_static_scratch(self, desc: GemmDesc, stream) -> None:
        """Split-K matmul whose partial sums use the library's fixed 32 MiB array: no device allocation at
        call time (see b200_gemm_static_scratch in the header). `stream` is required."""
        check(lib().b200_gemm_static_scratch(self.device, C.byref(desc), C.c_void_p(ptr(stream))))

    def matmul_host(self, desc: GemmDesc, panels: int = 0) -> None:
        """The product with HOST operand / result pointers in `desc`: pipelined upload, compute and download."""
        check(lib().b200_matmul_host(self._h, C.byref(desc), panels))

    def gemm_scratch_bytes(self, desc: GemmDesc) -> int:
        n = C.c_size_t()
        check(lib().b200_gemm_scratch_bytes(self._h, C.byref(desc), C.byref(n)))
        return n.value

    # ---- row ops, element-wise ops, optimisers: thin pass-throughs (see the header for semantics) ---------------
    def _s(self, stream):
        return C.c_void_p(ptr(stream))

    @staticmethod
    def attn_operand(x, stride_b, stride_h, stride_s, offset=0) -> AttnOperand:
        """Strided bf16 view for the fused attention calls; `offset` in elements from the start of x."""
        return AttnOperand(ptr(x) + 2 * offset, stride_b, stride_h, stride_s)

    def attention_forward(self, q, k, v, o, lse, B, H, S, *, head_dim=64, scale=None, causal=True, o_lo=None, stream=None):
        """q, k, v, o: AttnOperand; lse: fp32 [B, H, S]. o_lo (optional AttnOperand): receives bf16(O - bf16(O)) for
        the backward pass's row term (b200_attention_forward_hp)."""
        scale = head_dim ** -0.5 if scale is None else scale
        check(lib().b200_attention_forward_hp(self._h, C.byref(q), C.byref(k), C.byref(v), C.byref(o),
                                              C.byref(o_lo) if o_lo is not None else None, ptr(lse), B, H, S, head_dim, scale,
                                              int(causal), self._s(stream)))

    def attention_backward(self, q, k, v, o, d_o, lse, d_q, d_k, d_v, B, H, S, *, head_dim=64, scale=None, causal=True,
                           o_lo=None, deterministic=False, stream=None):
        """deterministic=True: dQ summed over the key tiles in key order (B200_ATTN_DETERMINISTIC) instead of by atomics."""
        scale = head_dim ** -0.5 if scale is None else scale
        check(lib().b200_attention_backward_opts(self._h, C.byref(q), C.byref(k), C.byref(v), C.byref(o),
                                                 C.byref(o_lo) if o_lo is not None else None, C.byref(d_o), ptr(lse),
                                                 C.byref(d_q), C.byref(d_k), C.byref(d_v), B, H, S, head_dim, scale,
                                                 int(causal), ATTN_DETERMINISTIC if deterministic else 0, self._s(stream)))

    def softmax(self, x, y, rows, cols, *, ldx=None, ldy=None, alpha=1.0, causal_period=0, stream=None):
        check(lib().b200_softmax(self._h, ptr(x), ldx or cols, ptr(y), ldy or cols, rows, cols, alpha, causal_period,
                                 self._s(stream)))

    def softmax_backward(self, dy, y, dx, rows, cols, *, alpha=1.0, stream=None):
        check(lib().b200_softmax_backward(self._h, ptr(dy), cols, ptr(y), cols, ptr(dx), cols, rows, cols, alpha,
                                          self._s(stream)))

    def log_softmax(self, x, y, rows, cols, *, stream=None):
        check(lib().b200_log_softmax(self._h, ptr(x), cols, ptr(y), cols, rows, cols, self._s(stream)))

    def log_softmax_backward(self, dy, log_y, dx, rows, cols, *, stream=None):
        check(lib().b200_log_softmax_backward(self._h, ptr(dy), cols, ptr(log_y), cols, ptr(dx), cols, rows, cols,
                                              self._s(stream)))

    def cross_entropy(self, logits, labels, rows, classes, *, ld=None, grad_scale=None, loss_sum=None, row_loss=None,
                      d_logits=None, ldd=None, stream=None):
        gs = (1.0 / rows if rows else 1.0) if grad_scale is None else grad_scale
        check(lib().b200_cross_entropy(self._h, ptr(logits), ld or classes, ptr(labels), rows, classes, gs, ptr(loss_sum),
                                       ptr(row_loss), ptr(d_logits), ldd or classes, self._s(stream)))

    def layernorm_forward(self, x, gamma, beta, y, mean, rstd, rows, cols, *, eps=1e-5, stream=None):
        check(lib().b200_layernorm_forward(self._h, ptr(x), cols, ptr(gamma), ptr(beta), ptr(y), cols, ptr(mean), ptr(rstd),
                                           rows, cols, eps, self._s(stream)))

    def layernorm_backward(self, dy, x, gamma, mean, rstd, dx, dgamma, dbeta, rows, cols, *, stream=None):
        check(lib().b200_layernorm_backward(self._h, ptr(dy), cols, ptr(x), cols, ptr(gamma), ptr(mean), ptr(rstd), ptr(dx),
                                            cols, ptr(dgamma), ptr(dbeta), rows, cols, self._s(stream)))

    def add_layernorm_forward(self, x, residual, sum_out, gamma, beta, y, mean, rstd, rows, cols, *, eps=1e-5, stream=None):
        """sum_out = x + residual; y = LayerNorm(sum_out)."""
        check(lib().b200_add_layernorm_forward(self._h, ptr(x), cols, ptr(residual), cols, ptr(sum_out), cols, ptr(gamma),
                                               ptr(beta), ptr(y), cols, ptr(mean), ptr(rstd), rows, cols, eps,
                                               self._s(stream)))

    def layernorm_backward_add(self, dy, x, gamma, mean, rstd, upstream, dx, dgamma, dbeta, rows, cols, *, stream=None):
        """dx = LayerNorm'(dy) + upstream."""
        check(lib().b200_layernorm_backward_add(self._h, ptr(dy), cols, ptr(x), cols, ptr(gamma), ptr(mean), ptr(rstd),
                                                ptr(upstream), cols, ptr(dx), cols, ptr(dgamma), ptr(dbeta), rows, cols,
                                                self._s(stream)))

    def layernorm_backward_full(self, dy, x, gamma, mean, rstd, upstream, dx, dgamma, dbeta, dx_colsum, rows, cols, *,
                                stream=None):
        """dx = LayerNorm'(dy) (+ upstream); dx_colsum (bf16 [cols], optional) = column sums of dx."""
        check(lib().b200_layernorm_backward_full(self._h, ptr(dy), cols, ptr(x), cols, ptr(gamma), ptr(mean), ptr(rstd),
                                                 ptr(upstream), cols, ptr(dx), cols, ptr(dgamma), ptr(dbeta), ptr(dx_colsum),
                                                 rows, cols, self._s(stream)))

    def unary(self, op, x, y, n, *, scalar=0.0, stream=None):
        check(lib().b200_unary(self._h, op, ptr(x), ptr(y), n, scalar, self._s(stream)))

    @staticmethod
    def _shape4(shape):
        shape = tuple(int(d) for d in shape)
        if len(shape) > 4:
            raise ValueError("rank > 4 is not supported")
        return (C.c_int64 * 4)(*((1,) * (4 - len(shape)) + shape))

    def binary(self, op, a, a_shape, b, b_shape, out, *, stream=None):
        check(lib().b200_binary(self._h, op, ptr(a), self._shape4(a_shape), ptr(b), self._shape4(b_shape), ptr(out),
                                self._s(stream)))

    def reduce(self, op, x, outer, R, inner, y, *, stream=None):
        check(lib().b200_reduce(self._h, op, ptr(x), outer, R, inner, ptr(y), self._s(stream)))

    def gelu_backward(self, dy, x_pre, dx, dx_colsum, rows, cols, *, stream=None):
        """dx = dy * GELU'(x_pre) over bf16 [rows, cols]; dx_colsum (bf16 [cols], optional) = column sums of dx."""
        check(lib().b200_gelu_backward(self._h, ptr(dy), ptr(x_pre), ptr(dx), ptr(dx_colsum), rows, cols, self._s(stream)))

    def absmax(self, x, n, out_f32, *, stream=None):
        """out_f32[0] = max |x| over n bf16 elements."""
        check(lib().b200_absmax(self._h, ptr(x), n, ptr(out_f32), self._s(stream)))

    def quantize_fp8(self, x, n, scale, y, *, stream=None):
        """y[i] = e4m3(x[i] * scale), saturating; y holds n bytes."""
        check(lib().b200_quantize_fp8(self._h, ptr(x), n, scale, ptr(y), self._s(stream)))

    def quantize_fp8_transposed(self, x, rows, cols, scale, y, *, ldx=None, ldy=None, stream=None):
        """y[c, r] = e4m3(x[r, c] * scale) for a [rows, cols] bf16 matrix; y is [cols, rows] bytes."""
        check(lib().b200_quantize_fp8_transposed(self._h, ptr(x), rows, cols, cols if ldx is None else ldx, scale, ptr(y),
                                                 rows if ldy is None else ldy, self._s(stream)))

    def fill(self, dst, n, dtype, value, *, stream=None):
        check(lib().b200_fill(self._h, ptr(dst), n, dtype, value, self._s(stream)))

    def cast(self, src, src_dtype, dst, dst_dtype, n, *, stream=None):
        check(lib().b200_cast(self._h, ptr(src), src_dtype, ptr(dst), dst_dtype, n, self._s(stream)))

    def permute(self, x, in_shape, perm, y, *, stream=None):
        check(lib().b200_permute(self._h, ptr(x), self._shape4(in_shape), (C.c_int32 * 4)(*perm), ptr(y), self._s(stream)))

    def triu(self, x, y, batch, rows, cols, diagonal, *, stream=None):
        check(lib().b200_triu(self._h, ptr(x), ptr(y), batch, rows, cols, diagonal, self._s(stream)))

    def embedding_forward(self, ids, n_ids, table, vocab, dim, out, *, stream=None):
        check(lib().b200_embedding_forward(self._h, ptr(ids), n_ids, ptr(table), vocab, dim, ptr(out), self._s(stream)))

    def embedding_backward(self, ids, n_ids, dy, vocab, dim, d_table_f32, *, stream=None):
        check(lib().b200_embedding_backward(self._h, ptr(ids), n_ids, ptr(dy), vocab, dim, ptr(d_table_f32),
                                            self._s(stream)))

    @staticmethod
    def _ptr_array(items):
        return (C.c_void_p * len(items))(*[ptr(i) or None for i in items])

    def sgd_step(self, params, grads, sizes, lr, *, p_dtype=BF16, g_dtype=BF16, shadows=None, stream=None):
        n = len(params)
        check(lib().b200_sgd_step(self._h, n, self._ptr_array(params), self._ptr_array(grads),
                                  self._ptr_array(shadows) if shadows else None, (C.c_int64 * n)(*sizes),
                                  p_dtype, g_dtype, lr, self._s(stream)))

    def adam_step(self, params, grads, m, v, sizes, step, *, lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8, p_dtype=BF16,
                  g_dtype=BF16, shadows=None, stream=None):
        n = len(params)
        check(lib().b200_adam_step(self._h, n, self._ptr_array(params), self._ptr_array(grads), self._ptr_array(m),
                                   self._ptr_array(v), self._ptr_array(shadows) if shadows else None,
                                   (C.c_int64 * n)(*sizes), p_dtype, g_dtype, lr, beta1, beta2, eps, step,
                                   self._s(stream)))

    def adam_step_device(self, params, grads, m, v, sizes, state, *, advance=True, lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8,
                         p_dtype=BF16, g_dtype=BF16, shadows=None, stream=None):
        """Adam with the step number in the 16-byte device buffer `state` (zero-filled once by the caller): a step
        recorded into a trace advances on every replay."""
        n = len(params)
        check(lib().b200_adam_step_device(self._h, n, self._ptr_array(params), self._ptr_array(grads), self._ptr_array(m),
                                          self._ptr_array(v), self._ptr_array(shadows) if shadows else None,
                                          (C.c_int64 * n)(*sizes), p_dtype, g_dtype, lr, beta1, beta2, eps, ptr(state),
                                          int(bool(advance)), self._s(stream)))

    # ---- sharded matmul --------------------------------------------------------------------------------------------
    def ipc_get_handle(self, dptr) -> bytes:
        buf = C.create_string_buffer(64)
        check(lib().b200_ipc_get_handle(self._h, ptr(dptr), buf))
        return buf.raw

    def ipc_open_handle(self, handle: bytes) -> int:
        out = C.c_void_p()
        check(lib().b200_ipc_open_handle(self._h, C.create_string_buffer(handle, 64), C.byref(out)))
        return out.value or 0

    def ipc_close_handle(self, dptr) -> None:
        check(lib().b200_ipc_close_handle(self._h, ptr(dptr)))

    def gemm_allgather(self, desc: GemmDesc, peer_c, my_rank: int, stream=None) -> None:
        check(lib().b200_gemm_allgather(self._h, C.byref(desc), self._ptr_array(peer_c), len(peer_c), my_rank,
                                        self._s(stream)))

    def peer_barrier(self, peer_flags, my_rank: int, local_epoch, stream=None) -> None:
        """A barrier between one-process-per-GPU ranks as one small kernel on the stream (see b200_peer_barrier)."""
        check(lib().b200_peer_barrier(self._h, self._ptr_array(peer_flags), len(peer_flags), my_rank, C.c_void_p(ptr(local_epoch)),
                                      self._s(stream)))

    def gemm_allgather_mc(self, desc: GemmDesc, mc_c, n_ranks: int, my_rank: int, *, use_multimem=True, stream=None) -> None:
        """The fused all-gather with one multicast destination (see b200_gemm_allgather_mc)."""
        check(lib().b200_gemm_allgather_mc(self._h, C.byref(desc), C.c_void_p(ptr(mc_c)), n_ranks, my_rank,
                                           int(bool(use_multimem)), self._s(stream)))

    def mc_broadcast(self, mc_dst, d_src, nbytes: int, stream=None) -> None:
        """This GPU's block -> the same offset of every rank's copy (one multimem.st per 16 bytes)."""
        check(lib().b200_mc_broadcast(self._h, C.c_void_p(ptr(mc_dst)), C.c_void_p(ptr(d_src)), nbytes, self._s(stream)))

    def mc_supported(self) -> bool:
        out = C.c_int()
        check(lib().b200_mc_supported(self._h, C.byref(out)))
        return bool(out.value)

    def gemm_reduce_scatter_partials(self, desc: GemmDesc, peer_slots, my_rank: int, stream=None) -> None:
        check(lib().b200_gemm_reduce_scatter_partials(self._h, C.byref(desc), self._ptr_array(peer_slots), len(peer_slots),
                                                      my_rank, self._s(stream)))

    def gemm_dist_plan(self, desc: GemmDesc, n_ranks: int, reduce_scatter: bool = False) -> GemmPlan:
        """Kernel and tile width the fused all-gather (or reduce-scatter) product uses for `desc`."""
        plan = GemmPlan()
        check(lib().b200_gemm_dist_plan_query(self._h, C.byref(desc), n_ranks, int(reduce_scatter), C.byref(plan)))
        return plan

    def reduce_slices(self, slices, n_slices: int, desc: GemmDesc, stream=None, slices_dtype=F32) -> None:
        check(lib().b200_reduce_slices_typed(self._h, ptr(slices), slices_dtype, n_slices, C.byref(desc), self._s(stream)))

    # ---- pool and traces ---------------------------------------------------------------------------------------------
    def pool_alloc(self, nbytes: int) -> int:
        out = C.c_void_p()
        check(lib().b200_pool_alloc(self._h, nbytes, C.byref(out)))
        return out.value or 0

    def pool_free(self, dptr) -> None:
        check(lib().b200_pool_free(self._h, ptr(dptr)))

    def pool_stats(self) -> tuple[int, int]:
        r, u = C.c_size_t(), C.c_size_t()
        check(lib().b200_pool_stats(self._h, C.byref(r), C.byref(u)))
        return r.value, u.value

    def trace_begin(self) -> int:
        tid = C.c_uint32()
        check(lib().b200_trace_begin(self._h, C.byref(tid)))
        return tid.value

    def trace_end(self, tid: int) -> None:
        check(lib().b200_trace_end(self._h, tid))

    def trace_execute(self, tid: int, blocking: bool = False) -> None:
        check(lib().b200_trace_execute(self._h, tid, int(blocking)))

    def trace_execute_on(self, tid: int, stream) -> None:
        """Replays the trace on the caller's stream (a cudaStream_t handle)."""
        check(lib().b200_trace_execute_on(self._h, tid, C.c_void_p(ptr(stream))))

    def trace_release(self, tid: int) -> None:
        check(lib().b200_trace_release(self._h, tid))


def comm_unique_id() -> bytes:
    """A fresh 128-byte communicator id (made on one rank; the host program ships it to the others)."""
    buf = C.create_string_buffer(128)
    check(lib().b200_comm_unique_id(buf))
    return buf.raw


class Comm:
    """One rank's communicator (NCCL behind the C ABI): stream-ordered barrier, exchange of small host blobs, all-reduce
    and all-gather of device buffers. `Comm(ctx, id, world, rank)` is collective over the ranks."""

    def __init__(self, ctx: Context, unique_id: bytes, world: int, rank: int):
        if len(unique_id) != 128:
            raise ValueError("the communicator id is 128 bytes")
        self.ctx, self.world, self.rank = ctx, int(world), int(rank)
        self._h = C.c_void_p()
        check(lib().b200_comm_create(ctx.handle, C.create_string_buffer(unique_id, 128), self.world, self.rank,
                                     C.byref(self._h)))

    def close(self) -> None:
        if getattr(self, "_h", None) is not None and self._h:
            lib().b200_comm_destroy(self._h)
            self._h = C.c_void_p()

    def barrier(self, stream=None) -> None:
        check(lib().b200_comm_barrier(self._h, C.c_void_p(ptr(stream))))

    def exchange(self, blob: bytes) -> list[bytes]:
        """All ranks' `blob` (same length everywhere) in rank order."""
        n = len(blob)
        recv = C.create_string_buffer(n * self.world)
        check(lib().b200_comm_exchange_host(self._h, C.create_string_buffer(blob, n), recv, n))
        return [recv.raw[i * n:(i + 1) * n] for i in range(self.world)]

    def allreduce(self, buf, count: int, dtype: int = F32, op: int = COMM_SUM, stream=None) -> None:
        check(lib().b200_comm_allreduce(self._h, C.c_void_p(ptr(buf)), count, dtype, op, C.c_void_p(ptr(stream))))

    def allgather(self, send, recv, bytes_per_rank: int, stream=None) -> None:
        check(lib().b200_comm_allgather(self._h, C.c_void_p(ptr(send)), C.c_void_p(ptr(recv)), bytes_per_rank,
                                        C.c_void_p(ptr(stream))))


class MulticastBuffer:
    """A device buffer per rank, all bound to one NVLink multicast object (collective over `comm`): `local` is this
    rank's copy, `multicast` the address at which one store reaches every rank's copy. close() is collective too and
    must run on every rank before any of them exits."""

    def __init__(self, comm: Comm, nbytes: int):
        self.comm, self.nbytes = comm, nbytes
        self._h, loc, mc = C.c_void_p(), C.c_void_p(), C.c_void_p()
        check(lib().b200_mc_alloc(comm._h, nbytes, C.byref(self._h), C.byref(loc), C.byref(mc)))
        self.local, self.multicast = loc.value or 0, mc.value or 0

    def close(self) -> None:
        if getattr(self, "_h", None) is not None and self._h:
            check(lib().b200_mc_free(self._h))
            self._h = C.c_void_p()
            self.local = self.multicast = 0
