"""Host-side mirror of the reference's `__co__` call signatures over torch tensors.

Each function takes device tensors in the reference's argument order
(lhs[M,K], rhs[N,K], output[M,N], schedule_m, schedule_n, scale tensors ...),
wraps them as spanned views and calls the C ABI of ``libcroq_b200``. Outputs are
caller-allocated, as for the reference's `void` `__co__` functions
(Documents/Documentation/io-and-linking.md:19-47); when ``output`` is omitted
one is allocated with torch. Calls are asynchronous on the current torch
stream; ``synchronize()`` blocks and surfaces device-side status.
"""
from __future__ import annotations

import ctypes

import torch

from . import _lib
from ._lib import CROQ_DTYPE_BF16, CROQ_DTYPE_F16, View1, View2, View3


def _stream() -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _need_cuda(*tensors: torch.Tensor) -> None:
    for t in tensors:
        if t is None:
            continue
        if not t.is_cuda:
            raise ValueError("libcroq_b200 takes device tensors only (no CPU path)")
        if not t.is_contiguous():
            raise ValueError("views are dense row-major: pass contiguous tensors")


def _v1(t: torch.Tensor | None):
    if t is None:
        return None
    return ctypes.byref(View1(t.data_ptr(), (ctypes.c_size_t * 1)(t.shape[0])))


def _v2(t: torch.Tensor):
    return ctypes.byref(View2(t.data_ptr(), (ctypes.c_size_t * 2)(t.shape[0], t.shape[1])))


def _v3(t: torch.Tensor):
    return ctypes.byref(View3(t.data_ptr(), (ctypes.c_size_t * 3)(*t.shape)))


def _out_dtype_flag(t: torch.Tensor) -> int:
    if t.dtype == torch.bfloat16:
        return CROQ_DTYPE_BF16
    if t.dtype == torch.float16:
        return CROQ_DTYPE_F16
    raise ValueError(f"output dtype must be float16 or bfloat16, got {t.dtype}")


def synchronize() -> None:
    """Blocks on the current stream; raises if a kernel reported a fault
    (wait budget exhausted, schedule or index out of range)."""
    lib = _lib.load()
    _lib.check(lib.croq_synchronize(_stream()), "croq_synchronize")


def last_kernel_clock() -> tuple[float, float]:
    """(SM MHz, duration in us) the last GEMM kernel measured on itself; call
    after ``synchronize()``."""
    lib = _lib.load()
    mhz, us = ctypes.c_double(), ctypes.c_double()
    _lib.check(lib.croq_last_kernel_clock(ctypes.byref(mhz), ctypes.byref(us)), "croq_last_kernel_clock")
    return mhz.value, us.value


def matmul(lhs: torch.Tensor, rhs: torch.Tensor, output: torch.Tensor | None = None,
           schedule_m: torch.Tensor | None = None, schedule_n: torch.Tensor | None = None,
           sched_tile_m: int = 256, sched_tile_n: int = 256) -> torch.Tensor:
    """output[M,N] = lhs[M,K] @ rhs[N,K]^T in f16 or bf16 with fp32 accumulation,
    visiting schedule tiles in the given order (see ``croq_matmul_f16``)."""
    lib = _lib.load()
    if output is None:
        output = torch.empty((lhs.shape[0], rhs.shape[0]), dtype=lhs.dtype, device=lhs.device)
    _need_cuda(lhs, rhs, output, schedule_m, schedule_n)
    if lhs.dtype != rhs.dtype or lhs.dtype != output.dtype:
        raise ValueError("lhs, rhs and output must share one 16-bit dtype")
    for s in (schedule_m, schedule_n):
        if s is not None and s.dtype != torch.int32:
            raise ValueError("schedules are s32 arrays")
    fn = {torch.float16: lib.croq_matmul_f16, torch.bfloat16: lib.croq_matmul_bf16}.get(lhs.dtype)
    if fn is None:
        raise ValueError(f"matmul supports float16 and bfloat16, got {lhs.dtype}")
    rc = fn(_v2(lhs), _v2(rhs), _v2(output), _v1(schedule_m), _v1(schedule_n),
            int(sched_tile_m), int(sched_tile_n), _stream())
    _lib.check(rc, fn.__name__)
    return output


def blockscale_gemm_e4m3(lhs: torch.Tensor, scale_lhs: torch.Tensor, rhs: torch.Tensor,
                         scale_rhs: torch.Tensor, output: torch.Tensor | None = None,
                         out_dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """FP8 e4m3 GEMM with fp32 scales per 1x128 (lhs) and 128x128 (rhs) block;
    argument order of the reference's ``blockscale_gemm_e4m3_ws_persis``."""
    lib = _lib.load()
    if output is None:
        output = torch.empty((lhs.shape[0], rhs.shape[0]), dtype=out_dtype, device=lhs.device)
    _need_cuda(lhs, scale_lhs, rhs, scale_rhs, output)
    if lhs.dtype != torch.float8_e4m3fn or rhs.dtype != torch.float8_e4m3fn:
        raise ValueError("lhs and rhs must be float8_e4m3fn")
    if scale_lhs.dtype != torch.float32 or scale_rhs.dtype != torch.float32:
        raise ValueError("scales are f32")
    rc = lib.croq_blockscale_gemm_e4m3(_v2(lhs), _v2(scale_lhs), _v2(rhs), _v2(scale_rhs),
                                       _v2(output), _out_dtype_flag(output), _stream())
    _lib.check(rc, "croq_blockscale_gemm_e4m3")
    return output
