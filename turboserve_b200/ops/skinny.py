"""Python face of ``gemm_skinny.cu``: the weight-streaming product for at most 64 rows."""

from __future__ import annotations

from ctypes import c_int, c_longlong, c_void_p

import torch

from . import kernels
from .kernels import KernelError, _check, _fn, _need, _ptr, _stream

_num_sms: dict[int, int] = {}


def num_sms(device: torch.device) -> int:
    index = device.index if device.index is not None else torch.cuda.current_device()
    if index not in _num_sms:
        _num_sms[index] = torch.cuda.get_device_properties(index).multi_processor_count
    return _num_sms[index]


def gemm_skinny(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, bias: torch.Tensor | None = None,
                m: int | None = None, ksplit: int = 0, early_trigger: bool = True) -> None:
    """``out[:m] = a[:m] @ w.T (+ bias)``; bfloat16 inputs, bfloat16 or float32 output, m <= 64."""
    _need(a, torch.bfloat16, "a"); _need(w, torch.bfloat16, "w"); _need(out, None, "out")
    if a.dim() != 2 or w.dim() != 2 or out.dim() != 2 or a.shape[1] != w.shape[1] or out.shape[1] != w.shape[0]:
        raise KernelError(f"gemm_skinny: shapes do not agree: a {tuple(a.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
    rows = a.shape[0] if m is None else m
    if a.shape[0] < rows or out.shape[0] < rows:
        raise KernelError("gemm_skinny: fewer rows than asked for")
    if bias is not None:
        _need(bias, torch.float32, "bias")
        if bias.numel() != w.shape[0]:
            raise KernelError("gemm_skinny: bias length does not match the output width")
    fn = _fn("gemm_skinny", "ts_gemm_skinny",
             [c_int, c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_void_p, c_longlong, c_int, c_int, c_int,
              c_int, c_int, c_int, c_void_p])
    _check(fn(kernels.dtype_code(out.dtype), _ptr(a), a.stride(0), _ptr(w), w.stride(0), _ptr(bias), _ptr(out),
              out.stride(0), rows, w.shape[0], a.shape[1], ksplit, num_sms(a.device), int(early_trigger), _stream()), "gemm_skinny")
