"""Stand-alone sm_100a element-wise kernels (``kernels/elementwise.cu``).

All run on the current PyTorch stream and raise if the native library or a GPU
is missing - there is no PyTorch fallback.
"""
from __future__ import annotations

import ctypes as C

import torch

from .. import _lib
from .._lib import DTYPES, check


def _stream() -> C.c_void_p:
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _code(t: torch.Tensor) -> int:
    return DTYPES[str(t.dtype).replace("torch.", "")]


def scale_cast(src: torch.Tensor, out: torch.Tensor, scale: float = 1.0) -> torch.Tensor:
    """out = (out.dtype)(src * scale); gradient scaling and bf16<->fp32 casts in one pass."""
    assert src.is_cuda and out.is_cuda and src.is_contiguous() and out.is_contiguous() and src.numel() == out.numel()
    check(_lib.load().al_scale_cast(C.c_void_p(out.data_ptr()), _code(out), C.c_void_p(src.data_ptr()), _code(src),
                                    src.numel(), float(scale), _stream()))
    return out


def sgd_momentum_step(param: torch.Tensor, momentum: torch.Tensor, grad: torch.Tensor, lr: float, mu: float = 0.9,
                      weight_decay: float = 0.0, grad_scale: float = 1.0, first_step: bool = False,
                      zero_grad: bool = False) -> None:
    """One fused momentum-SGD update over flat fp32 buffers (one launch for a whole model)."""
    for t in (param, momentum, grad):
        assert t.is_cuda and t.is_contiguous() and t.dtype == torch.float32
    assert param.numel() == momentum.numel() == grad.numel()
    check(_lib.load().al_sgd_momentum(C.c_void_p(param.data_ptr()), C.c_void_p(momentum.data_ptr()),
                                      C.c_void_p(grad.data_ptr()), param.numel(), lr, mu, weight_decay, grad_scale,
                                      1 if first_step else 0, 1 if zero_grad else 0, _stream()))


def fill_u32(out: torch.Tensor, value: int = 0) -> None:
    """Fill a 4-byte-element tensor with a bit pattern (benchmarks use it to flush L2)."""
    assert out.is_cuda and out.is_contiguous() and out.element_size() == 4
    check(_lib.load().al_fill_u32(C.c_void_p(out.data_ptr()), out.numel(), value & 0xFFFFFFFF, _stream()))
