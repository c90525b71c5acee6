"""silu_and_mul and silu_and_mul_out: the stand-alone gated activation.

Signatures follow src/flaggems_vllm/ops/silu_and_mul.py:63-70 (forward kernel
:26-31, gradients :39-46).  The fused-MoE layer of this package never calls
them (its GEMM1 applies the activation in its epilogue); they exist for callers
that used the reference's op directly."""

from __future__ import annotations

import logging

import torch

from . import _lib

logger = logging.getLogger(__name__)


def _prepare(A: torch.Tensor, B: torch.Tensor, what: str):
    _lib.require_cuda(A, what)
    if A.device != B.device:
        raise ValueError(f"{what}: operands on different devices")
    dtype = torch.promote_types(A.dtype, B.dtype)
    if dtype not in (torch.float32, torch.float16, torch.bfloat16):
        raise ValueError(f"Unsupported dtype: {dtype}")
    shape = torch.broadcast_shapes(A.shape, B.shape)
    a = A.to(dtype).expand(shape).contiguous()
    b = B.to(dtype).expand(shape).contiguous()
    return a, b, dtype, shape


def _forward(a, b, out):
    _lib.check(_lib.lib().moe_silu_and_mul(a.data_ptr(), b.data_ptr(), out.data_ptr(), _lib.dtype_code(out.dtype),
                                           out.numel(), _lib.stream_of(out)))
    return out


class _SiluAndMul(torch.autograd.Function):
    @staticmethod
    def forward(ctx, A, B):
        a, b, dtype, shape = _prepare(A, B, "silu_and_mul")
        ctx.save_for_backward(a, b)
        ctx.shapes = (A.shape, B.shape, A.dtype, B.dtype)
        return _forward(a, b, torch.empty(shape, dtype=dtype, device=a.device))

    @staticmethod
    def backward(ctx, grad_output):
        a, b = ctx.saved_tensors
        shape_a, shape_b, dtype_a, dtype_b = ctx.shapes
        g = grad_output.to(a.dtype).contiguous()
        da, db = torch.empty_like(a), torch.empty_like(b)
        _lib.check(_lib.lib().moe_silu_and_mul_grad(a.data_ptr(), b.data_ptr(), g.data_ptr(), da.data_ptr(),
                                                    db.data_ptr(), _lib.dtype_code(a.dtype), a.numel(),
                                                    _lib.stream_of(a)))
        # operands that were broadcast or widened get the gradient of their own shape and dtype
        return da.sum_to_size(shape_a).to(dtype_a), db.sum_to_size(shape_b).to(dtype_b)


def silu_and_mul(A: torch.Tensor, B: torch.Tensor) -> torch.Tensor:
    """SiLU(A) * B, computed in fp32 and rounded once to the promoted dtype; differentiable."""
    logger.debug("GEMS SILU AND MUL FORWARD")
    return _SiluAndMul.apply(A, B)


def silu_and_mul_out(A: torch.Tensor, B: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """SiLU(A) * B written into ``out`` (returned)."""
    logger.debug("GEMS SILU AND MUL OUT")
    a, b, dtype, shape = _prepare(A, B, "silu_and_mul_out")
    if tuple(out.shape) != tuple(shape):
        raise ValueError(f"silu_and_mul_out: out has shape {tuple(out.shape)}, expected {tuple(shape)}")
    if out.dtype == dtype and out.is_contiguous():
        return _forward(a, b, out)
    tmp = _forward(a, b, torch.empty(shape, dtype=dtype, device=a.device))
    out.copy_(tmp)
    return out
