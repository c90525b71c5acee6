"""Router GEMMs in front of the routing kernels: fp32 logits from the hidden states.

Mirrors ``router_gemm`` (src/flaggems_vllm/ops/router_gemm.py:207-237) and
``fp32_router_gemm`` / ``supports_fp32_router_gemm``
(src/flaggems_vllm/ops/fp32_router_gemm.py:17-145): same names, argument meaning
and error behaviour.  Decode-sized batches run the deterministic CUDA kernel of
``csrc/router_gemm.cu``; a large prefill batch of ``router_gemm`` is a plain
library GEMM (cuBLAS through ``torch.mm``) with fp32 output.
"""

from __future__ import annotations

import logging

import torch

from . import _lib

logger = logging.getLogger(__name__)

# above this many rows the plain [M, K] x [K, N] product is left to cuBLAS
KERNEL_MAX_ROWS = 256


def _launch(x: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    M, K = x.shape
    N = weight.shape[0]
    out = torch.empty((M, N), device=x.device, dtype=torch.float32)
    if M == 0:
        return out
    xc = x if x.stride(1) == 1 and x.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0 else x.contiguous()
    wc = weight if weight.is_contiguous() else weight.contiguous()
    _lib.check(_lib.lib().moe_router_gemm(xc.data_ptr(), _lib.dtype_code(xc.dtype), xc.stride(0), wc.data_ptr(),
                                          _lib.dtype_code(wc.dtype), M, N, K, out.data_ptr(), _lib.stream_of(x)))
    return out


def router_gemm(x: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    """bf16 x bf16 -> fp32 GEMM for the MoE router gate: ``x`` [M, K], ``weight`` [N, K]."""
    logger.debug("GEMS ROUTER GEMM")
    if x.ndim != 2 or weight.ndim != 2:
        raise ValueError("router_gemm expects 2D x and weight tensors")
    if x.shape[1] != weight.shape[1]:
        raise ValueError("router_gemm expects x.shape[1] == weight.shape[1]")
    if x.device != weight.device:
        raise ValueError("router_gemm expects x and weight to be on the same device")
    _lib.require_cuda(x, "router_gemm")
    M, K = x.shape
    if M <= KERNEL_MAX_ROWS and K % 8 == 0:
        return _launch(x, weight)
    # plain library GEMM with fp32 accumulation and output
    try:
        return torch.mm(x, weight.t(), out_dtype=torch.float32)
    except TypeError:
        return torch.mm(x.float(), weight.float().t())


def supports_fp32_router_gemm(hidden_size, num_experts, input_dtype, weight_dtype):
    """Metadata predicate for the model dimensions the reference validates."""
    return (
        (hidden_size, num_experts) == (6144, 128)
        and input_dtype in (torch.bfloat16, torch.float32)
        and weight_dtype == torch.float32
    )


def fp32_router_gemm(input: torch.Tensor, router_weight: torch.Tensor) -> torch.Tensor:
    """Fresh fp32 [M, 128] logits for ``input`` [M, 6144] (bf16/fp32) and fp32 ``router_weight``
    [128, 6144]; M <= 32.  Other sizes raise ``NotImplementedError`` like the reference."""
    logger.debug("GEMS FP32 ROUTER GEMM")
    if input.ndim != 2 or router_weight.ndim != 2:
        raise ValueError("FP32 router GEMM requires 2D input and router_weight")
    if input.device.type != "cuda" or router_weight.device != input.device:
        raise ValueError("FP32 router input and weight must share a CUDA device")
    if input.shape[1] != router_weight.shape[1]:
        raise ValueError("FP32 router input and weight hidden dimensions must match")
    if not supports_fp32_router_gemm(input.shape[1], router_weight.shape[0], input.dtype, router_weight.dtype):
        raise NotImplementedError(
            "FP32 router GEMM supports MiniMax-M3 [M,6144] input in BF16/FP32 and [128,6144] FP32 weight")
    if input.shape[0] > 32:
        raise NotImplementedError("FP32 router specialization supports M<=32")
    return _launch(input, router_weight)
