"""Router GEMMs in front of the routing kernels: fp32 logits from the hidden states.

Mirrors ``router_gemm`` (src/flaggems_vllm/ops/router_gemm.py:207-237) and
``fp32_router_gemm`` / ``supports_fp32_router_gemm``
(src/flaggems_vllm/ops/fp32_router_gemm.py:17-145): same names, argument meaning
and error behaviour.  Both kernels of ``csrc/router_gemm.cu`` are deterministic: a
row-streaming fp32 kernel for decode-sized batches (and for every dtype pair), a
tensor-core (warp MMA, fp32 accumulate) kernel for half-precision batches above 320 rows.
No library GEMM is called.  ``router_gemm_grouped_topk`` fuses the GEMM with the
group-limited routing for decode batches (no counterpart in the reference, which runs the
two ops back to back).
"""

from __future__ import annotations

import logging

import torch

from . import _lib

logger = logging.getLogger(__name__)

# up to this many rows the fused GEMM + routing kernel (one CTA per token) beats two launches
FUSED_MAX_ROWS = 64


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
    if x.shape[1] % 8 != 0:
        raise ValueError("router_gemm: the hidden size must be a multiple of 8")
    return _launch(x, weight)


def router_gemm_grouped_topk(x: torch.Tensor, weight: torch.Tensor, n_group: int, topk_group: int, topk: int,
                             renormalize: bool, routed_scaling_factor: float, bias: torch.Tensor,
                             scoring_func: int = 0, return_logits: bool = False):
    """``grouped_topk(router_gemm(x, weight), ...)`` in one launch: hidden states [M, K] and router
    weight [E, K] in, (topk_weights fp32 [M, topk], topk_ids int32 [M, topk]) out; the logits stay on
    chip (``return_logits=True`` also returns a copy).  Results equal the two separate calls bit for
    bit.  Meant for decode batches (one CTA per token); any M is accepted."""
    logger.debug("GEMS ROUTER GEMM + GROUPED TOPK")
    if x.ndim != 2 or weight.ndim != 2 or x.shape[1] != weight.shape[1]:
        raise ValueError("router_gemm_grouped_topk expects x [M, K] and weight [E, K]")
    if scoring_func not in (0, 1):
        raise ValueError(f"Unsupported scoring_func: {scoring_func}")
    _lib.require_cuda(x, "router_gemm_grouped_topk")
    M, K = x.shape
    E = weight.shape[0]
    if bias.numel() != E:
        raise ValueError(f"bias length {bias.numel()} does not match the expert count {E}")
    xc = x if x.stride(1) == 1 and x.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0 else x.contiguous()
    wc = weight if weight.is_contiguous() else weight.contiguous()
    b = bias.to(torch.float32).contiguous()
    tw = torch.empty((M, topk), dtype=torch.float32, device=x.device)
    ti = torch.empty((M, topk), dtype=torch.int32, device=x.device)
    logits = torch.empty((M, E), dtype=torch.float32, device=x.device) if return_logits else None
    _lib.check(_lib.lib().moe_router_gemm_grouped_topk(
        xc.data_ptr(), _lib.dtype_code(xc.dtype), xc.stride(0), wc.data_ptr(), _lib.dtype_code(wc.dtype), b.data_ptr(),
        M, E, K, n_group, topk_group, topk, int(bool(renormalize)), float(routed_scaling_factor), scoring_func,
        tw.data_ptr(), ti.data_ptr(), _lib.ptr(logits), _lib.stream_of(x)))
    return (tw, ti, logits) if return_logits else (tw, ti)


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
