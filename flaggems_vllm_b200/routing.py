"""grouped_topk: host side of the warp-per-token routing kernel.

Signature, argument checks and error types mirror the reference function
(src/flaggems_vllm/ops/grouped_topk.py:1674-1739)."""

from __future__ import annotations

import logging
from typing import Optional

import torch

from . import _lib

logger = logging.getLogger(__name__)


def _validate_padding(scores, bias, is_padding, n_group, topk_group, topk):
    # mirrors src/flaggems_vllm/ops/grouped_topk.py:1638-1671
    rows, experts = scores.shape
    if (
        is_padding.dtype != torch.bool
        or is_padding.shape != (rows,)
        or is_padding.device != scores.device
        or not is_padding.is_contiguous()
    ):
        raise ValueError("is_padding must be contiguous bool [num_tokens] on the scores device")
    if (
        bias.shape != (experts,)
        or bias.device != scores.device
        or not bias.is_contiguous()
        or scores.stride(1) != 1
        or scores.stride(0) < experts
    ):
        raise ValueError("masked grouped_topk needs row-major scores and contiguous same-device bias")
    if not 1 <= topk_group <= n_group <= 32 or not 1 <= topk <= 32:
        raise ValueError("expected valid group counts and topk in [1, 32]")
    if experts // n_group < 2 or experts > 4096 or topk > (experts // n_group) * topk_group:
        raise ValueError(
            "masked grouped_topk needs at least 2 experts per group, at most 4096 "
            "experts, and at least topk candidates after group selection"
        )


def grouped_topk(
    scores: torch.Tensor,
    n_group: int,
    topk_group: int,
    topk: int,
    renormalize: bool,
    routed_scaling_factor: float,
    bias: torch.Tensor,
    scoring_func: int = 0,
    is_padding: Optional[torch.Tensor] = None,
):
    """Route scores; optional padding rows emit zero weights and -1 ids.

    Returns (topk_weights fp32 [M, topk], topk_ids int32 [M, topk])."""
    logger.debug("GEMS GROUPED TOPK")
    if scores.ndim != 2:
        raise ValueError("scores must be a 2D Tensor")
    num_tokens, num_experts = scores.shape
    if is_padding is not None:
        _validate_padding(scores, bias, is_padding, n_group, topk_group, topk)
    if num_experts % n_group != 0:
        raise ValueError("num_experts must be divisible by n_group")
    if n_group > 32:
        raise ValueError("n_group should be smaller than or equal to 32")
    if topk > 32:
        raise ValueError("topk should be smaller than or equal to 32 for now")
    if scoring_func not in (0, 1):
        raise ValueError("scoring_func must be 0 (none) or 1 (sigmoid)")
    if bias.ndim != 1:
        bias = bias.flatten()
    if len(bias) != num_experts:
        raise ValueError(f"bias length ({len(bias)}) must match num_experts ({num_experts})")
    sdt = _lib.dtype_code(scores.dtype)  # ValueError("Unsupported dtype") like the reference
    if bias.dtype not in (torch.float32, torch.float16, torch.bfloat16):
        bias = bias.float()
    if not bias.is_contiguous():
        bias = bias.contiguous()
    if bias.device != scores.device:
        raise ValueError("bias must be on the scores device")

    _lib.require_cuda(scores, "grouped_topk")
    weights = torch.empty((num_tokens, topk), device=scores.device, dtype=torch.float32)
    ids = torch.empty((num_tokens, topk), device=scores.device, dtype=torch.int32)
    if num_tokens == 0:
        return weights, ids
    pad = is_padding.view(torch.uint8) if is_padding is not None else None
    rc = _lib.lib().moe_grouped_topk(
        scores.data_ptr(), sdt, scores.stride(0), scores.stride(1), bias.data_ptr(),
        _lib.dtype_code(bias.dtype), _lib.ptr(pad), num_tokens, num_experts, n_group, topk_group, topk,
        int(bool(renormalize)), float(routed_scaling_factor), int(scoring_func), weights.data_ptr(),
        ids.data_ptr(), _lib.stream_of(scores))
    _lib.check(rc)
    return weights, ids
